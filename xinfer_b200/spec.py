"""Host-side handle of the speculative decode runtime (xinfer_spec_decoder_* in the C-ABI)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import ModelConfig, check, lib


@dataclass
class Shape:
    """Shape fields of the reference's ModelConfig (src/targets/qwen3_8_27b/weights.h:58-107)."""
    hidden_size: int = 5120
    intermediate_size: int = 17408
    num_hidden_layers: int = 64
    num_attention_heads: int = 24
    num_key_value_heads: int = 4
    vocab_size: int = 151936
    linear_num_v_heads: int = 48
    linear_num_k_heads: int = 16
    full_attention_interval: int = 4
    rope_dim: int = 64
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1.0e7

    def to_c(self) -> ModelConfig:
        return ModelConfig(self.hidden_size, self.intermediate_size, self.num_hidden_layers, self.num_attention_heads,
                           self.num_key_value_heads, self.vocab_size, self.linear_num_v_heads, self.linear_num_k_heads,
                           self.full_attention_interval, self.rope_dim, self.rms_norm_eps, self.rope_theta)

    @property
    def conv_channels(self) -> int:
        return 2 * self.linear_num_k_heads * 128 + self.linear_num_v_heads * 128


_DTYPES = {"w": np.uint8, "s": np.float16}


class GenerationConfig(C.Structure):
    """``xinfer_generation_config``."""
    _fields_ = [("max_new_tokens", C.c_int32), ("temperature", C.c_float), ("top_p", C.c_float),
                ("eos_token_id", C.c_int64), ("im_end_token_id", C.c_int64), ("seed", C.c_uint64)]


class GenerationStats(C.Structure):
    """``xinfer_generation_stats``."""
    _fields_ = [("prompt_tokens", C.c_int64), ("generated_tokens", C.c_int64), ("steps", C.c_int64),
                ("time_to_first_token_sec", C.c_double), ("decode_tokens_per_sec", C.c_double),
                ("total_time_sec", C.c_double)]


@dataclass
class GenerationResult:
    """The token-level fields of the reference's ``GenerationResult`` (include/xinfer/engine.h:44-57) for one
    sequence; text and tokenizer fields are the caller's."""
    token_ids: list
    prompt_tokens: int
    generated_tokens: int
    finish_reason: str
    time_to_first_token_sec: float
    decode_tokens_per_sec: float
    total_time_sec: float
    steps: int


class SpecDecoder:
    def __init__(self, shape: Shape, batch: int = 8, k: int = 3, max_seq: int = 8448, seed: int = 0, tp=None):
        """``tp``: a connected ``xinfer_b200.tp.TpGroup`` for the N-split step (every rank creates its decoder with the
        same arguments), None for one GPU."""
        self.shape, self.batch, self.k, self.max_seq = shape, batch, k, max_seq
        self.tp = tp
        h = C.c_void_p()
        cfg = shape.to_c()
        code = lib().xinfer_spec_decoder_create_tp(C.byref(cfg), batch, k, max_seq, seed,
                                                   None if tp is None else tp.handle, C.byref(h))
        if code == _lib.ERR_OUT_OF_MEMORY:
            raise MemoryError("SpecDecoder: device allocation failed")
        check(code, "spec_decoder_create")
        self._h = h
        self._emitted = np.zeros((batch, k + 1), np.int64)
        self._counts = np.zeros(batch, np.int32)

    @staticmethod
    def exchange_bytes(shape: Shape, batch: int, k: int, world: int) -> int:
        """Size of the exchange region a ``TpGroup`` needs for this decoder."""
        cfg = shape.to_c()
        return int(lib().xinfer_spec_decoder_exchange_bytes(C.byref(cfg), batch, k, world))

    def set_sampling(self, temperature: float, seed: int = 0) -> None:
        """temperature <= 0: greedy (default).  Otherwise stochastic drafting and the reference's rejection rule with
        Philox uniforms of (seed, step index); call before ``capture`` (``xinfer_spec_decoder_set_sampling``)."""
        code = lib().xinfer_spec_decoder_set_sampling(self._h, float(temperature), int(seed))
        if code != 0:
            raise _lib.XInferError(code, "spec_decoder_set_sampling: " + self._err())

    def set_top_p(self, top_p: float) -> None:
        """Nucleus sampling on both sides of the stochastic rule (``xinfer_spec_decoder_set_top_p``); 1 = off."""
        code = lib().xinfer_spec_decoder_set_top_p(self._h, float(top_p))
        if code != 0:
            raise _lib.XInferError(code, "spec_decoder_set_top_p: " + self._err())

    def prefill(self, prompt, stream=None) -> None:
        """Builds the context from ``prompt`` (int64 [batch][T]); call ``reset(0, seed)`` first.  Afterwards the
        context length is T - 1 and the last prompt token is the current token (``xinfer_spec_decoder_prefill``)."""
        p = np.ascontiguousarray(prompt, np.int64)
        assert p.ndim == 2 and p.shape[0] == self.batch
        s = stream if stream is not None else torch.cuda.current_stream()
        code = lib().xinfer_spec_decoder_prefill(self._h, C.c_void_p(s.cuda_stream), p.ctypes.data_as(C.c_void_p), p.shape[1])
        if code != 0:
            raise _lib.XInferError(code, "spec_decoder_prefill: " + self._err())

    def generate(self, prompt, max_new_tokens: int = 256, temperature: float = 0.0, top_p: float = 1.0,
                 eos_token_id: int = -1, im_end_token_id: int = -1, seed: int = 0, stream=None):
        """The speculative generate loop for ``prompt`` (int64 [batch][T]) with the fields of the reference's
        ``GenerationConfig`` (include/xinfer/engine.h:17-25): reset, prefill, steps until every sequence has met a stop
        token or holds ``max_new_tokens`` tokens (``xinfer_spec_decoder_generate``).  Returns one ``GenerationResult``
        per sequence; the timing fields describe the whole batch."""
        p = np.ascontiguousarray(prompt, np.int64)
        assert p.ndim == 2 and p.shape[0] == self.batch
        cfg = GenerationConfig(int(max_new_tokens), float(temperature), float(top_p), int(eos_token_id),
                               int(im_end_token_id), int(seed))
        cap = max(int(max_new_tokens), 1)
        toks = np.full((self.batch, cap), -1, np.int64)
        n = np.zeros(self.batch, np.int32)
        fin = np.zeros(self.batch, np.int32)
        st = GenerationStats()
        s = stream if stream is not None else torch.cuda.current_stream()
        code = lib().xinfer_spec_decoder_generate(self._h, C.c_void_p(s.cuda_stream), p.ctypes.data_as(C.c_void_p), p.shape[1],
                                                  C.byref(cfg), toks.ctypes.data_as(C.c_void_p), n.ctypes.data_as(C.c_void_p),
                                                  fin.ctypes.data_as(C.c_void_p), C.byref(st))
        if code != 0:
            raise _lib.XInferError(code, "spec_decoder_generate: " + self._err())
        return [GenerationResult(token_ids=toks[b, :n[b]].tolist(), prompt_tokens=int(st.prompt_tokens),
                                 generated_tokens=int(n[b]), finish_reason="stop" if fin[b] == 0 else "length",
                                 time_to_first_token_sec=st.time_to_first_token_sec,
                                 decode_tokens_per_sec=st.decode_tokens_per_sec, total_time_sec=st.total_time_sec,
                                 steps=int(st.steps)) for b in range(self.batch)]

    def load_artifact(self, reader, verify: bool = True) -> None:
        """Replaces the synthetic weights by the tensors of an open ``xinfer_b200.artifact.ArtifactReader``
        (section names of the reference's loader, src/targets/qwen3_8_27b/weights.cpp:358-640)."""
        check(lib().xinfer_spec_decoder_load_artifact(self._h, reader._h, 1 if verify else 0), "spec_decoder_load_artifact")

    def close(self):
        if getattr(self, "_h", None):
            lib().xinfer_spec_decoder_destroy(self._h)
            self._h = None

    __del__ = close

    def _err(self):
        return lib().xinfer_spec_decoder_error(self._h).decode()

    def reset(self, context_len: int, seed: int = 0):
        check(lib().xinfer_spec_decoder_reset(self._h, context_len, seed), "spec_decoder_reset")

    def set_tokens(self, toks):
        t = np.ascontiguousarray(toks, np.int64)
        check(lib().xinfer_spec_decoder_set_tokens(self._h, t.ctypes.data_as(C.c_void_p)), "set_tokens")

    def override_drafts(self, drafts):
        """Test hook: verify these [batch, k] tokens instead of the MTP head's (None disarms)."""
        if drafts is None:
            check(lib().xinfer_spec_decoder_override_drafts(self._h, None), "override_drafts")
            return
        t = np.ascontiguousarray(drafts, np.int64)
        check(lib().xinfer_spec_decoder_override_drafts(self._h, t.ctypes.data_as(C.c_void_p)), "override_drafts")

    def step(self):
        code = lib().xinfer_spec_decoder_step(self._h, torch.cuda.current_stream().cuda_stream)
        if code < 0:
            raise _lib.XInferError(code, "spec_decoder_step: " + self._err())

    def enqueue_linears(self):
        """Measurement: only the W4A16 launches of one step, on the current stream."""
        code = lib().xinfer_spec_decoder_enqueue_linears(self._h, torch.cuda.current_stream().cuda_stream)
        if code < 0:
            raise _lib.XInferError(code, "enqueue_linears: " + self._err())

    def capture(self, stream: torch.cuda.Stream):
        code = lib().xinfer_spec_decoder_capture(self._h, stream.cuda_stream)
        if code < 0:
            raise _lib.XInferError(code, "spec_decoder_capture: " + self._err())

    def results(self):
        """(emitted [batch, k+1] int64 with -1 padding, counts [batch]); synchronises the stream."""
        check(lib().xinfer_spec_decoder_results(self._h, torch.cuda.current_stream().cuda_stream,
                                                self._emitted.ctypes.data_as(C.c_void_p),
                                                self._counts.ctypes.data_as(C.c_void_p)), "spec_decoder_results")
        return self._emitted.copy(), self._counts.copy()

    def info(self, what: int) -> int:
        return int(lib().xinfer_spec_decoder_info(self._h, what))

    def tensor(self, layer: int, name: str, dtype, shape=None) -> np.ndarray:
        """Host copy of a named device tensor (weights or state)."""
        nbytes = C.c_int64()
        ptr = lib().xinfer_spec_decoder_tensor(self._h, layer, name.encode(), C.byref(nbytes))
        if not ptr:
            raise KeyError(f"{layer}:{name}")
        torch.cuda.synchronize()
        raw = np.empty(nbytes.value, np.uint8)
        check(lib().xinfer_copy_device_to_host(raw.ctypes.data_as(C.c_void_p), ptr, nbytes.value), "copy_device_to_host")
        arr = raw.view(dtype)
        return arr.reshape(shape) if shape is not None else arr

    def write_tensor(self, layer: int, name: str, array: np.ndarray):
        nbytes = C.c_int64()
        ptr = lib().xinfer_spec_decoder_tensor(self._h, layer, name.encode(), C.byref(nbytes))
        if not ptr:
            raise KeyError(f"{layer}:{name}")
        a = np.ascontiguousarray(array)
        assert a.nbytes == nbytes.value, (a.nbytes, nbytes.value)
        torch.cuda.synchronize()
        check(lib().xinfer_copy_host_to_device(ptr, a.ctypes.data_as(C.c_void_p), a.nbytes), "copy_host_to_device")

    def is_full(self, layer: int) -> bool:
        return bool(lib().xinfer_spec_decoder_tensor(self._h, layer, b"is_full", None))
