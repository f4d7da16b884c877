"""Host-side mirror of the reference's ops interface for this path (``xinfer::ops`` in
src/ops/linear.h and src/ops/sampling.h), on torch CUDA tensors.

Same names, argument order and meaning as the reference: outputs first, raw row-major buffers, shapes as
integers, ``group_size`` defaulting to 128.  The ``sycl::queue&`` becomes the current torch CUDA stream.
Every function calls the C-ABI of libxinfer_b200.so; nothing here computes on the host.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import AcceptRecord, AcceptResult, FusedDesc, check, lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype, name: str):
    if not t.is_cuda or t.dtype != dtype or not t.is_contiguous():
        raise ValueError(f"{name}: expected a contiguous CUDA tensor of {dtype}, got {t.dtype} on {t.device}")


def linear_int4(Y: torch.Tensor, X: torch.Tensor, W_int4: torch.Tensor, scales: torch.Tensor,
                bias: Optional[torch.Tensor], M: int, N: int, K: int, group_size: int = 128) -> int:
    """``xinfer::ops::linear_int4`` (src/ops/linear.h:30-63): Y[M,N] = X[M,K] W^T + bias.

    The overload is chosen from the dtypes like the reference's three C++ overloads:
    fp16->fp16, fp16->fp32, fp32->fp32.
    """
    _need(W_int4, torch.uint8, "W_int4")
    _need(scales, torch.float16, "scales")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if X.dtype == torch.float16 and Y.dtype == torch.float16:
        fn = lib().xinfer_linear_int4_f16f16
    elif X.dtype == torch.float16 and Y.dtype == torch.float32:
        fn = lib().xinfer_linear_int4_f16f32
    elif X.dtype == torch.float32 and Y.dtype == torch.float32:
        fn = lib().xinfer_linear_int4_f32f32
    else:
        raise TypeError(f"no linear_int4 overload for X {X.dtype} -> Y {Y.dtype}")
    return check(fn(_stream(), _ptr(Y), _ptr(X), _ptr(W_int4), _ptr(scales), _ptr(bias), M, N, K, group_size),
                 "linear_int4")


def linear_int4_ld(Y: torch.Tensor, ldy: int, X, W_int4, scales, bias, M: int, N: int, K: int,
                   group_size: int = 128) -> int:
    """fp16->fp16 linear_int4 writing rows of stride ``ldy`` (the N-split tensor-parallel form)."""
    return check(lib().xinfer_linear_int4_f16f16_ld(_stream(), _ptr(Y), ldy, _ptr(X), _ptr(W_int4), _ptr(scales),
                                                    _ptr(bias), M, N, K, group_size), "linear_int4_ld")


def linear_int4_noalloc(Y: torch.Tensor, X, W_int4, scales, bias, M: int, N: int, K: int, group_size: int = 128) -> int:
    """fp16 -> fp16 linear_int4 through the entry point that allocates nothing (fixed in-library scratch); for
    hosts that cannot call cudaMalloc once running.  Refuses shapes outside its limits with ERR_INVALID_ARGUMENT."""
    return check(lib().xinfer_linear_int4_f16f16_noalloc(_stream(), _ptr(Y), _ptr(X), _ptr(W_int4), _ptr(scales),
                                                         _ptr(bias), M, N, K, group_size), "linear_int4_noalloc")


class LinearPlan:
    """Launch plan for a fixed sequence of fp16 ``linear_int4`` / fused / SwiGLU calls (one decode or verify pass).

    ``with plan.record(): run_the_sequence()`` once, then ``plan.rewind()`` before every later round: each launch
    of a round also pulls the first weight tiles of the next launch into L2.  Results are unchanged; a call
    outside the recorded order switches the hints off.  One plan per process."""

    class _Rec:
        def __enter__(self):
            lib().xinfer_linear_plan_record_begin()

        def __exit__(self, *exc):
            lib().xinfer_linear_plan_record_end()
            return False

    def record(self):
        return LinearPlan._Rec()

    @staticmethod
    def rewind() -> None:
        lib().xinfer_linear_plan_rewind()

    @staticmethod
    def clear() -> None:
        lib().xinfer_linear_plan_clear()


def linear_int4_fused(X: torch.Tensor, descs: Sequence[dict], M: int, K: int, group_size: int = 128) -> int:
    """``xinfer::ops::linear_int4_fused`` (src/ops/linear.h:96-111).

    ``descs`` holds up to four dicts with the fields of FusedProjectionDesc: Y, W_int4, scales, bias, N.
    """
    n = len(descs)
    arr = (FusedDesc * max(n, 1))()
    for i, d in enumerate(descs):
        arr[i].Y = _ptr(d["Y"])
        arr[i].W_int4 = _ptr(d["W_int4"])
        arr[i].scales = _ptr(d["scales"])
        arr[i].bias = _ptr(d.get("bias"))
        arr[i].N = int(d["N"])
    fn = lib().xinfer_linear_int4_fused_f16 if X.dtype == torch.float16 else lib().xinfer_linear_int4_fused_f32
    return check(fn(_stream(), _ptr(X), arr, n, M, K, group_size), "linear_int4_fused")


def mlp_gate_up_swiglu_int4(Y_swiglu: torch.Tensor, X: torch.Tensor, W_gate, scales_gate, W_up, scales_up,
                            M: int, N: int, K: int, group_size: int = 128) -> int:
    """``xinfer::ops::mlp_gate_up_swiglu_int4`` (src/ops/linear.h:117-139): Y = silu(gate x) * (up x)."""
    fn = (lib().xinfer_mlp_gate_up_swiglu_int4_f16 if X.dtype == torch.float16
          else lib().xinfer_mlp_gate_up_swiglu_int4_f32)
    return check(fn(_stream(), _ptr(Y_swiglu), _ptr(X), _ptr(W_gate), _ptr(scales_gate), _ptr(W_up), _ptr(scales_up),
                    M, N, K, group_size), "mlp_gate_up_swiglu_int4")


def argmax_scratch_size(vocab_size: int) -> int:
    """``xinfer::ops::argmax_scratch_size`` (src/ops/sampling.h:11-15)."""
    return int(lib().xinfer_argmax_scratch_size(vocab_size))


def argmax(logits: Optional[torch.Tensor], vocab_size: int, partial_max: Optional[torch.Tensor] = None,
           partial_idx: Optional[torch.Tensor] = None) -> int:
    """``xinfer::ops::argmax`` (src/ops/sampling.h:17-25); synchronous, returns the token id."""
    r = int(lib().xinfer_argmax(_stream(), _ptr(logits), vocab_size, _ptr(partial_max), _ptr(partial_idx)))
    if r < 0:
        raise _lib.XInferError(r, "argmax")
    return r


def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> int:
    """Batched asynchronous argmax: out[r] (int64, device) = argmax(logits[r])."""
    rows, vocab = logits.shape
    return check(lib().xinfer_argmax_rows(_stream(), _ptr(logits), logits.stride(0), rows, vocab, _ptr(out)),
                 "argmax_rows")


def speculative_accept_reject(draft_tokens: Sequence[int], num_draft_tokens: int, target_logits: Optional[torch.Tensor],
                              vocab_size: int, draft_probs: Optional[Sequence[float]] = None,
                              rand_uniform: Optional[Sequence[float]] = None) -> dict:
    """``xinfer::ops::speculative_accept_reject`` (src/ops/sampling.h:42-49).

    Host token / probability / uniform arrays, device logits, synchronous, returns the fields of
    SpeculativeAcceptanceResult.  Raises XInferError(ERR_CONTRACT) where the reference throws
    std::logic_error.
    """
    n = int(num_draft_tokens)
    toks = (C.c_int64 * max(n, 1))(*[int(t) for t in draft_tokens][:n]) if draft_tokens is not None else None
    probs = (C.c_float * max(n, 1))(*[float(p) for p in draft_probs][:n]) if draft_probs is not None else None
    unif = (C.c_float * max(n, 1))(*[float(u) for u in rand_uniform][:n]) if rand_uniform is not None else None
    res = AcceptResult()
    check(lib().xinfer_speculative_accept_reject(
        _stream(), C.cast(toks, C.c_void_p) if toks is not None else None, n, _ptr(target_logits), vocab_size,
        C.cast(probs, C.c_void_p) if probs is not None else None,
        C.cast(unif, C.c_void_p) if unif is not None else None, C.byref(res)), "speculative_accept_reject")
    return {
        "accepted_tokens": [int(res.accepted_tokens[i]) for i in range(res.num_accepted)],
        "bonus_or_resampled_token": int(res.bonus_or_resampled_token),
        "has_rejected_token": bool(res.has_rejected_token),
        "rejected_token": int(res.rejected_token),
        "num_accepted": int(res.num_accepted),
        "num_rejected": int(res.num_rejected),
        "num_resampled": int(res.num_resampled),
        "num_remaining": int(res.num_remaining),
    }


ACCEPT_RECORD_BYTES = C.sizeof(AcceptRecord)


def speculative_accept_reject_batched(draft_tokens: torch.Tensor, target_logits: torch.Tensor,
                                      draft_probs: Optional[torch.Tensor], rand_uniform: Optional[torch.Tensor],
                                      out_records: torch.Tensor, inv_temperature: float = 1.0,
                                      bonus_row: Optional[int] = None) -> int:
    """Device-side batched acceptance.  target_logits is [batch, rows_per_seq, vocab] fp32, draft_tokens
    [batch, k] int64, out_records a uint8 tensor of batch * ACCEPT_RECORD_BYTES bytes."""
    batch, rows_per_seq, vocab = target_logits.shape
    k = draft_tokens.shape[1]
    if bonus_row is None:
        bonus_row = k - 1
    return check(lib().xinfer_speculative_accept_reject_batched(
        _stream(), _ptr(draft_tokens), _ptr(target_logits), target_logits.stride(1), vocab, _ptr(draft_probs),
        _ptr(rand_uniform), inv_temperature, batch, k, rows_per_seq, bonus_row, _ptr(out_records)),
        "speculative_accept_reject_batched")


def sample_tokens(logits: torch.Tensor, rand_uniform: torch.Tensor, tokens_out: torch.Tensor, probs_out: torch.Tensor,
                  inv_temperature: float = 1.0) -> int:
    """One token per row of ``logits`` [rows, vocab] fp32 from softmax(logits * inv_temperature) at the row's uniform, and
    its probability (``xinfer_sample_tokens``): the draft token and p_draft of the stochastic acceptance rule."""
    rows, vocab = logits.shape
    return check(lib().xinfer_sample_tokens(_stream(), _ptr(logits), logits.stride(0), vocab, rows, inv_temperature,
                                            _ptr(rand_uniform), _ptr(tokens_out), _ptr(probs_out)), "sample_tokens")


def sample_tokens_top_p(logits: torch.Tensor, rand_uniform: torch.Tensor, tokens_out: torch.Tensor, probs_out: torch.Tensor,
                        inv_temperature: float, top_p: float) -> int:
    """``sample_tokens`` restricted to each row's nucleus at ``top_p`` (``xinfer_sample_tokens_top_p``)."""
    rows, vocab = logits.shape
    return check(lib().xinfer_sample_tokens_top_p(_stream(), _ptr(logits), logits.stride(0), vocab, rows, inv_temperature,
                                                  top_p, _ptr(rand_uniform), _ptr(tokens_out), _ptr(probs_out)),
                 "sample_tokens_top_p")


def decode_accept_records(out_records: torch.Tensor) -> list:
    raw = out_records.cpu().numpy().tobytes()
    n = len(raw) // ACCEPT_RECORD_BYTES
    recs = (AcceptRecord * n).from_buffer_copy(raw)
    return [{f: int(getattr(r, f)) for f, _ in AcceptRecord._fields_ if f != "reserved"} for r in recs]


def philox_uniform(out: torch.Tensor, seed: int, subsequence: int = 0) -> int:
    return check(lib().xinfer_philox_uniform(_stream(), _ptr(out), out.numel(), seed, subsequence), "philox_uniform")


def device_status(device: int = 0) -> int:
    return int(lib().xinfer_device_status(device))


def set_wait_hooks(limit_clocks: int = 0, withhold_x_from_stage: int = -1) -> None:
    """Test hook for the bounded device-side waits of the tcgen05 linear kernel (0 / -1 restore the defaults)."""
    lib().xinfer_debug_set_wait_hooks(limit_clocks, withhold_x_from_stage)


# ---- per-layer mixer ops (fp16 overloads of the reference's ops) -------------------------------------------
def rmsnorm(out: torch.Tensor, inp: torch.Tensor, weight: torch.Tensor, num_tokens: int, hidden_size: int,
            eps: float = 1e-6) -> int:
    """``xinfer::ops::rmsnorm`` (src/ops/rmsnorm.h:17-23), fp16 in/out, fp32 weight."""
    return check(lib().xinfer_rmsnorm_f16(_stream(), _ptr(out), _ptr(inp), _ptr(weight), num_tokens, hidden_size, eps),
                 "rmsnorm")


def rmsnorm_residual(out, residual, inp, weight, num_tokens: int, hidden_size: int, eps: float = 1e-6) -> int:
    """``xinfer::ops::rmsnorm_residual`` (src/ops/rmsnorm.h:35-42): residual += in; out = rmsnorm(residual)."""
    return check(lib().xinfer_rmsnorm_residual_f16(_stream(), _ptr(out), _ptr(residual), _ptr(inp), _ptr(weight),
                                                   num_tokens, hidden_size, eps), "rmsnorm_residual")


def rope(q: Optional[torch.Tensor], k: Optional[torch.Tensor], num_tokens: int, num_q_heads: int, num_kv_heads: int,
         head_dim: int, positions: torch.Tensor, theta: float = 1.0e7, rotary_dim: int = 64) -> int:
    """``xinfer::ops::rope`` (src/ops/rope.h:25-34), in place; positions is a device int64 tensor."""
    return check(lib().xinfer_rope_f16(_stream(), _ptr(q), _ptr(k), num_tokens, num_q_heads, num_kv_heads, head_dim,
                                       _ptr(positions), theta, rotary_dim), "rope")


def attention_write_kv_cache(k_cache, v_cache, K_in, V_in, start_pos: int, num_tokens: int, num_kv_heads: int,
                             head_dim: int, max_seq_len: int = 0) -> int:
    """``xinfer::ops::attention_write_kv_cache`` (src/ops/attention.h:49-58)."""
    return check(lib().xinfer_attention_write_kv_cache_f16(_stream(), _ptr(k_cache), _ptr(v_cache), _ptr(K_in), _ptr(V_in),
                                                           start_pos, num_tokens, num_kv_heads, head_dim, max_seq_len),
                 "attention_write_kv_cache")


def sdpa_causal_cached(out, Q, k_cache, v_cache, start_pos: int, num_q_tokens: int, num_q_heads: int, num_kv_heads: int,
                       head_dim: int, scale: float = 0.0, max_seq_len: int = 0) -> int:
    """``xinfer::ops::sdpa_causal_cached`` (src/ops/attention.h:102-113)."""
    return check(lib().xinfer_sdpa_causal_cached_f16(_stream(), _ptr(out), _ptr(Q), _ptr(k_cache), _ptr(v_cache), start_pos,
                                                     num_q_tokens, num_q_heads, num_kv_heads, head_dim, scale, max_seq_len),
                 "sdpa_causal_cached")


def causal_conv1d_silu(out_qkv, in_qkv, conv_w, seq_len: int, conv_state: Optional[torch.Tensor] = None,
                       num_channels: int = 10240) -> int:
    """``targets::qwen3_8::causal_conv1d_silu`` (src/targets/qwen3_8/linear_attn.h:15-21)."""
    return check(lib().xinfer_causal_conv1d_silu_f16(_stream(), _ptr(out_qkv), _ptr(in_qkv), _ptr(conv_w), seq_len,
                                                     _ptr(conv_state), num_channels), "causal_conv1d_silu")


def recurrent_gated_delta_net(out, qkv, z, b, a, A_log, dt_bias, norm_weight, state_buffer, seq_len: int,
                              zero_state: bool = False, num_v_heads: int = 48, num_k_heads: int = 16) -> int:
    """``targets::qwen3_8::recurrent_gated_delta_net`` (src/targets/qwen3_8/linear_attn.h:41-58)."""
    return check(lib().xinfer_recurrent_gated_delta_net_f16(_stream(), _ptr(out), _ptr(qkv), _ptr(z), _ptr(b), _ptr(a),
                                                            _ptr(A_log), _ptr(dt_bias), _ptr(norm_weight), _ptr(state_buffer),
                                                            seq_len, 1 if zero_state else 0, num_v_heads, num_k_heads),
                 "recurrent_gated_delta_net")


def last_linear_path() -> int:
    return int(lib().xinfer_last_linear_path())


def set_linear_path(path: int) -> None:
    lib().xinfer_set_linear_path(path)


class DeviceArena:
    """``xinfer::core::DeviceArena`` (src/core/arena.h:14-66) over the C-ABI arena."""

    DEFAULT_ALIGNMENT = 64

    def __init__(self, capacity_bytes: int, default_alignment: int = 64):
        h = C.c_void_p()
        code = lib().xinfer_arena_create(capacity_bytes, default_alignment, C.byref(h))
        if code == _lib.ERR_OUT_OF_MEMORY:
            raise MemoryError("DeviceArena: device allocation failed")
        check(code, "arena_create")
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            lib().xinfer_arena_destroy(self._h)
            self._h = None

    __del__ = close

    def _call(self, fn, bytes_, alignment, what):
        out = C.c_void_p()
        code = fn(self._h, bytes_, alignment, C.byref(out))
        if code == _lib.ERR_OUT_OF_MEMORY:
            raise MemoryError(what)          # std::bad_alloc in the reference
        if code == _lib.ERR_INVALID_ARGUMENT:
            raise ValueError(what)           # std::invalid_argument in the reference
        check(code, what)
        return out.value

    def allocate(self, bytes_: int, alignment: int = 0):
        return self._call(lib().xinfer_arena_allocate, bytes_, alignment, "DeviceArena.allocate")

    def allocate_persistent(self, bytes_: int, alignment: int = 0):
        return self._call(lib().xinfer_arena_allocate_persistent, bytes_, alignment, "DeviceArena.allocate_persistent")

    def persistent_buffer(self, bytes_: int = 0, alignment: int = 0):
        return self._call(lib().xinfer_arena_persistent_buffer, bytes_, alignment, "DeviceArena.persistent_buffer")

    def reset(self):
        lib().xinfer_arena_reset(self._h)

    def capacity(self):
        return int(lib().xinfer_arena_capacity(self._h))

    def allocated_bytes(self):
        return int(lib().xinfer_arena_allocated_bytes(self._h))

    def remaining_bytes(self):
        return int(lib().xinfer_arena_remaining_bytes(self._h))

    def peak_allocated_bytes(self):
        return int(lib().xinfer_arena_peak_allocated_bytes(self._h))

    def base_ptr(self):
        return lib().xinfer_arena_base_ptr(self._h)


def crc64(data: bytes) -> int:
    buf = C.create_string_buffer(data, len(data))
    return int(lib().xinfer_crc64(C.cast(buf, C.c_void_p), len(data)))


def crc64_file(path: str, max_bytes: int = 0) -> int:
    return int(lib().xinfer_crc64_file(path.encode(), max_bytes))
