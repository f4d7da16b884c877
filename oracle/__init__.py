"""numpy-facing loader for the CPU oracle (test infrastructure; the product never imports this).

Only the test-suite, ``__graft_entry__.smoke()`` and ``bench.py``'s cpu_baseline / reference arm
may import this package.  Every function forwards to ``liboracle.so`` built from the C++
restatement beside this file (see ``build.py``); the C++ sources cite the reference lines they follow.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


class AcceptResult(C.Structure):
    _fields_ = [
        ("accepted_tokens", C.c_int64 * 64),
        ("bonus_or_resampled_token", C.c_int64),
        ("rejected_token", C.c_int64),
        ("num_accepted", C.c_int64),
        ("num_rejected", C.c_int64),
        ("num_resampled", C.c_int64),
        ("num_remaining", C.c_int64),
        ("has_rejected_token", C.c_int32),
        ("contract_violated", C.c_int32),
    ]


def lib():
    global _lib
    if _lib is None:
        path = _build.LIB
        if not os.path.exists(path) or _build._stale(path, _build._sources()):
            path = _build.build_oracle()
        _lib = C.CDLL(path)
        _lib.oracle_argmax.restype = C.c_int64
        _lib.oracle_token_prob_f32.restype = C.c_float
        _lib.oracle_token_prob_f64.restype = C.c_double
        _lib.oracle_crc64.restype = C.c_uint64
        _lib.oracle_crc64.argtypes = [C.c_void_p, C.c_size_t]
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def unpack_int4(packed: np.ndarray, shift_form: bool = False) -> np.ndarray:
    packed = _c(packed, np.uint8)
    out = np.empty(packed.size * 2, dtype=np.int8)
    fn = lib().oracle_unpack_int4_shift if shift_form else lib().oracle_unpack_int4
    fn(_p(packed), C.c_int64(packed.size), _p(out))
    return out.reshape(packed.shape[:-1] + (packed.shape[-1] * 2,))


def quantize_int4(w: np.ndarray, group_size: int = 128):
    w = _c(w, np.float32)
    rows, K = w.shape
    packed = np.empty((rows, K // 2), dtype=np.uint8)
    scales = np.empty((rows, K // group_size), dtype=np.float16)
    lib().oracle_quantize_int4(_p(w), C.c_int64(rows), C.c_int64(K), C.c_int(group_size), _p(packed), _p(scales))
    return packed, scales


def _linear(fn, X, W, scales, bias, group_size):
    X = _c(X, np.float32)
    W = _c(W, np.uint8)
    scales = _c(scales, np.float16)
    bias = _c(bias, np.float32)
    M, K = X.shape
    N = W.shape[0]
    Y = np.zeros((M, N), dtype=np.float32)
    fn(_p(Y), _p(X), _p(W), _p(scales), _p(bias), C.c_int64(M), C.c_int64(N), C.c_int64(K), C.c_int(group_size))
    return Y


def linear_int4_f64(X, W, scales, bias=None, group_size=128):
    """fp64-accumulate oracle of tests/test_ops_oracle.cpp:318-348 (X given as fp32 values)."""
    return _linear(lib().oracle_linear_int4_f64, X, W, scales, bias, group_size)


def linear_int4_naive_f32(X, W, scales, bias=None, group_size=128):
    """linear_int4_naive of src/ops/linear.cpp:681-730 (fp32 sequential)."""
    return _linear(lib().oracle_linear_int4_naive_f32, X, W, scales, bias, group_size)


def linear_int4_grouped_f32(X, W, scales, bias=None, group_size=128):
    """production association of src/ops/linear.cpp:239-298 (per-group dot, then * scale)."""
    return _linear(lib().oracle_linear_int4_grouped_f32, X, W, scales, bias, group_size)


def mlp_gate_up_swiglu_f64(X, Wg, sg, Wu, su, group_size=128):
    X = _c(X, np.float32)
    Wg, Wu = _c(Wg, np.uint8), _c(Wu, np.uint8)
    sg, su = _c(sg, np.float16), _c(su, np.float16)
    M, K = X.shape
    N = Wg.shape[0]
    Y = np.zeros((M, N), dtype=np.float32)
    lib().oracle_mlp_gate_up_swiglu_f64(_p(Y), _p(X), _p(Wg), _p(sg), _p(Wu), _p(su),
                                        C.c_int64(M), C.c_int64(N), C.c_int64(K), C.c_int(group_size))
    return Y


def argmax(logits: np.ndarray) -> int:
    logits = _c(logits, np.float32)
    return int(lib().oracle_argmax(_p(logits), C.c_int64(logits.size)))


def token_prob_f32(logits, tok) -> float:
    logits = _c(logits, np.float32)
    return float(lib().oracle_token_prob_f32(_p(logits), C.c_int64(logits.size), C.c_int64(int(tok))))


def token_prob_f64(logits, tok) -> float:
    logits = _c(logits, np.float32)
    return float(lib().oracle_token_prob_f64(_p(logits), C.c_int64(logits.size), C.c_int64(int(tok))))


def speculative_accept_reject(draft_tokens, target_logits, draft_probs=None, rand_uniform=None,
                              inv_temperature: float = 1.0) -> dict:
    """Literal restatement of src/ops/sampling.cpp:94-199; returns the result struct as a dict."""
    res = AcceptResult()
    dt = _c(draft_tokens, np.int64)
    tl = _c(target_logits, np.float32)
    n = 0 if dt is None else dt.size
    vocab = 0 if tl is None or tl.ndim < 2 else tl.shape[-1]
    dp = _c(draft_probs, np.float32)
    ru = _c(rand_uniform, np.float32)
    lib().oracle_speculative_accept_reject(_p(dt), C.c_int64(n), _p(tl), C.c_int64(vocab), _p(dp), _p(ru),
                                           C.c_float(inv_temperature), C.byref(res))
    return {
        "accepted_tokens": [int(res.accepted_tokens[i]) for i in range(res.num_accepted)],
        "bonus_or_resampled_token": int(res.bonus_or_resampled_token),
        "has_rejected_token": bool(res.has_rejected_token),
        "rejected_token": int(res.rejected_token),
        "num_accepted": int(res.num_accepted),
        "num_rejected": int(res.num_rejected),
        "num_resampled": int(res.num_resampled),
        "num_remaining": int(res.num_remaining),
        "contract_violated": bool(res.contract_violated),
    }


def softmax(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty_like(x)
    rows = int(np.prod(x.shape[:-1])) if x.ndim > 1 else 1
    lib().oracle_softmax(_p(out), _p(x), C.c_int64(rows), C.c_int64(x.shape[-1]))
    return out


def philox4x32_10(ctr, key):
    c = (C.c_uint32 * 4)(*[int(v) for v in ctr])
    k = (C.c_uint32 * 2)(*[int(v) for v in key])
    o = (C.c_uint32 * 4)()
    lib().oracle_philox4x32_10(c, k, o)
    return [int(v) for v in o]


def philox_uniform(n: int, seed: int, subsequence: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().oracle_philox_uniform(_p(out), C.c_int64(n), C.c_uint64(seed), C.c_uint64(subsequence))
    return out


def crc64(data: bytes) -> int:
    buf = C.create_string_buffer(data, len(data))
    return int(lib().oracle_crc64(C.cast(buf, C.c_void_p), C.c_size_t(len(data))))


def reference_crc_lib():
    """The reference's own libxinfer_artifact_c.so (oracle/_ref), or None when it was never built."""
    path = _build.build_reference_crc()
    if not path or not os.path.exists(path):
        return None
    ref = C.CDLL(path)
    ref.xinfer_crc64.restype = C.c_uint64
    ref.xinfer_crc64.argtypes = [C.c_void_p, C.c_size_t]
    ref.xinfer_crc64_file.restype = C.c_uint64
    ref.xinfer_crc64_file.argtypes = [C.c_char_p, C.c_uint64]
    return ref


# ------------------------------------------------------------------------------------------------
# Per-layer glue (mixers_oracle.cpp).  fp16 arrays are numpy float16; states are float32, updated in place.
# ------------------------------------------------------------------------------------------------
def _h(a):
    return np.ascontiguousarray(a, dtype=np.float16)


def embed(table_bf16_bits: np.ndarray, tokens, vocab: int) -> np.ndarray:
    """embed_tokens_lookup (src/targets/qwen3_8/forward.cpp:17-64); table given as uint16 bf16 bits."""
    table = _c(table_bf16_bits, np.uint16)
    toks = _c(tokens, np.int64)
    hidden = table.shape[1]
    out = np.empty((toks.size, hidden), np.float16)
    lib().oracle_embed(_p(out), _p(table), _p(toks), C.c_int64(toks.size), C.c_int64(hidden), C.c_int64(vocab))
    return out


def rmsnorm_f16(x, w, eps: float = 1e-6) -> np.ndarray:
    x = _h(x)
    w = _c(w, np.float32)
    hidden = x.shape[-1]
    out = np.empty_like(x)
    lib().oracle_rmsnorm_f16(_p(out), _p(x), _p(w), C.c_int64(x.size // hidden), C.c_int64(hidden), C.c_float(eps))
    return out


def add_inplace_f16(a, b) -> np.ndarray:
    a = _h(a).copy()
    b = _h(b)
    lib().oracle_add_inplace_f16(_p(a), _p(b), C.c_int64(a.size))
    return a


def rope_f16(q, k, positions, theta: float, rotary_dim: int):
    """In place on copies; q [T, hq, hd], k [T, hkv, hd]."""
    q = _h(q).copy()
    k = _h(k).copy()
    pos = _c(positions, np.int64)
    T, hq, hd = q.shape
    lib().oracle_rope_f16(_p(q), _p(k), C.c_int64(T), C.c_int64(hq), C.c_int64(k.shape[1]), C.c_int64(hd), _p(pos),
                          C.c_float(theta), C.c_int64(rotary_dim))
    return q, k


def kv_write(k_cache, v_cache, k_in, v_in, start_pos: int):
    """Caches [max_seq, hkv, hd] float16, modified in place."""
    assert k_cache.dtype == np.float16 and k_cache.flags.c_contiguous
    k_in, v_in = _h(k_in), _h(v_in)
    T, hkv, hd = k_in.shape
    lib().oracle_kv_write(_p(k_cache), _p(v_cache), _p(k_in), _p(v_in), C.c_int64(start_pos), C.c_int64(T),
                          C.c_int64(hkv), C.c_int64(hd), C.c_int64(k_cache.shape[0]))


def sdpa_cached(q, k_cache, v_cache, start_pos: int) -> np.ndarray:
    q = _h(q)
    T, hq, hd = q.shape
    out = np.zeros_like(q)
    lib().oracle_sdpa_cached(_p(out), _p(q), _p(k_cache), _p(v_cache), C.c_int64(start_pos), C.c_int64(T),
                             C.c_int64(hq), C.c_int64(k_cache.shape[1]), C.c_int64(hd), C.c_float(0.0),
                             C.c_int64(k_cache.shape[0]))
    return out


def conv1d_silu(x, conv_w, conv_state) -> np.ndarray:
    """x [T, C] fp16; conv_state [3, C] float32 updated in place (or None)."""
    x = _h(x)
    w = _c(conv_w, np.float32)
    out = np.empty_like(x)
    if conv_state is not None:
        assert conv_state.dtype == np.float32 and conv_state.flags.c_contiguous
    lib().oracle_conv1d_silu(_p(out), _p(x), _p(w), C.c_int64(x.shape[0]), _p(conv_state), C.c_int64(x.shape[1]))
    return out


def gdn(qkv, z, b, a, A_log, dt_bias, norm_w, state, hv: int, hk: int, zero_state: bool = False) -> np.ndarray:
    """state [hv, 128, 128] float32 updated in place."""
    qkv, z, b, a = _h(qkv), _h(z), _h(b), _h(a)
    assert state.dtype == np.float32 and state.flags.c_contiguous
    T = qkv.shape[0]
    out = np.empty((T, hv * 128), np.float16)
    lib().oracle_gdn(_p(out), _p(qkv), _p(z), _p(b), _p(a), _p(_c(A_log, np.float32)), _p(_c(dt_bias, np.float32)),
                     _p(_c(norm_w, np.float32)), _p(state), C.c_int64(T), C.c_int(1 if zero_state else 0),
                     C.c_int64(hv), C.c_int64(hk))
    return out


def split_q(q_gate, hq: int, hd: int) -> np.ndarray:
    q_gate = _h(q_gate)
    T = q_gate.shape[0]
    out = np.empty((T, hq, hd), np.float16)
    lib().oracle_split_q(_p(out), _p(q_gate), C.c_int64(T), C.c_int64(hq), C.c_int64(hd))
    return out


def gate_output(attn, q_gate, hq: int, hd: int) -> np.ndarray:
    attn = _h(attn).copy()
    q_gate = _h(q_gate)
    lib().oracle_gate_output(_p(attn), _p(q_gate), C.c_int64(attn.shape[0]), C.c_int64(hq), C.c_int64(hd))
    return attn
