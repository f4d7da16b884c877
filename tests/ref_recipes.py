"""The reference tests' own input recipes and inline fp64 oracles for the per-layer mixer ops, restated in
numpy (test infrastructure).  Each function cites the lines of the reference test it follows; expected values
are recomputed at run time exactly as those tests do, from inputs that are pinned by a CRC-64 of the
generated stream (tests/golden/mixer_streams.json)."""
from __future__ import annotations

import functools
import json
import os
import subprocess
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden")
_TMP = tempfile.mkdtemp(prefix="xinfer_mt_")


@functools.lru_cache(maxsize=None)
def _exe() -> str:
    exe = os.path.join(_TMP, "mt_uniform")
    subprocess.check_call(["g++", "-O2", "-o", exe, os.path.join(GOLDEN, "mt_uniform.cpp")])
    return exe


def mt_stream(seed: int, lo: float, hi: float, n: int) -> np.ndarray:
    """n draws of std::uniform_real_distribution<float>(lo, hi) over std::mt19937(seed) (libstdc++)."""
    out = os.path.join(_TMP, f"s{seed}_{n}.bin")
    subprocess.check_call([_exe(), str(seed), repr(lo), repr(hi), str(n), out])
    return np.fromfile(out, dtype=np.float32)


def pinned_streams() -> dict:
    with open(os.path.join(GOLDEN, "mixer_streams.json")) as f:
        return json.load(f)


# ---------------------------------------------------------------------------------------------- RMSNorm
def rmsnorm_case():
    """tests/test_ops_oracle.cpp:50-66: 4 tokens x 5120, mt19937(42) U(-1,1); weight = draw + 1."""
    s = mt_stream(42, -1.0, 1.0, 4 * 5120 + 5120)
    x = s[:4 * 5120].reshape(4, 5120)
    w = (s[4 * 5120:] + np.float32(1.0)).astype(np.float32)
    return x, w, 1e-6, s


def rmsnorm_expected(x, w, eps):
    """tests/test_ops_oracle.cpp:68-82: fp64 sum of squares, float rsqrt, float products."""
    x64 = x.astype(np.float64)
    mean_sq = (x64 * x64).sum(axis=1) / x.shape[1]
    r = (1.0 / np.sqrt(mean_sq + np.float64(np.float32(eps)))).astype(np.float32)
    return (x * r[:, None] * w[None, :]).astype(np.float32)


# ---------------------------------------------------------------------------------------------- RoPE
def rope_case():
    """tests/test_ops_oracle.cpp:108-129: 4 tokens, 24 q / 4 kv heads, head_dim 256, positions 0,1,15,256,
    mt19937(43) U(-1,1), theta 1e7, rotary_dim 64."""
    nq, nk = 4 * 24 * 256, 4 * 4 * 256
    s = mt_stream(43, -1.0, 1.0, nq + nk)
    q = s[:nq].reshape(4, 24, 256)
    k = s[nq:].reshape(4, 4, 256)
    return q, k, np.array([0, 1, 15, 256], np.int64), 1.0e7, 64, s


def rope_expected(buf, positions, theta, rotary_dim):
    """tests/test_ops_oracle.cpp:131-153: fp64 frequency and angle, float cos/sin, float rotation."""
    out = buf.astype(np.float32).copy()
    half = rotary_dim // 2
    p = np.arange(half, dtype=np.float64)
    freq = 1.0 / np.power(np.float64(np.float32(theta)), 2.0 * p / rotary_dim)
    for t, pos in enumerate(positions):
        ang = np.float64(pos) * freq
        c = np.cos(ang).astype(np.float32)[None, :]
        sn = np.sin(ang).astype(np.float32)[None, :]
        v0 = out[t, :, :half].copy()
        v1 = out[t, :, half:rotary_dim].copy()
        out[t, :, :half] = v0 * c - v1 * sn
        out[t, :, half:rotary_dim] = v1 * c + v0 * sn
    return out


# ---------------------------------------------------------------------------------------------- SDPA
def sdpa_case():
    """tests/test_ops_oracle.cpp:797-817: seq 8, 24 q / 4 kv heads, head_dim 256, mt19937(47) U(-0.5,0.5)."""
    nq, nkv = 8 * 24 * 256, 8 * 4 * 256
    s = mt_stream(47, -0.5, 0.5, nq + 2 * nkv)
    Q = s[:nq].reshape(8, 24, 256)
    K = s[nq:nq + nkv].reshape(8, 4, 256)
    V = s[nq + nkv:].reshape(8, 4, 256)
    return Q, K, V, s


def sdpa_expected(Q, K, V, start_pos=0):
    """tests/test_ops_oracle.cpp:819-864: fp64 dot and weighted sum, float scores / exp / weights; query i sees
    keys 0 .. start_pos + i of K, V (which hold start_pos + len(Q) positions)."""
    T, hq, hd = Q.shape
    hkv = K.shape[1]
    ratio = hq // hkv
    scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    out = np.zeros((T, hq, hd), np.float32)
    for i in range(T):
        n = start_pos + i + 1
        for h in range(hq):
            kv = h // ratio
            dots = K[:n, kv, :].astype(np.float64) @ Q[i, h, :].astype(np.float64)
            s = (dots * np.float64(scale)).astype(np.float32)
            e = np.exp(s - s.max()).astype(np.float32)
            w = (e * np.float32(1.0 / e.astype(np.float64).sum())).astype(np.float32)
            out[i, h, :] = (w.astype(np.float64) @ V[:n, kv, :].astype(np.float64)).astype(np.float32)
    return out


# ---------------------------------------------------------------------------------------------- conv1d
def conv1d_expected_chunks():
    """tests/test_decode_graph.cpp:208-284: weights (0.1, 0.2, 0.3, 0.4) per channel, zero state; a call with one
    row of 1.0, then a call with rows 2.0 and 3.0.  Returns [(input rows, expected outputs, expected state)]."""
    def silu(v):
        v = np.float32(v)
        return np.float32(v / (np.float32(1.0) + np.exp(-v)))
    return [
        ([1.0], [silu(0.4)], [0.0, 0.0, 1.0]),
        ([2.0, 3.0], [silu(np.float32(0.3) * 1 + np.float32(0.4) * 2), silu(np.float32(0.2) * 1 + np.float32(0.3) * 2 + np.float32(0.4) * 3)],
         [1.0, 2.0, 3.0]),
    ]
