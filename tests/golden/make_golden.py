"""Regenerates tests/golden/ref_vectors.npz and ref_vectors.json.

Inputs follow the reference's own test recipes (tests/test_ops_oracle.cpp:290-792 for the linear
family, :911-947 for argmax, tests/test_speculative_mtp.cpp:83-189 for acceptance); expected outputs
come from the CPU oracle in oracle/, which restates the inline oracles of those tests.  The
reference stores no output files, so these arrays are the pinned form of "what its tests expect".

Run from the repository root:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402


def mt_uniform(seed: int, lo: float, hi: float, n: int) -> np.ndarray:
    with tempfile.TemporaryDirectory() as td:
        exe = os.path.join(td, "mt_uniform")
        subprocess.check_call(["g++", "-O2", "-o", exe, os.path.join(HERE, "mt_uniform.cpp")])
        out = os.path.join(td, "o.bin")
        subprocess.check_call([exe, str(seed), repr(lo), repr(hi), str(n), out])
        return np.fromfile(out, dtype=np.float32)


def fill_weights(n_bytes: int, a: int, b: int) -> np.ndarray:
    """W[i] = ((i+a)&0xF) | (((i+b)&0xF)<<4), tests/test_ops_oracle.cpp:312-316."""
    i = np.arange(n_bytes, dtype=np.int64)
    return (((i + a) & 0xF) | (((i + b) & 0xF) << 4)).astype(np.uint8)


def fill_scales(n: int, base: float = 0.015, shift: int = 0) -> np.ndarray:
    """scale[i] = half(base + ((i+shift)%10)*0.001), tests/test_ops_oracle.cpp:309-311."""
    i = np.arange(n, dtype=np.int64)
    f = np.float32(base) + ((i + shift) % 10).astype(np.float32) * np.float32(0.001)
    return f.astype(np.float32).astype(np.float16)


def main() -> None:
    arrays: dict[str, np.ndarray] = {}
    meta: dict = {}
    # One mt19937(46) stream feeds every sub-test of test_linear_oracle in order.
    n_total = 2 * 5120 + 5120 + 512 + 512 + 512
    stream = mt_uniform(46, -1.0, 1.0, n_total)
    off = 0

    def take(n):
        nonlocal off
        v = stream[off:off + n].copy()
        off += n
        return v

    # (1) M=2, K=5120, N=2048, fp32 activations, max-abs <= 1e-4  (:292-369)
    M, K, N = 2, 5120, 2048
    X = take(M * K).reshape(M, K)
    W = fill_weights(N * K // 2, 3, 7).reshape(N, K // 2)
    S = fill_scales(N * (K // 128)).reshape(N, K // 128)
    arrays["lin_X"] = X
    arrays["lin_Y"] = oracle.linear_int4_f64(X, W, S)
    meta["lin"] = {"M": M, "K": K, "N": N, "w_fill": [3, 7], "tol_abs": 1e-4}

    # (2) split-K shape M=1, K=5120, N=48, max-abs <= 1e-3  (:389-466)
    M, K, N = 1, 5120, 48
    X = take(M * K).reshape(M, K)
    W = fill_weights(N * K // 2, 5, 11).reshape(N, K // 2)
    S = fill_scales(N * (K // 128)).reshape(N, K // 128)
    arrays["splitk_X"] = X
    arrays["splitk_Y"] = oracle.linear_int4_f64(X, W, S)
    meta["splitk"] = {"M": M, "K": K, "N": N, "w_fill": [5, 11], "tol_abs": 1e-3}

    # (3) fused 4 projections N={128,64,48,48}, K=512, M=1, max-abs <= 1e-4  (:499-599)
    K = 512
    X = take(K).reshape(1, K)
    arrays["fused_X"] = X
    for p, n in enumerate([128, 64, 48, 48]):
        W = fill_weights(n * K // 2, p + 3, p + 7).reshape(n, K // 2)
        S = fill_scales(n * (K // 128), shift=p).reshape(n, K // 128)
        arrays[f"fused_Y{p}"] = oracle.linear_int4_f64(X, W, S)
    meta["fused"] = {"M": 1, "K": K, "N": [128, 64, 48, 48], "tol_abs": 1e-4}

    # (4) gate/up/SwiGLU N=256, K=512, M=1, max-abs <= 1e-4  (:604-702)
    N = 256
    X = take(K).reshape(1, K)
    Wg = fill_weights(N * K // 2, 2, 5).reshape(N, K // 2)
    Wu = fill_weights(N * K // 2, 4, 9).reshape(N, K // 2)
    Sg = fill_scales(N * (K // 128)).reshape(N, K // 128)
    Su = fill_scales(N * (K // 128), base=0.020, shift=3).reshape(N, K // 128)
    arrays["swiglu_X"] = X
    arrays["swiglu_Y"] = oracle.mlp_gate_up_swiglu_f64(X, Wg, Sg, Wu, Su)
    meta["swiglu"] = {"M": 1, "K": K, "N": N, "tol_abs": 1e-4}

    # (5) fp16 activations N=256, K=512: fp16 out <= 5e-3, fp32 out <= 1e-4  (:707-791)
    Xf = take(K).reshape(1, K)
    Xh = Xf.astype(np.float16)
    W = fill_weights(N * K // 2, 2, 5).reshape(N, K // 2)
    S = fill_scales(N * (K // 128)).reshape(N, K // 128)
    arrays["half_X"] = Xh
    arrays["half_Y"] = oracle.linear_int4_f64(Xh.astype(np.float32), W, S)
    meta["half"] = {"M": 1, "K": K, "N": N, "w_fill": [2, 5], "tol_abs_f16": 5e-3, "tol_abs_f32": 1e-4}
    assert off == n_total

    # (6) argmax over 248320 logits, mt19937(48) U(-100,100), planted 999 at 123456  (:911-947)
    V = 248320
    logits = mt_uniform(48, -100.0, 100.0, V)
    logits[123456] = np.float32(999.0)
    meta["argmax"] = {"vocab": V, "seed": 48, "planted": 123456, "expected": oracle.argmax(logits),
                      "logits_crc64": f"{oracle.crc64(logits.tobytes()):016x}"}
    assert meta["argmax"]["expected"] == 123456

    # (7) acceptance scenarios A-D, vocab 1000, N=4  (tests/test_speculative_mtp.cpp:85-189)
    tl = np.full((4, 1000), -10.0, dtype=np.float32)
    for i, t in enumerate([42, 100, 200, 300]):
        tl[i, t] = 10.0
    scen = {
        "A": {"draft": [42, 100, 200, 300]},
        "B": {"draft": [42, 100, 999, 300]},
        "C": {"draft": [999, 100, 200, 300]},
        "D": {"draft": [42, 100, 200, 300], "draft_probs": [1.0] * 4, "rand_uniform": [0.1] * 4},
    }
    for k, s in scen.items():
        s["expected"] = oracle.speculative_accept_reject(
            np.array(s["draft"], dtype=np.int64), tl,
            None if "draft_probs" not in s else np.array(s["draft_probs"], dtype=np.float32),
            None if "rand_uniform" not in s else np.array(s["rand_uniform"], dtype=np.float32))
    meta["accept"] = {"vocab": 1000, "argmax_tokens": [42, 100, 200, 300], "scenarios": scen}

    # (8) CRC-64 known answers (src/artifact/checksum.cpp:8-55), cross-checked against the
    # reference's own library when it is built under oracle/_ref.
    kat = {"123456789": f"{oracle.crc64(b'123456789'):016x}", "xinfer": f"{oracle.crc64(b'xinfer'):016x}"}
    ref = oracle.reference_crc_lib()
    if ref is not None:
        import ctypes
        for text, want in kat.items():
            buf = ctypes.create_string_buffer(text.encode(), len(text))
            got = ref.xinfer_crc64(ctypes.cast(buf, ctypes.c_void_p), len(text))
            assert f"{got:016x}" == want, (text, want, got)
        meta["crc64_checked_against_reference_build"] = True
    meta["crc64"] = kat

    # Philox4x32-10 known answers (Random123 kat_vectors)
    meta["philox4x32_10"] = [
        {"ctr": [0, 0, 0, 0], "key": [0, 0], "out": oracle.philox4x32_10([0] * 4, [0] * 2)},
        {"ctr": [0xFFFFFFFF] * 4, "key": [0xFFFFFFFF] * 2,
         "out": oracle.philox4x32_10([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2)},
        {"ctr": [0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], "key": [0xA4093822, 0x299F31D0],
         "out": oracle.philox4x32_10([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0])},
    ]

    # Input streams of the reference's mixer op tests (tests/test_ops_oracle.cpp:50-285, 797-906): regenerated at
    # test time by tests/ref_recipes.py, pinned here by length and CRC-64.
    sys.path.insert(0, os.path.dirname(HERE))
    import ref_recipes
    streams = {}
    for name, case in (("rmsnorm", ref_recipes.rmsnorm_case), ("rope", ref_recipes.rope_case), ("sdpa", ref_recipes.sdpa_case)):
        st = case()[-1]
        streams[name] = {"n": int(st.size), "crc64": f"{oracle.crc64(st.tobytes()):016x}", "first": float(st[0]),
                         "last": float(st[-1])}
    with open(os.path.join(HERE, "mixer_streams.json"), "w") as f:
        json.dump(streams, f, indent=1, sort_keys=True)

    np.savez_compressed(os.path.join(HERE, "ref_vectors.npz"), **arrays)
    with open(os.path.join(HERE, "ref_vectors.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)
    print("wrote", len(arrays), "arrays;", os.path.getsize(os.path.join(HERE, "ref_vectors.npz")), "bytes")


if __name__ == "__main__":
    main()
