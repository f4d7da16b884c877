"""CPU suite: the oracle against every golden vector and known answer the reference's tests hold."""
import ctypes
import os

import numpy as np
import pytest

import oracle
from conftest import fill_scales, fill_weights, synth_linear


def _maxabs(a, b):
    return float(np.max(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64))))


def test_unpack_int4_forms_agree_and_match_definition():
    packed = np.arange(256, dtype=np.uint8).repeat(4).reshape(16, 64)
    a = oracle.unpack_int4(packed)
    b = oracle.unpack_int4(packed, shift_form=True)
    assert np.array_equal(a, b)
    lo = (packed & 0xF).astype(np.int8)
    lo = np.where(lo >= 8, lo - 16, lo)
    hi = (packed >> 4).astype(np.int8)
    hi = np.where(hi >= 8, hi - 16, hi)
    assert np.array_equal(a[:, 0::2], lo) and np.array_equal(a[:, 1::2], hi)
    assert a.min() == -8 and a.max() == 7


def test_quantize_roundtrip_matches_converter_rules():
    rng = np.random.default_rng(3)
    w = rng.normal(0, 0.05, size=(8, 256)).astype(np.float32)
    packed, scales = oracle.quantize_int4(w)
    q = oracle.unpack_int4(packed).astype(np.float32)
    s = np.maximum(np.abs(w).reshape(8, 2, 128).max(-1) / 7.0, 1e-8).astype(np.float32)
    assert np.array_equal(scales, s.astype(np.float16))
    qq = np.clip(np.rint(w.reshape(8, 2, 128) / s[..., None]), -8, 7).reshape(8, 256)
    assert np.array_equal(q, qq)


def test_linear_golden_m2_k5120_n2048(golden):
    arrays, meta = golden
    m = meta["lin"]
    W = fill_weights(m["N"] * m["K"] // 2, *m["w_fill"]).reshape(m["N"], m["K"] // 2)
    S = fill_scales(m["N"] * (m["K"] // 128)).reshape(m["N"], m["K"] // 128)
    X = arrays["lin_X"]
    assert np.array_equal(oracle.linear_int4_f64(X, W, S), arrays["lin_Y"])
    # the reference's own device-side oracle (linear_int4_naive) must pass the reference's tolerance
    assert _maxabs(oracle.linear_int4_naive_f32(X, W, S), arrays["lin_Y"]) <= m["tol_abs"]
    assert _maxabs(oracle.linear_int4_grouped_f32(X, W, S), arrays["lin_Y"]) <= m["tol_abs"]


def test_linear_golden_splitk_n48(golden):
    arrays, meta = golden
    m = meta["splitk"]
    W = fill_weights(m["N"] * m["K"] // 2, *m["w_fill"]).reshape(m["N"], m["K"] // 2)
    S = fill_scales(m["N"] * (m["K"] // 128)).reshape(m["N"], m["K"] // 128)
    assert np.array_equal(oracle.linear_int4_f64(arrays["splitk_X"], W, S), arrays["splitk_Y"])
    assert _maxabs(oracle.linear_int4_grouped_f32(arrays["splitk_X"], W, S), arrays["splitk_Y"]) <= m["tol_abs"]


def test_linear_golden_fused_and_swiglu_and_half(golden):
    arrays, meta = golden
    K = meta["fused"]["K"]
    for p, n in enumerate(meta["fused"]["N"]):
        W = fill_weights(n * K // 2, p + 3, p + 7).reshape(n, K // 2)
        S = fill_scales(n * (K // 128), shift=p).reshape(n, K // 128)
        assert np.array_equal(oracle.linear_int4_f64(arrays["fused_X"], W, S), arrays[f"fused_Y{p}"])
    N = meta["swiglu"]["N"]
    Wg = fill_weights(N * K // 2, 2, 5).reshape(N, K // 2)
    Wu = fill_weights(N * K // 2, 4, 9).reshape(N, K // 2)
    Sg = fill_scales(N * (K // 128)).reshape(N, K // 128)
    Su = fill_scales(N * (K // 128), base=0.020, shift=3).reshape(N, K // 128)
    assert np.array_equal(oracle.mlp_gate_up_swiglu_f64(arrays["swiglu_X"], Wg, Sg, Wu, Su), arrays["swiglu_Y"])
    Xh = arrays["half_X"]
    assert Xh.dtype == np.float16
    W = fill_weights(N * K // 2, 2, 5).reshape(N, K // 2)
    S = fill_scales(N * (K // 128)).reshape(N, K // 128)
    assert np.array_equal(oracle.linear_int4_f64(Xh.astype(np.float32), W, S), arrays["half_Y"])


def test_golden_inputs_are_the_mt19937_stream(golden):
    """The committed activations are std::mt19937(46) through libstdc++'s uniform_real_distribution:
    float(u32) * 2^-32 (clamped below 1) mapped to [-1, 1).  numpy's legacy RandomState seeds the same
    generator, so the stream can be regenerated without the C++ helper."""
    arrays, _ = golden
    raw = np.random.RandomState(46).randint(0, 2**32, size=2 * 5120, dtype=np.uint64).astype(np.uint32)
    u = raw.astype(np.float32) * np.float32(2.0 ** -32)
    u = np.where(u >= 1.0, np.nextafter(np.float32(1.0), np.float32(0.0)), u).astype(np.float32)
    x = u * np.float32(2.0) + np.float32(-1.0)
    assert np.array_equal(x.reshape(2, 5120), arrays["lin_X"])


def test_argmax_golden_and_ties(golden):
    _, meta = golden
    a = meta["argmax"]
    raw = np.random.RandomState(a["seed"]).randint(0, 2**32, size=a["vocab"], dtype=np.uint64).astype(np.uint32)
    u = raw.astype(np.float32) * np.float32(2.0 ** -32)
    u = np.where(u >= 1.0, np.nextafter(np.float32(1.0), np.float32(0.0)), u).astype(np.float32)
    logits = (u * np.float32(200.0) + np.float32(-100.0)).astype(np.float32)
    logits[a["planted"]] = 999.0
    assert f"{oracle.crc64(logits.tobytes()):016x}" == a["logits_crc64"]
    assert oracle.argmax(logits) == a["expected"] == 123456
    # ties: lowest index wins (strict '>' in src/ops/sampling.cpp:60-64, 80-83)
    t = np.zeros(1000, np.float32)
    t[[700, 300, 999]] = 5.0
    assert oracle.argmax(t) == 300
    assert oracle.argmax(np.zeros(1, np.float32)) == 0
    assert oracle.argmax(np.full(513, -np.inf, np.float32)) == 0


def test_accept_reject_scenarios(golden):
    _, meta = golden
    acc = meta["accept"]
    tl = np.full((4, acc["vocab"]), -10.0, np.float32)
    for i, t in enumerate(acc["argmax_tokens"]):
        tl[i, t] = 10.0
    for name, s in acc["scenarios"].items():
        got = oracle.speculative_accept_reject(
            np.array(s["draft"], np.int64), tl,
            None if "draft_probs" not in s else np.array(s["draft_probs"], np.float32),
            None if "rand_uniform" not in s else np.array(s["rand_uniform"], np.float32))
        assert got == s["expected"], name
    # the reference test's own assertions (tests/test_speculative_mtp.cpp:104-185)
    A, B, Cc, D = (acc["scenarios"][k]["expected"] for k in "ABCD")
    assert not A["has_rejected_token"] and A["num_accepted"] == 4 and A["num_rejected"] == 0 and A["num_remaining"] == 0
    assert A["bonus_or_resampled_token"] == 300
    assert B["num_accepted"] == 2 and B["num_rejected"] == 1 and B["num_remaining"] == 1
    assert B["bonus_or_resampled_token"] == 200 and B["rejected_token"] == 999
    assert Cc["num_accepted"] == 0 and Cc["num_rejected"] == 1 and Cc["num_remaining"] == 3
    assert D["num_accepted"] == 4
    # empty / invalid input -> default struct with bonus -1 (src/ops/sampling.cpp:102-104)
    e = oracle.speculative_accept_reject(np.zeros(0, np.int64), tl)
    assert e["bonus_or_resampled_token"] == -1 and e["num_accepted"] == 0


def test_accept_reject_stochastic_rules():
    V = 64
    rng = np.random.default_rng(5)
    tl = rng.normal(0, 2, size=(3, V)).astype(np.float32)
    am = [int(np.argmax(tl[i])) for i in range(3)]
    p = [oracle.token_prob_f32(tl[i], am[i]) for i in range(3)]
    # r below the ratio accepts, r above rejects and the replacement is the target argmax
    r = oracle.speculative_accept_reject(np.array(am, np.int64), tl, np.array([1.0, 1.0, 1.0], np.float32),
                                         np.array([p[0] * 0.5, p[1] * 1.5, 0.0], np.float32))
    assert r["num_accepted"] == 1 and r["rejected_token"] == am[1] and r["bonus_or_resampled_token"] == am[1]
    # p_draft <= 0 falls back to the greedy rule; missing uniforms mean r = 0
    r = oracle.speculative_accept_reject(np.array(am, np.int64), tl, np.array([0.0, -1.0, 0.5], np.float32), None)
    assert r["num_accepted"] == 3
    # out-of-range draft token has p_target = 0 and is rejected for any r >= 0
    r = oracle.speculative_accept_reject(np.array([V + 5], np.int64), tl[:1], np.array([0.5], np.float32),
                                         np.array([0.0], np.float32))
    assert r["num_accepted"] == 0 and r["num_remaining"] == 0
    assert abs(oracle.token_prob_f32(tl[0], am[0]) - oracle.token_prob_f64(tl[0], am[0])) < 1e-6
    sm = oracle.softmax(tl)
    assert np.allclose(sm.sum(-1), 1.0, atol=1e-5) and abs(sm[0, am[0]] - p[0]) < 1e-6


def test_crc64_known_answers_and_reference_build(golden, tmp_path):
    _, meta = golden
    for text, want in meta["crc64"].items():
        assert f"{oracle.crc64(text.encode()):016x}" == want
    assert meta["crc64"]["123456789"] == "995dc9bbdf1939fa"
    assert oracle.crc64(b"") == 0
    ref = oracle.reference_crc_lib()
    if ref is None:
        pytest.skip("reference tree absent and oracle/_ref not prebuilt")
    rng = np.random.default_rng(11)
    for n in (1, 7, 8, 255, 4096, 100003):
        data = rng.integers(0, 256, size=n, dtype=np.uint8).tobytes()
        buf = ctypes.create_string_buffer(data, n)
        assert ref.xinfer_crc64(ctypes.cast(buf, ctypes.c_void_p), n) == oracle.crc64(data)
    f = tmp_path / "blob.bin"
    data = rng.integers(0, 256, size=70001, dtype=np.uint8).tobytes()
    f.write_bytes(data)
    assert ref.xinfer_crc64_file(str(f).encode(), 0) == oracle.crc64(data)
    assert ref.xinfer_crc64_file(str(f).encode(), 1000) == oracle.crc64(data[:1000])


def test_philox_known_answers(golden):
    _, meta = golden
    for kat in meta["philox4x32_10"]:
        assert oracle.philox4x32_10(kat["ctr"], kat["key"]) == kat["out"]
    # Random123 known-answer vectors for Philox4x32-10
    assert oracle.philox4x32_10([0] * 4, [0] * 2) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert oracle.philox4x32_10([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    u = oracle.philox_uniform(10001, seed=1234, subsequence=7)
    assert u.min() >= 0.0 and u.max() < 1.0 and abs(float(u.mean()) - 0.5) < 0.02
    assert np.array_equal(u[:5], oracle.philox_uniform(5, seed=1234, subsequence=7))


def test_oracle_variants_agree_on_benchmark_distribution():
    X, W, S, q = synth_linear(4, 1024, 96, seed=0)
    assert np.array_equal(oracle.unpack_int4(W), q)
    ref = oracle.linear_int4_f64(X.astype(np.float32), W, S)
    # independent numpy restatement of the same sum
    deq = q.astype(np.float64).reshape(96, 8, 128) * S.astype(np.float64)[..., None]
    want = X.astype(np.float64) @ deq.reshape(96, 1024).T
    assert np.allclose(ref, want, rtol=1e-6, atol=1e-7)
    for fn in (oracle.linear_int4_naive_f32, oracle.linear_int4_grouped_f32):
        got = fn(X.astype(np.float32), W, S)
        assert np.max(np.abs(got - ref)) <= 1e-3 * np.sqrt(np.mean(ref ** 2))
    b = np.linspace(-1, 1, 96).astype(np.float32)
    assert np.allclose(oracle.linear_int4_f64(X.astype(np.float32), W, S, b), ref + b, atol=1e-6)
