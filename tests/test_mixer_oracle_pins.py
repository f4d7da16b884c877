"""CPU suite: the oracle's restatements of the per-layer mixer ops (oracle/mixers_oracle.cpp) against the
reference's own test cases for those ops - same input streams (pinned by CRC-64), expected values recomputed
by the tests' inline fp64 recipes (tests/ref_recipes.py).  The reference's cases are fp32; the hot path (and
the oracle) is fp16, so inputs are rounded to fp16 first, the recipe runs on the rounded values, and the bound
is the reference's tolerance plus one fp16 rounding of the output."""
import numpy as np

import oracle
import ref_recipes as rr


def _half_ulp(x):
    """Half an fp16 ulp at |x| (the rounding of an exact value to fp16), elementwise."""
    ax = np.maximum(np.abs(np.asarray(x, np.float64)), 2.0 ** -14)
    return 2.0 ** (np.floor(np.log2(ax)) - 11)


def _within(got, want, tol_abs):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    excess = np.abs(got - want) - (tol_abs + _half_ulp(want))
    assert float(excess.max()) <= 0.0, float(excess.max())


def test_streams_are_the_pinned_ones():
    pins = rr.pinned_streams()
    for name, case in (("rmsnorm", rr.rmsnorm_case), ("rope", rr.rope_case), ("sdpa", rr.sdpa_case)):
        st = case()[-1]
        assert st.size == pins[name]["n"]
        assert f"{oracle.crc64(st.tobytes()):016x}" == pins[name]["crc64"], name


def test_rmsnorm_oracle_on_the_reference_case():
    x, w, eps, _ = rr.rmsnorm_case()
    xh = x.astype(np.float16)
    want = rr.rmsnorm_expected(xh.astype(np.float32), w, eps)
    _within(oracle.rmsnorm_f16(xh, w, eps), want, 1e-4)           # tests/test_ops_oracle.cpp:101 (max-abs 1e-4)


def test_rope_oracle_on_the_reference_case():
    q, k, pos, theta, rd, _ = rr.rope_case()
    qh, kh = q.astype(np.float16), k.astype(np.float16)
    gq, gk = oracle.rope_f16(qh, kh, pos, theta, rd)
    _within(gq, rr.rope_expected(qh.astype(np.float32), pos, theta, rd), 1e-4)   # :183-184
    _within(gk, rr.rope_expected(kh.astype(np.float32), pos, theta, rd), 1e-4)
    # dims beyond rotary_dim are untouched
    assert np.array_equal(gq[..., rd:], qh[..., rd:]) and np.array_equal(gk[..., rd:], kh[..., rd:])


def test_cached_sdpa_oracle_on_the_reference_case():
    Q, K, V, _ = rr.sdpa_case()
    Qh, Kh, Vh = Q.astype(np.float16), K.astype(np.float16), V.astype(np.float16)
    kc = np.zeros((8, 4, 256), np.float16)
    vc = np.zeros((8, 4, 256), np.float16)
    oracle.kv_write(kc, vc, Kh, Vh, 0)
    assert np.array_equal(kc, Kh) and np.array_equal(vc, Vh)
    got = oracle.sdpa_cached(Qh, kc, vc, 0)
    want = rr.sdpa_expected(Qh.astype(np.float32), Kh.astype(np.float32), Vh.astype(np.float32))
    _within(got, want, 1e-3)                                      # :903 (fp16 KV cache tolerance 1e-3)


def test_conv1d_oracle_chunk_boundaries():
    """tests/test_decode_graph.cpp:208-284, one channel block."""
    C = 256
    w = np.tile(np.array([0.1, 0.2, 0.3, 0.4], np.float32), (C, 1))
    state = np.zeros((3, C), np.float32)
    for rows, outs, st in rr.conv1d_expected_chunks():
        x = np.repeat(np.array(rows, np.float16)[:, None], C, axis=1)
        y = oracle.conv1d_silu(x, w, state).astype(np.float32)
        for t, e in enumerate(outs):
            assert np.all(np.abs(y[t] - e) < 1e-4 + 1e-3 * abs(e))   # 1e-4 there; fp16 output here
        assert np.allclose(state[:, 0], st, atol=1e-4) and np.all(state == state[:, :1])


def test_kv_rollback_is_a_length_change():
    """tests/test_kv_cache.cpp:286-314: rollback lowers the sequence length and nothing else; rows written past
    the new length are simply overwritten by the next write at that position."""
    kc = np.zeros((32, 2, 256), np.float16)
    vc = np.zeros((32, 2, 256), np.float16)
    rng = np.random.default_rng(0)
    a = rng.normal(size=(20, 2, 256)).astype(np.float16)
    oracle.kv_write(kc, vc, a, a, 0)
    seq_len = 20 - 5                       # rollback(5): 20 -> 15
    b = rng.normal(size=(3, 2, 256)).astype(np.float16)
    oracle.kv_write(kc, vc, b, b, seq_len)
    assert np.array_equal(kc[:15], a[:15]) and np.array_equal(kc[15:18], b) and np.array_equal(kc[18:20], a[18:20])
