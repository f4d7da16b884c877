"""GPU parity of the per-layer mixer ops, one op at a time through the C-ABI (xinfer_rmsnorm_f16, xinfer_rope_f16,
xinfer_attention_write_kv_cache_f16, xinfer_sdpa_causal_cached_f16, xinfer_causal_conv1d_silu_f16,
xinfer_recurrent_gated_delta_net_f16), on the reference's own test cases (tests/ref_recipes.py) and against the
CPU oracle on the same fp16 inputs.  The kernels are the ones the speculative step launches."""
import numpy as np
import pytest
import torch

import oracle
import ref_recipes as rr

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def half_ulp(x):
    ax = np.maximum(np.abs(np.asarray(x, np.float64)), 2.0 ** -14)
    return 2.0 ** (np.floor(np.log2(ax)) - 11)


def within(got, want, tol_abs, ulps=1.0):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    excess = np.abs(got - want) - (tol_abs + ulps * half_ulp(want))
    assert float(excess.max()) <= 0.0, float(excess.max())


def fp16_steps_apart(a, b):
    """Largest distance between two fp16 arrays, in units of half an fp16 ulp at the value."""
    a64, b64 = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float((np.abs(a64 - b64) / half_ulp(b64)).max())


def test_rmsnorm_reference_case(cuda):
    x, w, eps, _ = rr.rmsnorm_case()
    xh = x.astype(np.float16)
    out = torch.empty((4, 5120), dtype=torch.float16, device="cuda")
    assert cuda.rmsnorm(out, dev(xh), dev(w), 4, 5120, eps) == 0
    got = host(out)
    within(got, rr.rmsnorm_expected(xh.astype(np.float32), w, eps), 1e-4)      # tests/test_ops_oracle.cpp:101
    assert fp16_steps_apart(got, oracle.rmsnorm_f16(xh, w, eps)) <= 2.0        # at most one fp16 step from the oracle


def test_rmsnorm_residual_and_ragged_width(cuda):
    rng = np.random.default_rng(1)
    for tokens, hidden in [(3, 1000), (32, 5120), (1, 8)]:
        res = rng.normal(size=(tokens, hidden)).astype(np.float16)
        inc = rng.normal(size=(tokens, hidden)).astype(np.float16)
        w = (1 + rng.normal(0, 0.02, size=hidden)).astype(np.float32)
        r_d, out = dev(res), torch.empty((tokens, hidden), dtype=torch.float16, device="cuda")
        assert cuda.rmsnorm_residual(out, r_d, dev(inc), dev(w), tokens, hidden, 1e-6) == 0
        summed = oracle.add_inplace_f16(res, inc)
        assert np.array_equal(host(r_d), summed)                                # the fp16 add is exact to the bit
        assert fp16_steps_apart(host(out), oracle.rmsnorm_f16(summed, w, 1e-6)) <= 2.0
    assert cuda.rmsnorm(out, out, dev(w), 0, 8, 1e-6) == 1                      # empty shape: no-op status


def test_rope_reference_case(cuda):
    q, k, pos, theta, rd, _ = rr.rope_case()
    qh, kh = q.astype(np.float16), k.astype(np.float16)
    q_d, k_d = dev(qh), dev(kh)
    assert cuda.rope(q_d, k_d, 4, 24, 4, 256, dev(pos), theta, rd) == 0
    within(host(q_d), rr.rope_expected(qh.astype(np.float32), pos, theta, rd), 1e-4)   # :183-184
    within(host(k_d), rr.rope_expected(kh.astype(np.float32), pos, theta, rd), 1e-4)
    oq, ok = oracle.rope_f16(qh, kh, pos, theta, rd)
    assert fp16_steps_apart(host(q_d), oq) <= 2.0 and fp16_steps_apart(host(k_d), ok) <= 2.0
    assert np.array_equal(host(q_d)[..., rd:], qh[..., rd:])                    # beyond rotary_dim: untouched


def test_kv_write_and_cached_sdpa_reference_case(cuda):
    Q, K, V, _ = rr.sdpa_case()
    Qh, Kh, Vh = Q.astype(np.float16), K.astype(np.float16), V.astype(np.float16)
    kc = torch.zeros((8, 4, 256), dtype=torch.float16, device="cuda")
    vc = torch.zeros((8, 4, 256), dtype=torch.float16, device="cuda")
    assert cuda.attention_write_kv_cache(kc, vc, dev(Kh), dev(Vh), 0, 8, 4, 256) == 0
    assert np.array_equal(host(kc), Kh) and np.array_equal(host(vc), Vh)
    out = torch.empty((8, 24, 256), dtype=torch.float16, device="cuda")
    assert cuda.sdpa_causal_cached(out, dev(Qh), kc, vc, 0, 8, 24, 4, 256, 1.0 / 16.0) == 0
    want = rr.sdpa_expected(Qh.astype(np.float32), Kh.astype(np.float32), Vh.astype(np.float32))
    within(host(out), want, 1e-3)                                               # :903, fp16 KV cache tolerance
    within(host(out), oracle.sdpa_cached(Qh, Kh, Vh, 0).astype(np.float32), 2e-4, ulps=2.0)


def test_cached_sdpa_with_a_prefix_and_bounds(cuda):
    """Row i sees keys 0 .. start_pos + i (src/ops/attention.cpp:196): 300 cached positions, 4 new rows."""
    from xinfer_b200 import _lib
    rng = np.random.default_rng(7)
    start, T, hq, hkv = 300, 4, 12, 2
    kc = (rng.normal(size=(start + T, hkv, 256)) * 0.5).astype(np.float16)
    vc = (rng.normal(size=(start + T, hkv, 256)) * 0.5).astype(np.float16)
    q = (rng.normal(size=(T, hq, 256)) * 0.5).astype(np.float16)
    out = torch.empty((T, hq, 256), dtype=torch.float16, device="cuda")
    assert cuda.sdpa_causal_cached(out, dev(q), dev(kc), dev(vc), start, T, hq, hkv, 256, 0.0, start + T) == 0
    within(host(out), oracle.sdpa_cached(q, kc, vc, start).astype(np.float32), 2e-4, ulps=2.0)
    with pytest.raises(_lib.XInferError):   # rows beyond a bounded cache are refused, not dropped
        cuda.sdpa_causal_cached(out, dev(q), dev(kc), dev(vc), start, T, hq, hkv, 256, 0.0, start + T - 1)
    with pytest.raises(_lib.XInferError):
        cuda.attention_write_kv_cache(dev(kc), dev(vc), dev(kc[:T]), dev(vc[:T]), start + 1, T, hkv, 256, start + T)


def test_kv_rollback_overwrites_in_place(cuda):
    """tests/test_kv_cache.cpp:286-314: rollback is a length change; the next write lands on the rolled-back rows."""
    rng = np.random.default_rng(0)
    a = rng.normal(size=(20, 2, 256)).astype(np.float16)
    b = rng.normal(size=(3, 2, 256)).astype(np.float16)
    kc = torch.zeros((32, 2, 256), dtype=torch.float16, device="cuda")
    vc = torch.zeros((32, 2, 256), dtype=torch.float16, device="cuda")
    cuda.attention_write_kv_cache(kc, vc, dev(a), dev(a), 0, 20, 2, 256, 32)
    cuda.attention_write_kv_cache(kc, vc, dev(b), dev(b), 15, 3, 2, 256, 32)    # after rollback(5)
    got = host(kc)
    assert np.array_equal(got[:15], a[:15]) and np.array_equal(got[15:18], b) and np.array_equal(got[18:20], a[18:20])
    assert not got[20:].any()


def test_conv1d_chunk_boundaries_reference_case(cuda):
    """tests/test_decode_graph.cpp:208-284 at the reference's 10240 channels."""
    C = 10240
    w = dev(np.tile(np.array([0.1, 0.2, 0.3, 0.4], np.float32), (C, 1)))
    state = torch.zeros((3, C), dtype=torch.float32, device="cuda")
    for rows, outs, st in rr.conv1d_expected_chunks():
        x = dev(np.repeat(np.array(rows, np.float16)[:, None], C, axis=1))
        y = torch.empty_like(x)
        assert cuda.causal_conv1d_silu(y, x, w, len(rows), state, C) == 0
        yh = host(y).astype(np.float32)
        for t, e in enumerate(outs):
            assert np.all(np.abs(yh[t] - e) < 1e-4 + 1e-3 * abs(e))
        assert np.allclose(host(state)[:, 0], st, atol=1e-4) and np.all(host(state) == host(state)[:, :1])


@pytest.mark.parametrize("seq_len", [1, 5, 8, 11, 19])
def test_conv1d_matches_oracle_across_internal_chunks(cuda, seq_len):
    rng = np.random.default_rng(seq_len)
    C = 1536
    w = rng.normal(0, 0.5, size=(C, 4)).astype(np.float32)
    st0 = rng.normal(size=(3, C)).astype(np.float32)
    x = rng.normal(size=(seq_len, C)).astype(np.float16)
    st_ref = st0.copy()
    want = oracle.conv1d_silu(x, w, st_ref)
    st_d = dev(st0)
    y = torch.empty((seq_len, C), dtype=torch.float16, device="cuda")
    assert cuda.causal_conv1d_silu(y, dev(x), dev(w), seq_len, st_d, C) == 0
    assert fp16_steps_apart(host(y), want) <= 2.0
    assert np.array_equal(host(st_d), st_ref)
    # no state: zeros for the past, nothing kept
    y2 = torch.empty_like(y)
    assert cuda.causal_conv1d_silu(y2, dev(x), dev(w), seq_len, None, C) == 0
    assert fp16_steps_apart(host(y2), oracle.conv1d_silu(x, w, None)) <= 2.0


@pytest.mark.parametrize("seq_len,zero", [(1, False), (4, True), (8, False), (13, False)])
def test_gated_delta_net_matches_oracle(cuda, seq_len, zero):
    rng = np.random.default_rng(100 + seq_len)
    hv, hk = 6, 2
    ch = 2 * hk * 128 + hv * 128
    qkv = rng.normal(size=(seq_len, ch)).astype(np.float16)
    z = rng.normal(size=(seq_len, hv * 128)).astype(np.float16)
    b = rng.normal(size=(seq_len, hv)).astype(np.float16)
    a = rng.normal(size=(seq_len, hv)).astype(np.float16)
    A_log = rng.normal(0.5, 0.5, size=hv).astype(np.float32)
    dtb = rng.normal(0, 0.5, size=hv).astype(np.float32)
    nw = (1 + rng.normal(0, 0.02, size=128)).astype(np.float32)
    S0 = (rng.normal(size=(hv, 128, 128)) * 0.05).astype(np.float32)
    S_ref = S0.copy()
    want = oracle.gdn(qkv, z, b, a, A_log, dtb, nw, S_ref, hv, hk, zero_state=zero)
    S_d = dev(S0)
    out = torch.empty((seq_len, hv * 128), dtype=torch.float16, device="cuda")
    assert cuda.recurrent_gated_delta_net(out, dev(qkv), dev(z), dev(b), dev(a), dev(A_log), dev(dtb), dev(nw), S_d,
                                          seq_len, zero, hv, hk) == 0
    got = host(out).astype(np.float64)
    ref = want.astype(np.float64)
    # fp32 sums in a different order than the oracle's: a few fp16 steps on outputs, 1e-5 relative on the state
    assert np.max(np.abs(got - ref) / (np.abs(ref) + 0.05)) < 5e-3
    assert np.max(np.abs(host(S_d) - S_ref)) <= 1e-5 * max(1.0, float(np.abs(S_ref).max()))


def test_shape_validation_like_the_reference(cuda):
    """tests/test_decode_graph.cpp:23-49: conv1d refuses num_channels <= 0, the delta rule refuses head counts it was
    not built for (here: v heads not a multiple of k heads); both before touching any pointer."""
    from xinfer_b200 import _lib
    with pytest.raises(_lib.XInferError) as e:
        cuda.causal_conv1d_silu(None, None, None, 1, None, 0)
    assert e.value.code == _lib.ERR_INVALID_ARGUMENT
    with pytest.raises(_lib.XInferError) as e:
        cuda.recurrent_gated_delta_net(None, None, None, None, None, None, None, None, None, 1, False, 32, 5)
    assert e.value.code == _lib.ERR_INVALID_ARGUMENT
