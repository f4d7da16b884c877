"""GPU parity: argmax, speculative acceptance and the Philox uniform source against the CPU oracle.
Token ids and accept counts are integers: the bar is exact equality."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def mt_logits(seed, n, lo, hi):
    raw = np.random.RandomState(seed).randint(0, 2**32, size=n, dtype=np.uint64).astype(np.uint32)
    u = raw.astype(np.float32) * np.float32(2.0 ** -32)
    u = np.where(u >= 1.0, np.nextafter(np.float32(1.0), np.float32(0.0)), u).astype(np.float32)
    return (u * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


def test_argmax_reference_case(cuda, golden):
    _, meta = golden
    a = meta["argmax"]
    logits = mt_logits(a["seed"], a["vocab"], -100.0, 100.0)
    logits[a["planted"]] = 999.0
    assert f"{oracle.crc64(logits.tobytes()):016x}" == a["logits_crc64"]
    d = dev(logits)
    assert cuda.argmax(d, a["vocab"]) == a["expected"]
    # with caller scratch, as the reference allows (src/ops/sampling.h:17-25)
    n = cuda.argmax_scratch_size(a["vocab"])
    assert n == (a["vocab"] + 255) // 256
    pm = torch.empty(n, dtype=torch.float32, device="cuda")
    pi = torch.empty(n, dtype=torch.int64, device="cuda")
    assert cuda.argmax(d, a["vocab"], pm, pi) == a["expected"]


def test_argmax_edges_and_ties(cuda):
    assert cuda.argmax(None, 100) == 0
    z = dev(np.zeros(5, np.float32))
    assert cuda.argmax(z, 0) == 0 and cuda.argmax(z, -3) == 0 and cuda.argmax(z, 1) == 0
    rng = np.random.default_rng(0)
    for V in (2, 255, 256, 257, 4095, 4096, 4097, 151936):
        x = rng.normal(0, 3, V).astype(np.float32)
        assert cuda.argmax(dev(x), V) == oracle.argmax(x)
        # ties: lowest index wins, also across block boundaries
        t = np.zeros(V, np.float32)
        idx = np.unique(rng.integers(0, V, 5))
        t[idx] = 9.0
        assert cuda.argmax(dev(t), V) == int(idx.min()) == oracle.argmax(t)
    allneg = np.full(5000, -np.inf, np.float32)
    assert cuda.argmax(dev(allneg), 5000) == oracle.argmax(allneg) == 0


def test_argmax_rows_batched(cuda):
    rng = np.random.default_rng(1)
    x = rng.normal(0, 3, size=(32, 151936)).astype(np.float32)
    out = torch.empty(32, dtype=torch.int64, device="cuda")
    assert cuda.argmax_rows(dev(x), out) == 0
    torch.cuda.synchronize()
    assert out.cpu().tolist() == [oracle.argmax(r) for r in x]


def test_accept_reject_reference_scenarios(cuda, golden):
    _, meta = golden
    acc = meta["accept"]
    V = acc["vocab"]
    tl = np.full((4, V), -10.0, np.float32)
    for i, t in enumerate(acc["argmax_tokens"]):
        tl[i, t] = 10.0
    d = dev(tl)
    for name, s in acc["scenarios"].items():
        got = cuda.speculative_accept_reject(s["draft"], 4, d, V, s.get("draft_probs"), s.get("rand_uniform"))
        want = {k: v for k, v in s["expected"].items() if k != "contract_violated"}
        assert got == want, name
    empty = cuda.speculative_accept_reject([], 0, d, V)
    assert empty["bonus_or_resampled_token"] == -1 and empty["num_accepted"] == 0
    assert cuda.speculative_accept_reject([1], 1, None, V)["bonus_or_resampled_token"] == -1


def make_config2(seed, B=8, k=3, V=151936, temperature=0.7):
    """Benchmark acceptance configuration: draft logits N(0, 3), target = draft + N(0, 1)."""
    rng = np.random.default_rng(seed)
    draft = rng.normal(0, 3, size=(B, k, V)).astype(np.float32)
    target = (draft + rng.normal(0, 1, size=(B, k, V)).astype(np.float32)).astype(np.float32)
    return draft, target


def test_config2_greedy_exact(cuda):
    B, k, V = 8, 3, 151936
    draft, target = make_config2(0)
    toks = np.array([[oracle.argmax(draft[b, i]) for i in range(k)] for b in range(B)], np.int64)
    # make the outcome varied: force some draft tokens to the target's argmax
    for b in range(0, B, 2):
        toks[b, 0] = oracle.argmax(target[b, 0])
    toks[0, 1] = oracle.argmax(target[0, 1])
    toks[0, 2] = oracle.argmax(target[0, 2])
    out = torch.zeros(B * cuda.ACCEPT_RECORD_BYTES, dtype=torch.uint8, device="cuda")
    assert cuda.speculative_accept_reject_batched(dev(toks), dev(target), None, None, out) == 0
    recs = cuda.decode_accept_records(out)
    n_acc = []
    for b in range(B):
        want = oracle.speculative_accept_reject(toks[b], target[b])
        for f in ("bonus_or_resampled_token", "rejected_token", "num_accepted", "num_rejected", "num_resampled",
                  "num_remaining"):
            assert recs[b][f] == want[f], (b, f)
        assert bool(recs[b]["has_rejected_token"]) == want["has_rejected_token"]
        n_acc.append(want["num_accepted"])
        # the host-facing synchronous form agrees too
        single = cuda.speculative_accept_reject(toks[b].tolist(), k, dev(target[b]), V)
        assert single == {kk: v for kk, v in want.items() if kk != "contract_violated"}
    assert n_acc[0] == 3 and 0 in n_acc  # both outcomes are present


@pytest.mark.parametrize("seed", [0, 1])
def test_config2_stochastic_exact_with_philox_uniforms(cuda, seed):
    """Temperature 0.7, draft tokens sampled from softmax(draft / T) on the host, acceptance uniforms
    from Philox generated ON THE DEVICE and checked bit-exactly against the oracle's generator; both
    sides then see identical uniforms and must take identical decisions."""
    B, k, V, T = 8, 3, 151936, 0.7
    inv_t = np.float32(1.0 / T)
    draft, target = make_config2(seed)
    u_dev = torch.empty(B * k, dtype=torch.float32, device="cuda")
    assert cuda.philox_uniform(u_dev, seed=1000 + seed, subsequence=1) == 0
    uni = oracle.philox_uniform(B * k, seed=1000 + seed, subsequence=1)
    assert np.array_equal(u_dev.cpu().numpy(), uni)
    pick = oracle.philox_uniform(B * k, seed=1000 + seed, subsequence=0).reshape(B, k)
    toks = np.zeros((B, k), np.int64)
    probs = np.zeros((B, k), np.float32)
    for b in range(B):
        for i in range(k):
            p = oracle.softmax((draft[b, i] * inv_t)[None])[0].astype(np.float64)
            c = np.cumsum(p)
            t = int(min(np.searchsorted(c, pick[b, i] * c[-1], side="right"), V - 1))
            toks[b, i] = t
            probs[b, i] = np.float32(p[t])
    uni = uni.reshape(B, k)
    out = torch.zeros(B * cuda.ACCEPT_RECORD_BYTES, dtype=torch.uint8, device="cuda")
    assert cuda.speculative_accept_reject_batched(dev(toks), dev(target), dev(probs), dev(uni), out,
                                                  inv_temperature=float(inv_t)) == 0
    recs = cuda.decode_accept_records(out)
    accepted_total = 0
    for b in range(B):
        want = oracle.speculative_accept_reject(toks[b], target[b], probs[b], uni[b], inv_temperature=float(inv_t))
        assert not want["contract_violated"]
        for f in ("bonus_or_resampled_token", "rejected_token", "num_accepted", "num_rejected", "num_resampled",
                  "num_remaining"):
            assert recs[b][f] == want[f], (b, f)
        accepted_total += want["num_accepted"]
    assert 0 < accepted_total < B * k  # the rule is exercised in both directions


def test_stochastic_margins_and_fallback_rules(cuda):
    """p_draft <= 0 -> greedy rule; missing uniforms -> r = 0; out-of-range token -> p_target = 0."""
    V = 5000
    rng = np.random.default_rng(3)
    tl = rng.normal(0, 2, size=(3, V)).astype(np.float32)
    am = [oracle.argmax(tl[i]) for i in range(3)]
    d = dev(tl)
    cases = [
        (am, [0.0, -1.0, 0.5], None),
        ([am[0], V + 9, am[2]], [0.5, 0.5, 0.5], [0.0, 0.0, 0.0]),
        (am, [1.0, 1.0, 1.0], [0.9999, 0.0, 0.5]),
        ([7, 8, 9], [1e-6, 1e-6, 1e-6], [0.5, 0.5, 0.5]),
    ]
    for toks, probs, unif in cases:
        got = cuda.speculative_accept_reject(toks, 3, d, V, probs, unif)
        want = oracle.speculative_accept_reject(np.array(toks, np.int64), tl, np.array(probs, np.float32),
                                                None if unif is None else np.array(unif, np.float32))
        assert got == {k: v for k, v in want.items() if k != "contract_violated"}


def test_bonus_row_convention_k_plus_one(cuda):
    """With k+1 target rows per sequence the bonus token comes from row k on full acceptance."""
    B, k, V = 2, 3, 2048
    rng = np.random.default_rng(9)
    tl = rng.normal(0, 1, size=(B, k + 1, V)).astype(np.float32)
    toks = np.array([[oracle.argmax(tl[b, i]) for i in range(k)] for b in range(B)], np.int64)
    toks[1, 1] = (toks[1, 1] + 1) % V
    out = torch.zeros(B * cuda.ACCEPT_RECORD_BYTES, dtype=torch.uint8, device="cuda")
    assert cuda.speculative_accept_reject_batched(dev(toks), dev(tl), None, None, out, bonus_row=k) == 0
    recs = cuda.decode_accept_records(out)
    assert recs[0]["num_accepted"] == 3 and recs[0]["bonus_or_resampled_token"] == oracle.argmax(tl[0, k])
    assert recs[1]["num_accepted"] == 1 and recs[1]["bonus_or_resampled_token"] == oracle.argmax(tl[1, 1])
    assert recs[1]["num_remaining"] == 1


def test_philox_uniform_bit_exact(cuda):
    for n, seed, sub in [(1, 0, 0), (3, 1, 2), (4, 2**40 + 3, 2**33 + 1), (10007, 77, 5)]:
        out = torch.empty(n, dtype=torch.float32, device="cuda")
        assert cuda.philox_uniform(out, seed=seed, subsequence=sub) == 0
        assert np.array_equal(out.cpu().numpy(), oracle.philox_uniform(n, seed, sub))


def test_stochastic_margin_run_200_seeds(cuda):
    """The device sums exp() in parallel fp32, the reference sequentially on the host (src/ops/sampling.cpp:144-147),
    so p_target can differ in its last bits and a decision r < p_target / p_draft can flip only where r is within
    rounding of the ratio.  200 seeds of the acceptance configuration (batch 8, k = 3, vocab 151936, T = 0.7):
    every sequence's accepted count is compared with the literal fp32-sequential oracle; where they differ, the
    diverging decision's margin |r - ratio| / ratio (ratio from the fp64 oracle) must lie inside 1e-6.  The test
    also reports the smallest margin seen."""
    B, k, V, T = 8, 3, 151936, 0.7
    inv_t = np.float32(1.0 / T)
    flips_inside, min_margin, decisions = 0, np.inf, 0
    out = torch.zeros(B * cuda.ACCEPT_RECORD_BYTES, dtype=torch.uint8, device="cuda")
    for seed in range(200):
        rng = np.random.default_rng(50_000 + seed)
        draft = rng.normal(0, 3, size=(B, k, V)).astype(np.float32)
        target = (draft + rng.normal(0, 1, size=(B, k, V)).astype(np.float32)).astype(np.float32)
        pick = oracle.philox_uniform(B * k, seed=9000 + seed, subsequence=0).reshape(B, k)
        uni = oracle.philox_uniform(B * k, seed=9000 + seed, subsequence=1).reshape(B, k)
        z = draft.astype(np.float64) * np.float64(inv_t)
        p = np.exp(z - z.max(axis=-1, keepdims=True))
        p /= p.sum(axis=-1, keepdims=True)
        c = np.cumsum(p, axis=-1)
        toks = np.zeros((B, k), np.int64)
        for b in range(B):
            for i in range(k):
                toks[b, i] = min(int(np.searchsorted(c[b, i], pick[b, i] * c[b, i, -1], side="right")), V - 1)
        probs = np.take_along_axis(p, toks[..., None], axis=-1)[..., 0].astype(np.float32)
        assert cuda.speculative_accept_reject_batched(dev(toks), dev(target), dev(probs), dev(uni), out,
                                                      inv_temperature=float(inv_t)) == 0
        recs = cuda.decode_accept_records(out)
        for b in range(B):
            want = oracle.speculative_accept_reject(toks[b], target[b], probs[b], uni[b], inv_temperature=float(inv_t))
            na_gpu, na_cpu = recs[b]["num_accepted"], want["num_accepted"]
            last = min(max(na_gpu, na_cpu), k - 1)
            for i in range(last + 1):                 # the decisions that were actually taken
                ratio = oracle.token_prob_f64(target[b, i] * inv_t, toks[b, i]) / float(probs[b, i])
                if ratio > 0:
                    min_margin = min(min_margin, abs(float(uni[b, i]) - ratio) / ratio)
                decisions += 1
            if na_gpu != na_cpu:
                i = min(na_gpu, na_cpu)               # the decision on which the two sides part
                ratio = oracle.token_prob_f64(target[b, i] * inv_t, toks[b, i]) / float(probs[b, i])
                margin = abs(float(uni[b, i]) - ratio) / ratio
                assert margin < 1e-6, (seed, b, i, margin, na_gpu, na_cpu)
                flips_inside += 1
            else:
                assert recs[b]["bonus_or_resampled_token"] == want["bonus_or_resampled_token"], (seed, b)
    print(f"stochastic margin run: {decisions} decisions, {flips_inside} flips inside the 1e-6 band, "
          f"smallest margin {min_margin:.3e}")
    assert decisions >= 200 * B


def test_sample_tokens_against_the_oracle_sampler(cuda):
    """Draft-token sampling at the acceptance configuration's shape (8 rows, vocab 151936, T = 0.7): the kernel inverts the
    cumulative distribution with a fixed two-level fp32 summation that `oracle.model.sample_token` restates; tokens
    must be equal and probabilities within fp32 rounding for every draw of 40 seeds, the probabilities must be the
    softmax's, and the empirical distribution over a small vocabulary must follow the softmax."""
    from oracle.model import sample_token
    B, V, T = 8, 151936, 0.7
    inv_t = float(np.float32(1.0) / np.float32(T))
    mismatches = 0
    for seed in range(40):
        rng = np.random.default_rng(500 + seed)
        logits = (rng.standard_normal((B, V)) * 3).astype(np.float32)
        u = oracle.philox_uniform(B, 4000 + seed, 0)
        tok = torch.empty(B, dtype=torch.int64, device="cuda")
        prob = torch.empty(B, dtype=torch.float32, device="cuda")
        assert cuda.sample_tokens(torch.from_numpy(logits).cuda(), torch.from_numpy(u).cuda(), tok, prob, inv_t) == 0
        tok, prob = tok.cpu().numpy(), prob.cpu().numpy()
        for b in range(B):
            want_t, want_p = sample_token(logits[b], inv_t, u[b])
            mismatches += int(tok[b] != want_t)
            if tok[b] == want_t:
                assert abs(prob[b] - want_p) <= 2e-5 * want_p
            p64 = oracle.token_prob_f64(logits[b] * np.float32(inv_t), int(tok[b]))
            assert abs(prob[b] - p64) <= 1e-4 * p64
    assert mismatches == 0
    # a small vocabulary (two chunks, ragged): 20000 draws follow the softmax
    V2 = 4096 + 37
    l2 = (np.random.default_rng(1).standard_normal(V2) * 2).astype(np.float32)
    n = 20000
    u = oracle.philox_uniform(n, 77, 3)
    rows = torch.from_numpy(np.broadcast_to(l2, (n, V2)).copy()).cuda()
    tok = torch.empty(n, dtype=torch.int64, device="cuda")
    prob = torch.empty(n, dtype=torch.float32, device="cuda")
    for i in range(0, n, 500):    # (the library's sampling scratch bounds rows x chunks per call)
        assert cuda.sample_tokens(rows[i:i + 500], torch.from_numpy(u[i:i + 500]).cuda(), tok[i:i + 500], prob[i:i + 500], 1.0) == 0
    tok = tok.cpu().numpy()
    p = np.exp(l2.astype(np.float64) - l2.max())
    p /= p.sum()
    top = np.argsort(-p)[:20]
    freq = np.bincount(tok, minlength=V2) / n
    assert tok.min() >= 0 and tok.max() < V2
    assert np.all(np.abs(freq[top] - p[top]) <= 5 * np.sqrt(p[top] * (1 - p[top]) / n) + 1e-3)


def test_sample_tokens_top_p_against_the_oracle(cuda):
    """Nucleus sampling (vocab 151936, T = 0.7): integer weights make every sum exact, so token and probability must
    equal the oracle's restatement for every draw (the two sides only have to agree on exp's bits; a token whose draw
    lands within one part in 10^6 of a boundary of the oracle's cumulative weights is excused and counted).  Properties
    that need no oracle: the drawn token lies inside the nucleus, top_p = 1 reproduces the whole-distribution
    probability, a tiny top_p always returns the arg-max with probability 1, and over a small vocabulary the draws
    follow the renormalised nucleus."""
    from oracle.model import nucleus, sample_token_top_p
    B, V, T = 6, 151936, 0.7
    inv_t = float(np.float32(1.0) / np.float32(T))
    near, total = 0, 0
    for seed in range(6):
        rng = np.random.default_rng(900 + seed)
        logits = (rng.standard_normal((B, V)) * (1.0 + seed)).astype(np.float32)   # flat to peaked rows
        u = oracle.philox_uniform(B, 5000 + seed, 0)
        u[0] = 0.0
        dl, du = torch.from_numpy(logits).cuda(), torch.from_numpy(u).cuda()
        for top_p in (0.5, 0.9, 0.999, 1.0):
            tok = torch.empty(B, dtype=torch.int64, device="cuda")
            prob = torch.empty(B, dtype=torch.float32, device="cuda")
            assert cuda.sample_tokens_top_p(dl, du, tok, prob, inv_t, top_p) == 0
            tok_h, prob_h = tok.cpu().numpy(), prob.cpu().numpy()
            for b in range(B):
                key, w, thr, z = nucleus(logits[b], inv_t, top_p)
                assert int(key[tok_h[b]]) >= thr, (seed, top_p, b)
                want_t, want_p = sample_token_top_p(logits[b], inv_t, top_p, u[b])
                total += 1
                if tok_h[b] != want_t:
                    # only a draw that sits on a boundary of the cumulative weights may differ
                    member = key >= np.uint32(thr)
                    cum = np.cumsum(np.where(member, w, np.uint64(0)).astype(np.uint64), dtype=np.uint64).astype(np.float64)
                    t2 = np.floor(float(u[b]) * float(z))
                    assert np.min(np.abs(cum - t2)) <= 1e-6 * z, (seed, top_p, b, tok_h[b], want_t)
                    near += 1
                else:
                    assert abs(prob_h[b] - want_p) <= 1e-5 * want_p
                if top_p == 1.0:
                    p64 = oracle.token_prob_f64(logits[b] * np.float32(inv_t), int(tok_h[b]))
                    assert abs(prob_h[b] - p64) <= 1e-4 * p64 + 2.0 ** -32   # weights are multiples of 2^-32
    assert near <= max(1, total // 50), (near, total)
    # rows of heavily tied logits: the threshold's bucket holds far more tokens than the kernel's candidate list, so
    # the selection runs over the row itself; ties at the threshold are all inside the nucleus
    rng = np.random.default_rng(17)
    tied = np.stack([rng.integers(0, 4, V).astype(np.float32) * np.float32(0.001),
                     rng.integers(0, 3, V).astype(np.float32) * np.float32(0.25),
                     np.zeros(V, np.float32)])
    u = oracle.philox_uniform(3, 6000, 1)
    for top_p in (0.3, 0.9):
        tok = torch.empty(3, dtype=torch.int64, device="cuda")
        prob = torch.empty(3, dtype=torch.float32, device="cuda")
        assert cuda.sample_tokens_top_p(torch.from_numpy(tied).cuda(), torch.from_numpy(u).cuda(), tok, prob, 1.0, top_p) == 0
        for b in range(3):
            want_t, want_p = sample_token_top_p(tied[b], 1.0, top_p, u[b])
            assert int(tok[b]) == want_t and abs(float(prob[b]) - want_p) <= 1e-5 * want_p, (top_p, b)
    # a nucleus of one token
    logits = (np.random.default_rng(3).standard_normal((4, 9000)) * 4).astype(np.float32)
    u = oracle.philox_uniform(4, 9, 9)
    tok = torch.empty(4, dtype=torch.int64, device="cuda")
    prob = torch.empty(4, dtype=torch.float32, device="cuda")
    assert cuda.sample_tokens_top_p(torch.from_numpy(logits).cuda(), torch.from_numpy(u).cuda(), tok, prob, 1.0, 1e-6) == 0
    assert tok.cpu().numpy().tolist() == logits.argmax(axis=1).tolist() and np.allclose(prob.cpu().numpy(), 1.0)
    # distribution over a small vocabulary
    V2, n, top_p = 4096 + 37, 20000, 0.8
    l2 = (np.random.default_rng(1).standard_normal(V2) * 2).astype(np.float32)
    u = oracle.philox_uniform(n, 78, 3)
    rows = torch.from_numpy(np.broadcast_to(l2, (n, V2)).copy()).cuda()
    tok = torch.empty(n, dtype=torch.int64, device="cuda")
    prob = torch.empty(n, dtype=torch.float32, device="cuda")
    assert cuda.sample_tokens_top_p(rows, torch.from_numpy(u).cuda(), tok, prob, 1.0, top_p) == 0
    tok = tok.cpu().numpy()
    key, w, thr, z = nucleus(l2, 1.0, top_p)
    member = key >= np.uint32(thr)
    assert member[tok].all()
    p = np.where(member, w.astype(np.float64), 0.0) / float(z)
    freq = np.bincount(tok, minlength=V2) / n
    for t in np.argsort(-p)[:20]:
        assert abs(freq[t] - p[t]) <= 5 * np.sqrt(p[t] * (1 - p[t]) / n) + 1e-3, (t, freq[t], p[t])
    # arguments
    from xinfer_b200 import _lib
    for bad in (0.0, 1.5, -0.1):
        with pytest.raises(_lib.XInferError):
            cuda.sample_tokens_top_p(rows[:2], torch.from_numpy(u[:2]).cuda(), torch.empty(2, dtype=torch.int64, device="cuda"),
                                     torch.empty(2, dtype=torch.float32, device="cuda"), 1.0, bad)

