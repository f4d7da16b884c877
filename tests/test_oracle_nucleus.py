"""CPU checks of the oracle's nucleus (top-p) restatement: the properties the definition promises, on small rows where
they can be verified by sorting."""
import numpy as np

from oracle.model import _order_key, accept_reject_top_p, nucleus, sample_token_top_p


def brute_nucleus(logits, inv_t, top_p):
    """Sort by scaled logit, take tokens until the integer weights reach ceil(top_p * Z), then add the ties."""
    import math
    s = (np.asarray(logits, np.float32) * np.float32(inv_t)).astype(np.float32)
    e = np.exp((s - s.max()).astype(np.float32)).astype(np.float32)
    w = np.rint(e.astype(np.float64) * 2.0 ** 32).astype(np.uint64)
    z = int(w.sum())
    target = min(z, max(1, int(math.ceil(float(np.float32(top_p)) * z))))
    order = np.argsort(-s, kind="stable")
    cum, thr = 0, None
    for i in order:
        cum += int(w[i])
        thr = s[i]
        if cum >= target:
            break
    members = s >= thr
    return members, int(w[members].sum()), w


def test_order_key_is_monotone():
    x = np.array([-np.inf, -3.5, -1e-30, -0.0, 0.0, 1e-30, 2.0, 7.25, np.inf], np.float32)
    k = _order_key(x).astype(np.int64)
    assert all(k[i] <= k[i + 1] for i in range(len(k) - 1))
    assert k[1] < k[2] < k[3] and k[4] < k[5] < k[6] < k[7]


def test_nucleus_matches_a_sort():
    rng = np.random.default_rng(0)
    for trial in range(30):
        v = int(rng.integers(5, 3000))
        logits = (rng.standard_normal(v) * rng.uniform(0.2, 6.0)).astype(np.float32)
        if trial % 3 == 0:   # heavy ties
            logits = np.round(logits * 2) / 2
        for top_p in (0.05, 0.5, 0.9, 0.999, 1.0):
            inv_t = float(rng.uniform(0.5, 2.0))
            key, w, thr, z = nucleus(logits, inv_t, top_p)
            members, z_b, w_b = brute_nucleus(logits, inv_t, top_p)
            assert np.array_equal(w, w_b)
            assert np.array_equal(key >= np.uint32(thr), members), (trial, top_p)
            assert z == z_b
            assert z >= float(np.float32(top_p)) * int(w.sum()) - 1   # the nucleus holds at least top_p of the weight


def test_sampling_walks_the_nucleus_in_index_order():
    rng = np.random.default_rng(1)
    logits = (rng.standard_normal(500) * 2).astype(np.float32)
    key, w, thr, z = nucleus(logits, 1.0, 0.7)
    member = key >= np.uint32(thr)
    ids = np.flatnonzero(member)
    assert sample_token_top_p(logits, 1.0, 0.7, 0.0)[0] == ids[0]
    assert sample_token_top_p(logits, 1.0, 0.7, np.float32(1.0) - np.float32(2.0 ** -24))[0] == ids[-1]
    # frequencies follow the renormalised weights
    n = 4000
    us = (np.arange(n) + 0.5) / n
    toks = np.array([sample_token_top_p(logits, 1.0, 0.7, u)[0] for u in us])
    assert member[toks].all()
    freq = np.bincount(toks, minlength=500) / n
    p = np.where(member, w.astype(np.float64), 0.0) / z
    assert np.abs(freq - p).max() < 2.0 / n + 1e-9
    tok, prob = sample_token_top_p(logits, 1.0, 0.7, 0.3)
    assert abs(prob - p[tok]) <= 1e-6 * p[tok]
    # a tiny top_p is the arg-max with probability one
    tok, prob = sample_token_top_p(logits, 1.0, 1e-6, 0.9)
    assert tok == int(np.argmax(logits)) and prob == 1.0


def test_accept_rule_inside_the_nucleus():
    rng = np.random.default_rng(2)
    v = 400
    rows = (rng.standard_normal((3, v)) * 3).astype(np.float32)
    am = [int(np.argmax(r)) for r in rows]
    key, w, thr, z = nucleus(rows[1], 1.0, 0.6)
    outside = int(np.flatnonzero(key < np.uint32(thr))[0])
    inside = int(np.flatnonzero((key >= np.uint32(thr)) & (np.arange(v) != am[1]))[0])
    p_in = float(w[inside]) / z
    # a token outside the target's nucleus has probability zero there: always rejected (the reference's r = 0 shortcut only
    # covers the arg-max token), the replacement is the target's arg-max
    r = accept_reject_top_p([am[0], outside, am[2]], rows, [0.5, 0.5, 0.5], [0.0, 0.0, 0.0], 1.0, 0.6)
    assert r["num_accepted"] == 1 and r["has_rejected_token"] and r["rejected_token"] == outside
    assert r["bonus_or_resampled_token"] == am[1]
    # a token inside it is accepted iff r < p_target / p_draft
    ok = accept_reject_top_p([am[0], inside, am[2]], rows, [0.5, p_in, 0.5], [0.0, 0.99, 0.0], 1.0, 0.6)
    assert ok["num_accepted"] == 3 and not ok["has_rejected_token"]
    no = accept_reject_top_p([am[0], inside, am[2]], rows, [0.5, min(1.0, 4 * p_in), 0.5], [0.0, 0.5, 0.0], 1.0, 0.6)
    assert no["num_accepted"] == 1 and no["rejected_token"] == inside
    # p_draft <= 0 falls back to the greedy rule
    g = accept_reject_top_p([am[0], am[1], 5], rows, [0.0, -1.0, 0.0], [0.3, 0.3, 0.3], 1.0, 0.6)
    assert g["num_accepted"] == (3 if am[2] == 5 else 2)
