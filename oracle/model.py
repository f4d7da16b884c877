"""CPU oracle of the speculative step, sequence by sequence, token by token (test infrastructure).

A literal composition of the reference's per-layer forward (src/targets/qwen3_8/forward.cpp:96-308)
from the oracle's restatements of its kernels, plus the pieces the reference does not have and this
repository defines: the MTP draft head and the (k+1)-row verify / accept / commit step.  Rejected
tokens are handled the slow, obviously-correct way: recurrent state is restored from a copy taken before
the verify pass and the accepted tokens are run again.
"""
from __future__ import annotations

import numpy as np

import oracle


class OracleLayer:
    def __init__(self, full, w):
        self.full = full
        self.w = w  # dict name -> numpy array


def linear16(x16, W, S):
    """fp16 activations -> fp16 output through the fp64-accumulate linear oracle."""
    return oracle.linear_int4_f64(np.asarray(x16, np.float16).astype(np.float32), W, S).astype(np.float16)


def sample_token(logits, inv_t, u):
    """One token from softmax(logits * inv_t) by inverting the cumulative distribution at u * Z, with the two-level
    summation of the device kernel (chunks of 4096 logits in chunk order; inside the chosen chunk groups of sixteen
    consecutive logits in group order, then the group's own running sum), all in fp32.  Returns (token, probability)."""
    f32 = np.float32
    l = np.asarray(logits, f32) * f32(inv_t)
    V = l.size
    nch = (V + 4095) // 4096
    ms = np.array([l[c * 4096:(c + 1) * 4096].max() for c in range(nch)], f32)
    se = np.array([np.exp(l[c * 4096:(c + 1) * 4096] - ms[c]).astype(f32).sum(dtype=f32) for c in range(nch)], f32)
    m = f32(ms.max())
    wts = (se * np.exp(ms - m).astype(f32)).astype(f32)
    z = f32(0)
    for x in wts:
        z = f32(z + x)
    target = f32(f32(u) * z)
    before, pick = f32(0), nch - 1
    for c in range(nch):
        if f32(before + wts[c]) > target:
            pick = c
            break
        if c + 1 < nch:
            before = f32(before + wts[c])
    rest = f32(target - before)
    lo, hi = pick * 4096, min(V, (pick + 1) * 4096)
    e = np.zeros(4096, f32)
    e[:hi - lo] = np.exp(l[lo:hi] - m).astype(f32)
    local = np.zeros(256, f32)
    for t in range(256):
        acc = f32(0)
        for j in range(16):
            acc = f32(acc + e[t * 16 + j])
        local[t] = acc
    last = (hi - lo - 1) // 16
    prefix, th = f32(0), 0
    for t in range(last + 1):
        th = t
        if f32(prefix + local[t]) > rest or t == last:
            break
        prefix = f32(prefix + local[t])
    cum, tok = prefix, -1
    for j in range(16):
        if lo + th * 16 + j < hi:
            tok = j
            cum = f32(cum + e[th * 16 + j])
            if cum > rest:
                break
    return lo + th * 16 + tok, float(f32(e[th * 16 + tok] / z))


def _order_key(s32):
    """Order-preserving uint32 key of float32 values (negative: all bits flipped; else the sign bit set)."""
    u = np.ascontiguousarray(s32, np.float32).view(np.uint32)
    return np.where(u & np.uint32(0x80000000), ~u, u | np.uint32(0x80000000)).astype(np.uint32)


def nucleus(logits, inv_t, top_p):
    """The nucleus of softmax(logits * inv_t) at top_p with the device kernel's integer weights
    w = rn(exp(s - max) * 2^32), s = logits * inv_t in fp32: the smallest set of highest-s tokens whose weights reach
    ceil(top_p * Z), all tokens tied with the threshold included.  Returns (keys, weights, threshold key, Z_nucleus)."""
    import math
    f32 = np.float32
    s = (np.asarray(logits, f32) * f32(inv_t)).astype(f32)
    ms = f32(s.max())
    e = np.exp((s - ms).astype(f32)).astype(f32)
    w = np.rint(e.astype(np.float64) * 4294967296.0).astype(np.uint64)
    key = _order_key(s)
    z = int(w.sum(dtype=np.uint64))
    want = math.ceil(float(f32(top_p)) * float(z))
    target = min(z, 1 if want <= 1 else int(want))
    uk, inv = np.unique(key, return_inverse=True)
    sums = np.zeros(len(uk), np.uint64)
    np.add.at(sums, inv, w)
    cum = 0
    thr = int(uk[0])
    for i in range(len(uk) - 1, -1, -1):
        cum += int(sums[i])
        thr = int(uk[i])
        if cum >= target:
            break
    return key, w, thr, cum


def sample_token_top_p(logits, inv_t, top_p, u):
    """One token from the nucleus: the first token, in index order, at which the running nucleus weight exceeds
    floor(u * Z_nucleus).  Returns (token, probability inside the nucleus)."""
    import math
    key, w, thr, z = nucleus(logits, inv_t, top_p)
    t2 = min(z - 1, max(0, int(math.floor(float(np.float32(u)) * float(z)))))
    member = key >= np.uint32(thr)
    cum = np.cumsum(np.where(member, w, np.uint64(0)).astype(np.uint64), dtype=np.uint64)
    tok = int(np.argmax(member & (cum > np.uint64(t2))))
    return tok, float(np.float32(float(w[tok]) / float(z)))


def accept_reject_top_p(drafts, logits_rows, draft_probs, uniforms, inv_t, top_p):
    """The reference's stochastic rule (src/ops/sampling.cpp:129-171) with the target's probability taken inside
    the target row's own nucleus (zero outside it); same result fields as oracle.speculative_accept_reject."""
    f32 = np.float32
    n = len(drafts)
    res = {"num_accepted": 0, "has_rejected_token": False, "bonus_or_resampled_token": -1, "rejected_token": -1}
    for i in range(n):
        t = oracle.argmax(logits_rows[i])
        d = int(drafts[i])
        p_draft, rr = f32(draft_probs[i]), f32(uniforms[i])
        if p_draft <= 0:
            ok = d == t
        elif d == t and rr <= 0:
            ok = True
        else:
            key, w, thr, z = nucleus(logits_rows[i], inv_t, top_p)
            p_target = f32(0)
            if 0 <= d < len(key) and z > 0 and int(key[d]) >= thr:
                p_target = f32(float(w[d]) / float(z))
            ok = bool(rr < f32(p_target / p_draft))
        if ok:
            res["num_accepted"] += 1
        else:
            res.update(has_rejected_token=True, rejected_token=d, bonus_or_resampled_token=t)
            return res
    return res


class OracleModel:
    def __init__(self, shape, layers, mtp_layer, top, k):
        self.s, self.layers, self.mtp_layer, self.top, self.k = shape, layers, mtp_layer, top, k

    # one sequence: x [T, H] fp16, positions start_pos .. start_pos + T - 1
    def forward_layer(self, L, x, start_pos, st):
        s = self.s
        w = L.w
        T = x.shape[0]
        normed = oracle.rmsnorm_f16(x, w["input_norm"], s.rms_norm_eps)
        if L.full:
            hq, hkv = s.num_attention_heads, s.num_key_value_heads
            q_gate = linear16(normed, w["q_proj.w"], w["q_proj.s"])
            kk = linear16(normed, w["k_proj.w"], w["k_proj.s"])
            vv = linear16(normed, w["v_proj.w"], w["v_proj.s"])
            q = oracle.split_q(q_gate, hq, 256)
            q = oracle.rmsnorm_f16(q.reshape(T * hq, 256), w["q_norm"], s.rms_norm_eps).reshape(T, hq, 256)
            kk = oracle.rmsnorm_f16(kk.reshape(T * hkv, 256), w["k_norm"], s.rms_norm_eps).reshape(T, hkv, 256)
            pos = np.arange(start_pos, start_pos + T, dtype=np.int64)
            q, kk = oracle.rope_f16(q, kk, pos, s.rope_theta, s.rope_dim)
            oracle.kv_write(st["k_cache"], st["v_cache"], kk, vv.reshape(T, hkv, 256), start_pos)
            attn = oracle.sdpa_cached(q, st["k_cache"], st["v_cache"], start_pos)
            attn = oracle.gate_output(attn.reshape(T, hq, 256), q_gate, hq, 256).reshape(T, hq * 256)
            proj = linear16(attn, w["o_proj.w"], w["o_proj.s"])
        else:
            hv, hk = s.linear_num_v_heads, s.linear_num_k_heads
            qkv = linear16(normed, w["in_qkv.w"], w["in_qkv.s"])
            z = linear16(normed, w["in_z.w"], w["in_z.s"])
            b = linear16(normed, w["in_b.w"], w["in_b.s"])
            a = linear16(normed, w["in_a.w"], w["in_a.s"])
            conv = oracle.conv1d_silu(qkv, w["conv_w"], st["conv_state"])
            delta = oracle.gdn(conv, z, b, a, w["A_log"], w["dt_bias"], w["gdn_norm"], st["S"], hv, hk)
            proj = linear16(delta, w["out_proj.w"], w["out_proj.s"])
        x = oracle.add_inplace_f16(x, proj)
        normed = oracle.rmsnorm_f16(x, w["post_norm"], s.rms_norm_eps)
        act = oracle.mlp_gate_up_swiglu_f64(normed.astype(np.float32), w["gate.w"], w["gate.s"], w["up.w"],
                                            w["up.s"]).astype(np.float16)
        proj = linear16(act, w["down.w"], w["down.s"])
        return oracle.add_inplace_f16(x, proj)

    def target(self, tokens, start_pos, seq_state):
        x = oracle.embed(self.top["embed"], tokens, self.s.vocab_size)
        for L, st in zip(self.layers, seq_state["layers"]):
            x = self.forward_layer(L, x, start_pos, st)
        normed = oracle.rmsnorm_f16(x, self.top["final_norm"], self.s.rms_norm_eps)
        logits = oracle.linear_int4_f64(normed.astype(np.float32), self.top["lm_head.w"], self.top["lm_head.s"])
        return x, logits

    def draft(self, tok, h_prev, pos, seq_state):
        e = oracle.embed(self.top["embed"], [tok], self.s.vocab_size)
        cat = np.concatenate([oracle.rmsnorm_f16(e, self.top["mtp_enorm"], self.s.rms_norm_eps),
                              oracle.rmsnorm_f16(h_prev[None], self.top["mtp_hnorm"], self.s.rms_norm_eps)], axis=1)
        x = linear16(cat, self.top["mtp_fc.w"], self.top["mtp_fc.s"])
        x = self.forward_layer(self.mtp_layer, x, pos, seq_state["mtp"])
        normed = oracle.rmsnorm_f16(x, self.top["final_norm"], self.s.rms_norm_eps)
        logits = oracle.linear_int4_f64(normed.astype(np.float32), self.top["lm_head.w"], self.top["lm_head.s"])
        return x[0], logits[0]

    def draft_fill(self, tok, h_prev, pos, seq_state):
        """The head's pass for `tok` at `pos` up to its attention layer's KV write (no attention, MLP or logits):
        fills the slot the next step's first draft pass attends to when all k drafts are accepted."""
        s = self.s
        w = self.mtp_layer.w
        e = oracle.embed(self.top["embed"], [tok], s.vocab_size)
        cat = np.concatenate([oracle.rmsnorm_f16(e, self.top["mtp_enorm"], s.rms_norm_eps),
                              oracle.rmsnorm_f16(h_prev[None], self.top["mtp_hnorm"], s.rms_norm_eps)], axis=1)
        x = linear16(cat, self.top["mtp_fc.w"], self.top["mtp_fc.s"])
        normed = oracle.rmsnorm_f16(x, w["input_norm"], s.rms_norm_eps)
        hkv = s.num_key_value_heads
        kk = linear16(normed, w["k_proj.w"], w["k_proj.s"])
        vv = linear16(normed, w["v_proj.w"], w["v_proj.s"])
        kk = oracle.rmsnorm_f16(kk.reshape(hkv, 256), w["k_norm"], s.rms_norm_eps).reshape(1, hkv, 256)
        _, kk = oracle.rope_f16(np.zeros((1, 1, 256), np.float16), kk, np.array([pos], np.int64), s.rope_theta, s.rope_dim)
        st = seq_state["mtp"]
        oracle.kv_write(st["k_cache"], st["v_cache"], kk, vv.reshape(1, hkv, 256), pos)

    def prefill(self, seq_state, tokens):
        """Builds the context of one sequence from a prompt, starting from the empty state: positions 0 .. T-2 go
        through the target (every row kept), the head's KV slot of position p is filled from (token p, hidden state of
        position p - 1; zeros in front of position 0), the last prompt token becomes the current token."""
        tokens = [int(t) for t in tokens]
        assert seq_state["ctx"] == 0 and len(tokens) >= 1
        h_prev = np.zeros(self.s.hidden_size, np.float16)
        R = self.k + 1
        body = tokens[:-1]
        pos = 0
        while pos < len(body):
            chunk = body[pos:pos + R]
            x, _ = self.target(chunk, pos, seq_state)
            for i, t in enumerate(chunk):
                self.draft_fill(t, h_prev if i == 0 else x[i - 1], pos + i, seq_state)
            h_prev = x[len(chunk) - 1]
            pos += len(chunk)
        seq_state["ctx"] = len(body)
        seq_state["cur_tok"] = tokens[-1]
        seq_state["h_last"] = h_prev.copy()

    def generate(self, seq_state, prompt, max_new_tokens, eos_token_id=-1, im_end_token_id=-1, max_seq=None):
        """The speculative generate loop of one sequence (src/runtime/engine.cpp:400-525) over (k+1)-row steps:
        prefill, then steps; a stop token ends the sequence and is not returned ("stop"), max_new_tokens tokens end
        it with "length" (tokens a step emits beyond that are dropped), and so does a full cache.
        Returns (token ids, finish reason)."""
        self.prefill(seq_state, prompt)
        out, finish = [], "length"
        while len(out) < max_new_tokens:
            if max_seq is not None and seq_state["ctx"] + self.k + 1 > max_seq:
                break
            emitted, _ = self.step(seq_state)
            done = False
            for t in emitted:
                if (eos_token_id >= 0 and t == eos_token_id) or (im_end_token_id >= 0 and t == im_end_token_id):
                    finish, done = "stop", True
                    break
                out.append(int(t))
                if len(out) == max_new_tokens:
                    done = True
                    break
            if done:
                break
        return out, finish

    def greedy_continuation(self, seq_state, n):
        """The n tokens the target itself would emit after cur_tok (state is left untouched)."""
        import copy
        st = copy.deepcopy(seq_state)
        toks, tok = [], st["cur_tok"]
        for i in range(n):
            _, lg = self.target([tok], st["ctx"] + i, st)
            tok = oracle.argmax(lg[0])
            toks.append(tok)
        return toks

    def step(self, seq_state, draft_override=None, sampling=None):
        """One speculative step of one sequence.  Returns (emitted tokens, debug dict).  `sampling` = dict(inv_t, u_draft[k],
        u_accept[k]): draft tokens drawn from softmax(head logits * inv_t), the reference's stochastic accept rule."""
        k = self.k
        ctx = seq_state["ctx"]
        tok, h = seq_state["cur_tok"], seq_state["h_last"]
        drafts = []
        draft_probs = []
        draft_logits = []
        for i in range(k):
            h, lg = self.draft(tok, h, ctx + i, seq_state)
            if sampling is None:
                tok = oracle.argmax(lg)
            else:
                if sampling.get("top_p", 1.0) < 1.0:
                    tok, p = sample_token_top_p(lg, sampling["inv_t"], sampling["top_p"], sampling["u_draft"][i])
                else:
                    tok, p = sample_token(lg, sampling["inv_t"], sampling["u_draft"][i])
                draft_probs.append(p)
            drafts.append(tok)
            draft_logits.append(lg)
        mtp_drafts = list(drafts)
        self.draft_fill(tok, h, ctx + k, seq_state)
        if draft_override is not None:
            drafts = [int(t) for t in draft_override]
        # verify: save recurrent state, run k+1 rows
        saved = [{n: (v.copy() if n in ("S", "conv_state") else v) for n, v in st.items()} for st in seq_state["layers"]]
        tokens = [seq_state["cur_tok"]] + drafts
        x, logits = self.target(tokens, ctx, seq_state)
        if sampling is None or draft_override is not None:
            res = oracle.speculative_accept_reject(np.array(drafts, np.int64), logits[:k])
        elif sampling.get("top_p", 1.0) < 1.0:
            res = accept_reject_top_p(drafts, logits[:k], np.array(draft_probs, np.float32),
                                      np.array(sampling["u_accept"], np.float32), float(sampling["inv_t"]), sampling["top_p"])
        else:
            res = oracle.speculative_accept_reject(np.array(drafts, np.int64), logits[:k], np.array(draft_probs, np.float32),
                                                   np.array(sampling["u_accept"], np.float32),
                                                   inv_temperature=float(sampling["inv_t"]))
        na = res["num_accepted"]
        bonus = res["bonus_or_resampled_token"] if res["has_rejected_token"] else oracle.argmax(logits[k])
        if na < k:  # roll the recurrent state back and run the accepted prefix again
            for st, sv in zip(seq_state["layers"], saved):
                for n in ("S", "conv_state"):
                    if n in st:
                        st[n][...] = sv[n]
            self.target(tokens[:na + 1], ctx, seq_state)
        seq_state["ctx"] = ctx + na + 1
        seq_state["cur_tok"] = bonus
        seq_state["h_last"] = x[na]
        return drafts[:na] + [bonus], {"drafts": drafts, "logits": logits, "hidden": x, "num_accepted": na,
                                       "draft_logits": draft_logits, "mtp_drafts": mtp_drafts}
