"""GPU parity of the per-layer mixers and of the whole speculative step against the CPU oracle.

The decoder is created with a reduced shape (the kernels are the production ones; only extents shrink),
its random weights and synthetic context are copied to the host, and the oracle replays the same step
sequence by sequence.  Integer results (draft tokens, accepted counts, emitted tokens, context lengths)
must match exactly; fp16 hidden states within a few fp16 roundings of the oracle (the two sides round
identical fp32 values at every fp16 boundary except where their fp32 sums differ in the last bits)."""
import numpy as np
import pytest
import torch

import oracle
from oracle.model import OracleLayer, OracleModel

pytestmark = pytest.mark.gpu

FULL_NAMES = {"q_proj.w": np.uint8, "q_proj.s": np.float16, "k_proj.w": np.uint8, "k_proj.s": np.float16,
              "v_proj.w": np.uint8, "v_proj.s": np.float16, "o_proj.w": np.uint8, "o_proj.s": np.float16,
              "q_norm": np.float32, "k_norm": np.float32}
GDN_NAMES = {"in_qkv.w": np.uint8, "in_qkv.s": np.float16, "in_z.w": np.uint8, "in_z.s": np.float16,
             "in_b.w": np.uint8, "in_b.s": np.float16, "in_a.w": np.uint8, "in_a.s": np.float16,
             "out_proj.w": np.uint8, "out_proj.s": np.float16, "conv_w": np.float32, "A_log": np.float32,
             "dt_bias": np.float32, "gdn_norm": np.float32}
COMMON = {"input_norm": np.float32, "post_norm": np.float32, "gate.w": np.uint8, "gate.s": np.float16,
          "up.w": np.uint8, "up.s": np.float16, "down.w": np.uint8, "down.s": np.float16}


def lin_shape(name, shape_cfg, full):
    s = shape_cfg
    H, F = s.hidden_size, s.intermediate_size
    dims = {"gate": (F, H), "up": (F, H), "down": (H, F), "q_proj": (s.num_attention_heads * 512, H),
            "k_proj": (s.num_key_value_heads * 256, H), "v_proj": (s.num_key_value_heads * 256, H),
            "o_proj": (H, s.num_attention_heads * 256), "in_qkv": (s.conv_channels, H),
            "in_z": (s.linear_num_v_heads * 128, H), "in_b": (s.linear_num_v_heads, H),
            "in_a": (s.linear_num_v_heads, H), "out_proj": (H, s.linear_num_v_heads * 128),
            "lm_head": (s.vocab_size, H), "mtp_fc": (H, 2 * H)}
    base, kind = name.rsplit(".", 1)
    n, k = dims[base]
    return (n, k // 2) if kind == "w" else (n, k // 128)


def pull_layer(dec, idx, shape_cfg):
    full = dec.is_full(idx)
    names = dict(COMMON)
    names.update(FULL_NAMES if full else GDN_NAMES)
    w = {}
    for n, dt in names.items():
        arr = dec.tensor(idx, n, dt)
        if n.endswith(".w") or n.endswith(".s"):
            arr = arr.reshape(lin_shape(n, shape_cfg, full))
        if n == "conv_w":
            arr = arr.reshape(shape_cfg.conv_channels, 4)
        w[n] = arr
    return OracleLayer(full, w)


def pull_model(dec, shape_cfg, k):
    L = shape_cfg.num_hidden_layers
    layers = [pull_layer(dec, i, shape_cfg) for i in range(L)]
    mtp = pull_layer(dec, L, shape_cfg)
    top = {"embed": dec.tensor(-1, "embed", np.uint16).reshape(shape_cfg.vocab_size, shape_cfg.hidden_size)}
    for n in ("final_norm", "mtp_enorm", "mtp_hnorm"):
        top[n] = dec.tensor(-1, n, np.float32)
    for n in ("lm_head", "mtp_fc"):
        top[n + ".w"] = dec.tensor(-1, n + ".w", np.uint8).reshape(lin_shape(n + ".w", shape_cfg, True))
        top[n + ".s"] = dec.tensor(-1, n + ".s", np.float16).reshape(lin_shape(n + ".s", shape_cfg, True))
    return OracleModel(shape_cfg, layers, mtp, top, k)


def pull_state(dec, model, shape_cfg, batch, max_seq):
    s = shape_cfg
    ctx = dec.tensor(-1, "ctx", np.int32)
    cur = dec.tensor(-1, "cur_tok", np.int64)
    h_last = dec.tensor(-1, "h_last", np.float16).reshape(batch, s.hidden_size)
    seqs = []
    per_layer = []
    for i in range(s.num_hidden_layers + 1):
        if dec.is_full(i):
            kc = dec.tensor(i, "k_cache", np.float16).reshape(batch, max_seq, s.num_key_value_heads, 256)
            vc = dec.tensor(i, "v_cache", np.float16).reshape(batch, max_seq, s.num_key_value_heads, 256)
            per_layer.append(("full", kc, vc))
        else:
            S = dec.tensor(i, "S", np.float32).reshape(batch, s.linear_num_v_heads, 128, 128)
            cs = dec.tensor(i, "conv_state", np.float32).reshape(batch, 3, s.conv_channels)
            per_layer.append(("gdn", S, cs))
    for b in range(batch):
        layers = []
        for kind, a0, a1 in per_layer[:-1]:
            if kind == "full":
                layers.append({"k_cache": np.ascontiguousarray(a0[b]), "v_cache": np.ascontiguousarray(a1[b])})
            else:
                layers.append({"S": np.ascontiguousarray(a0[b]), "conv_state": np.ascontiguousarray(a1[b])})
        _, kc, vc = per_layer[-1]
        seqs.append({"ctx": int(ctx[b]), "cur_tok": int(cur[b]), "h_last": h_last[b].copy(), "layers": layers,
                     "mtp": {"k_cache": np.ascontiguousarray(kc[b]), "v_cache": np.ascontiguousarray(vc[b])}})
    return seqs


def rel_rms(got, ref):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.sqrt(np.mean((got - ref) ** 2)) / (np.sqrt(np.mean(ref ** 2)) + 1e-30))


@pytest.fixture(scope="module")
def small():
    from xinfer_b200.spec import Shape, SpecDecoder
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    shape_cfg = Shape(hidden_size=1024, intermediate_size=2048, num_hidden_layers=4, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=4096, linear_num_v_heads=6, linear_num_k_heads=2)
    dec = SpecDecoder(shape_cfg, batch=2, k=3, max_seq=96, seed=5)
    yield dec, shape_cfg
    dec.close()


def compare_step(dec, model, seqs, shape_cfg, overrides=None, tag=""):
    B, k = dec.batch, dec.k
    dec.override_drafts(None if overrides is None else np.array(overrides, np.int64))
    dec.step()
    emitted, counts = dec.results()
    x_gpu = dec.tensor(-1, "x", np.float16).reshape(B, k + 1, shape_cfg.hidden_size)
    logits_gpu = dec.tensor(-1, "logits", np.float32).reshape(B, k + 1, shape_cfg.vocab_size)
    ctx_gpu = dec.tensor(-1, "ctx", np.int32)
    accepted = []
    for b in range(B):
        want, dbg = model.step(seqs[b], None if overrides is None else overrides[b])
        assert rel_rms(x_gpu[b], dbg["hidden"]) < 2e-2, (tag, b)
        assert rel_rms(logits_gpu[b], dbg["logits"]) < 2e-2, (tag, b)
        assert counts[b] == len(want) and emitted[b, :counts[b]].tolist() == want, (tag, b, emitted[b], want)
        assert (emitted[b, counts[b]:] == -1).all()
        assert ctx_gpu[b] == seqs[b]["ctx"], (tag, b)
        accepted.append(dbg["num_accepted"])
    dec.override_drafts(None)
    return accepted


@pytest.mark.parametrize("ctx0", [0, 37])
def test_speculative_steps_match_oracle(small, ctx0):
    """Plain steps: the MTP head drafts, the target verifies; every integer result equals the oracle's."""
    dec, shape_cfg = small
    dec.reset(ctx0, seed=ctx0 + 1)
    model = pull_model(dec, shape_cfg, dec.k)
    seqs = pull_state(dec, model, shape_cfg, dec.batch, dec.max_seq)
    for step in range(3):
        drafts_gpu_before = None
        compare_step(dec, model, seqs, shape_cfg, tag=f"plain{step}")
    assert dec.info(2) > 0


def test_acceptance_paths_and_lazy_state_commit(small):
    """Random weights almost never accept, so the drafts are overridden with the target's own greedy
    continuation (all accepted), then with a corrupted copy (partial acceptance).  Each following step
    replays the accepted recurrent updates of the one before; the tokens can only keep matching the
    oracle (which restores and recomputes its state) if that lazy commit is exact."""
    dec, shape_cfg = small
    B, k = dec.batch, dec.k
    dec.reset(25, seed=4)
    model = pull_model(dec, shape_cfg, k)
    seqs = pull_state(dec, model, shape_cfg, B, dec.max_seq)
    plans = [(k, k), (1, 2), (0, k), (2, 0), (k, 1)]  # accepted drafts wanted per sequence, per step
    for step, plan in enumerate(plans):
        overrides = []
        for b in range(B):
            cont = model.greedy_continuation(seqs[b], k)
            keep = plan[b]
            if keep < k:
                cont[keep] = (cont[keep] + 1 + b) % shape_cfg.vocab_size  # first wrong draft at index `keep`
            overrides.append(cont)
        accepted = compare_step(dec, model, seqs, shape_cfg, overrides, tag=f"forced{step}")
        assert accepted == list(plan), (step, accepted, plan)
    # two plain steps afterwards still agree
    for step in range(2):
        compare_step(dec, model, seqs, shape_cfg, tag=f"after{step}")


def test_long_context_attention_splits():
    """Context 2048 (the reduced-stack configuration's length): 65 key chunks over 8 splits."""
    from xinfer_b200.spec import Shape, SpecDecoder
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    shape_cfg = Shape(hidden_size=512, intermediate_size=1024, num_hidden_layers=4, num_attention_heads=12,
                      num_key_value_heads=2, vocab_size=2048, linear_num_v_heads=3, linear_num_k_heads=1)
    dec = SpecDecoder(shape_cfg, batch=1, k=3, max_seq=2100, seed=11)
    dec.reset(2048, seed=2)
    model = pull_model(dec, shape_cfg, dec.k)
    seqs = pull_state(dec, model, shape_cfg, dec.batch, dec.max_seq)
    compare_step(dec, model, seqs, shape_cfg, tag="long0")
    cont = model.greedy_continuation(seqs[0], 3)
    compare_step(dec, model, seqs, shape_cfg, [cont], tag="long1")
    dec.close()


def test_prefill_from_a_prompt_then_steps(small):
    """A prompt of 11 tokens per sequence (chunks of 4, 4 and 2 rows through the target, every row kept) builds the
    context from the empty state; the oracle does the same sequence by sequence; then speculative steps must emit the
    same tokens on both sides, with forced full acceptance first (which reads the MTP head's prompt slots)."""
    dec, shape_cfg = small
    B, k = dec.batch, dec.k
    dec.reset(0, seed=9)
    model = pull_model(dec, shape_cfg, k)
    seqs = pull_state(dec, model, shape_cfg, B, dec.max_seq)
    assert all(s["ctx"] == 0 for s in seqs)
    prompt = np.random.default_rng(4).integers(0, shape_cfg.vocab_size, size=(B, 11)).astype(np.int64)
    dec.prefill(prompt)
    for b in range(B):
        model.prefill(seqs[b], prompt[b])
    assert dec.tensor(-1, "ctx", np.int32).tolist() == [10] * B
    assert dec.tensor(-1, "cur_tok", np.int64).tolist() == prompt[:, -1].tolist()
    h_gpu = dec.tensor(-1, "h_last", np.float16).reshape(B, shape_cfg.hidden_size)
    for b in range(B):
        assert rel_rms(h_gpu[b], seqs[b]["h_last"]) < 2e-2
    cont = [model.greedy_continuation(seqs[b], k) for b in range(B)]
    compare_step(dec, model, seqs, shape_cfg, cont, tag="prefill-accept-all")
    compare_step(dec, model, seqs, shape_cfg, None, tag="prefill-free")
    compare_step(dec, model, seqs, shape_cfg, None, tag="prefill-free2")
    # a second prefill without a reset is refused
    from xinfer_b200 import _lib
    with pytest.raises(_lib.XInferError):
        dec.prefill(prompt)
    dec.reset(30, seed=3)   # leave the shared decoder as the other tests expect it


@pytest.mark.parametrize("batch,k", [(1, 1), (3, 2), (2, 4), (6, 4), (5, 1)])
def test_other_batch_and_draft_counts(batch, k):
    """The step at draft counts and batch sizes other than the benchmark's (k = 1, 2, 4; odd batches; 30 verify
    rows): a free step, a step with every draft forced to the target's own continuation (k accepted), one with the
    first draft wrong, against the oracle."""
    from xinfer_b200.spec import Shape, SpecDecoder
    shape_cfg = Shape(hidden_size=1024, intermediate_size=2048, num_hidden_layers=4, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=4096, linear_num_v_heads=6, linear_num_k_heads=2)
    dec = SpecDecoder(shape_cfg, batch=batch, k=k, max_seq=96, seed=11)
    dec.reset(17, seed=2)
    model = pull_model(dec, shape_cfg, k)
    seqs = pull_state(dec, model, shape_cfg, batch, dec.max_seq)
    compare_step(dec, model, seqs, shape_cfg, None, tag="free")
    cont = [model.greedy_continuation(seqs[b], k) for b in range(batch)]
    acc = compare_step(dec, model, seqs, shape_cfg, cont, tag="accept-all")
    assert acc == [k] * batch
    cont = [model.greedy_continuation(seqs[b], k) for b in range(batch)]
    for b in range(batch):
        cont[b][0] = (cont[b][0] + 1) % shape_cfg.vocab_size
    acc = compare_step(dec, model, seqs, shape_cfg, cont, tag="reject-first")
    assert acc == [0] * batch
    compare_step(dec, model, seqs, shape_cfg, None, tag="free-after")
    dec.close()


def test_generate_loop_against_the_oracle():
    """xinfer_spec_decoder_generate against the oracle's restatement of the reference's generate loop: a prompt of 11
    tokens per sequence, then tokens until max_new_tokens ("length") or a stop token ("stop", not returned).  Run
    eagerly, from the captured graph (the first step after a prefill whose last chunk is short must run eagerly), and
    with a stop token that ends sequence 0 early while sequence 1 runs on with lane 0 parked."""
    import copy
    from xinfer_b200 import _lib
    from xinfer_b200.spec import Shape, SpecDecoder
    shape_cfg = Shape(hidden_size=1024, intermediate_size=2048, num_hidden_layers=4, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=4096 + 512, linear_num_v_heads=6, linear_num_k_heads=2)
    B, k, T, cap = 2, 3, 11, 9
    dec = SpecDecoder(shape_cfg, batch=B, k=k, max_seq=96, seed=5)
    dec.reset(0, seed=9)
    model = pull_model(dec, shape_cfg, k)
    seqs0 = pull_state(dec, model, shape_cfg, B, dec.max_seq)
    prompt = np.random.default_rng(8).integers(0, shape_cfg.vocab_size, size=(B, T)).astype(np.int64)
    want = [model.generate(copy.deepcopy(seqs0[b]), prompt[b], cap) for b in range(B)]
    assert all(f == "length" and len(t) == cap for t, f in want)

    def check(results, expect):
        for b in range(B):
            assert results[b].token_ids == expect[b][0], (b, results[b].token_ids, expect[b][0])
            assert results[b].finish_reason == expect[b][1] and results[b].generated_tokens == len(expect[b][0])
            assert results[b].prompt_tokens == T

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        got = dec.generate(prompt, max_new_tokens=cap, seed=9)
        check(got, want)
        assert got[0].steps >= 3 and got[0].total_time_sec > 0 and got[0].decode_tokens_per_sec > 0
        dec.reset(20, seed=3)
        dec.capture(stream)
        assert dec.info(3) == 1
        check(dec.generate(prompt, max_new_tokens=cap, seed=9), want)
        # a stop token: the fifth token of sequence 0
        eos = want[0][0][4]
        want_eos = [model.generate(copy.deepcopy(seqs0[b]), prompt[b], cap, eos_token_id=eos) for b in range(B)]
        assert want_eos[0][1] == "stop" and len(want_eos[0][0]) <= 4
        check(dec.generate(prompt, max_new_tokens=cap, eos_token_id=eos, seed=9), want_eos)
        check(dec.generate(prompt, max_new_tokens=cap, im_end_token_id=eos, seed=9), want_eos)
        # the reference's argument checks
        for bad in ({"max_new_tokens": 0}, {"temperature": -1.0}, {"top_p": 0.9}, {"max_new_tokens": 96}):
            with pytest.raises(_lib.XInferError):
                dec.generate(prompt, **bad)
        # a changed sampling mode is refused once the step is captured
        with pytest.raises(_lib.XInferError):
            dec.generate(prompt, max_new_tokens=cap, temperature=0.7)
    dec.close()


def test_long_prompt_prefill_runs_in_chunks():
    """A prompt of 278 tokens per sequence, batch 2: the first chunk is 256 positions x 2 sequences = 512 rows (the
    projections run on the prefill GEMM), the second 21 positions (42 rows, 32-row slices of the decode kernel); the
    mixers take both four positions at a time.  Context, current token and last hidden state against the oracle's
    sequential prefill, then speculative steps must emit the oracle's tokens (forced full acceptance first, which
    reads the MTP head's cache slots that the prefill wrote)."""
    from xinfer_b200.spec import Shape, SpecDecoder
    shape_cfg = Shape(hidden_size=1024, intermediate_size=2048, num_hidden_layers=4, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=4096, linear_num_v_heads=6, linear_num_k_heads=2)
    import xinfer_b200.ops as ops
    B, k, T = 2, 3, 278
    dec = SpecDecoder(shape_cfg, batch=B, k=k, max_seq=400, seed=21)
    # (a prompt whose last chunk is 160 rows as well: the last projection of the prefill ran on the GEMM)
    dec.reset(0, seed=4)
    dec.prefill(np.random.default_rng(5).integers(0, shape_cfg.vocab_size, size=(B, 1 + 256 + 80)).astype(np.int64))
    assert ops.last_linear_path() == 3
    dec.reset(0, seed=4)
    model = pull_model(dec, shape_cfg, k)
    seqs = pull_state(dec, model, shape_cfg, B, dec.max_seq)
    prompt = np.random.default_rng(6).integers(0, shape_cfg.vocab_size, size=(B, T)).astype(np.int64)
    dec.prefill(prompt)
    for b in range(B):
        model.prefill(seqs[b], prompt[b])
    assert dec.tensor(-1, "ctx", np.int32).tolist() == [T - 1] * B
    assert dec.tensor(-1, "cur_tok", np.int64).tolist() == prompt[:, -1].tolist()
    h_gpu = dec.tensor(-1, "h_last", np.float16).reshape(B, shape_cfg.hidden_size)
    for b in range(B):
        assert rel_rms(h_gpu[b], seqs[b]["h_last"]) < 2e-2
    cont = [model.greedy_continuation(seqs[b], k) for b in range(B)]
    compare_step(dec, model, seqs, shape_cfg, cont, tag="chunked-accept-all")
    compare_step(dec, model, seqs, shape_cfg, None, tag="chunked-free")
    compare_step(dec, model, seqs, shape_cfg, None, tag="chunked-free2")
    dec.close()


def test_stochastic_drafting_and_acceptance_inside_the_step():
    """temperature 0.7: the step draws its draft tokens from the head's distribution and applies the reference's
    stochastic rule with Philox uniforms of (seed, step index); the oracle regenerates the same uniforms, samples with
    the same two-level sums and applies the literal rule.  Tokens, counts and contexts must agree over several steps,
    eagerly and from the captured graph (whose replays must draw fresh numbers)."""
    from xinfer_b200.spec import Shape, SpecDecoder
    shape_cfg = Shape(hidden_size=1024, intermediate_size=2048, num_hidden_layers=4, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=4096 + 512, linear_num_v_heads=6, linear_num_k_heads=2)
    B, k, T, seed = 2, 3, 0.7, 1234
    inv_t = float(np.float32(1.0) / np.float32(T))
    for graph in (False, True):
        dec = SpecDecoder(shape_cfg, batch=B, k=k, max_seq=96, seed=5)
        dec.set_sampling(T, seed)
        dec.reset(20, seed=3)
        model = pull_model(dec, shape_cfg, k)
        seqs = pull_state(dec, model, shape_cfg, B, dec.max_seq)
        stream = torch.cuda.Stream()
        accepted_total = 0
        with torch.cuda.stream(stream):
            for step in range(5):
                if graph and step == 0:
                    dec.capture(stream)       # runs step 0 eagerly, records the graph
                else:
                    dec.step()
                emitted, counts = dec.results()
                u = oracle.philox_uniform(2 * B * k, seed, step)
                for b in range(B):
                    samp = {"inv_t": inv_t, "u_draft": u[b * k:(b + 1) * k], "u_accept": u[B * k + b * k:B * k + (b + 1) * k]}
                    want, dbg = model.step(seqs[b], None, samp)
                    assert counts[b] == len(want) and emitted[b, :counts[b]].tolist() == want, (graph, step, b, emitted[b], want)
                    accepted_total += dbg["num_accepted"]
                assert dec.tensor(-1, "ctx", np.int32).tolist() == [s["ctx"] for s in seqs]
        assert accepted_total > 0   # (random weights: about a third of the drafts survive the stochastic rule at T = 0.7)
        dec.close()


def test_graph_replay_equals_eager(small):
    dec, shape_cfg = small
    B, k = dec.batch, dec.k
    from xinfer_b200.spec import SpecDecoder
    eager = SpecDecoder(shape_cfg, batch=B, k=k, max_seq=dec.max_seq, seed=5)
    graph = SpecDecoder(shape_cfg, batch=B, k=k, max_seq=dec.max_seq, seed=5)
    eager.reset(30, seed=3)
    graph.reset(30, seed=3)
    stream = torch.cuda.Stream()
    outs_e, outs_g = [], []
    with torch.cuda.stream(stream):
        eager.step()  # the capture runs one eager step first; mirror it
        outs_e.append(eager.results())
        graph.capture(stream)
        outs_g.append(graph.results())
        assert graph.info(3) == 1
        for _ in range(3):
            eager.step()
            outs_e.append(eager.results())
            graph.step()
            outs_g.append(graph.results())
    for (ee, ce), (eg, cg) in zip(outs_e, outs_g):
        assert np.array_equal(ee, eg) and np.array_equal(ce, cg)
    eager.close()
    graph.close()


def test_reduced_stack_at_full_layer_shapes():
    """The reduced-stack configuration with the 27B layer shapes (8 layers = 6 Gated-DeltaNet + 2 GQA 24q/4kv,
    hidden 5120, FFN 17408, k=3, batch 1, context 2048): every projection runs through the decomposition it
    gets in the benchmark (cluster split-K, fused 3- and 4-way launches, SwiGLU pairs), LM head at the full
    vocabulary of 151936."""
    from xinfer_b200.spec import Shape, SpecDecoder
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    shape_cfg = Shape(hidden_size=5120, intermediate_size=17408, num_hidden_layers=8, num_attention_heads=24,
                      num_key_value_heads=4, vocab_size=151936, linear_num_v_heads=48, linear_num_k_heads=16)
    dec = SpecDecoder(shape_cfg, batch=1, k=3, max_seq=2100, seed=21)
    dec.reset(2048, seed=7)
    model = pull_model(dec, shape_cfg, dec.k)
    seqs = pull_state(dec, model, shape_cfg, dec.batch, dec.max_seq)
    compare_step(dec, model, seqs, shape_cfg, tag="cfg3-plain")
    cont = model.greedy_continuation(seqs[0], 3)
    accepted = compare_step(dec, model, seqs, shape_cfg, [cont], tag="cfg3-accept-all")
    assert accepted == [3]
    compare_step(dec, model, seqs, shape_cfg, tag="cfg3-after")
    dec.close()


def test_batch8_context8192_at_full_layer_shapes():
    """The benchmark's extents for the mixers: batch 8, context 8192, k = 3 (32 verify rows, the 9-split attention
    grid over 8 sequences, the DeltaNet grid over 8 x 48 heads), on a 2-layer stack (one Gated-DeltaNet, one GQA
    layer) at the 27B layer shapes.  Hidden rows are bounded per row by their largest element, not by an RMS
    over the tensor; tokens, counts and context lengths must match exactly."""
    from xinfer_b200.spec import Shape, SpecDecoder
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    shape_cfg = Shape(hidden_size=5120, intermediate_size=17408, num_hidden_layers=2, num_attention_heads=24,
                      num_key_value_heads=4, vocab_size=8192, linear_num_v_heads=48, linear_num_k_heads=16,
                      full_attention_interval=2)
    B, k = 8, 3
    dec = SpecDecoder(shape_cfg, batch=B, k=k, max_seq=8192 + 64, seed=33)
    dec.reset(8192, seed=9)
    model = pull_model(dec, shape_cfg, k)
    seqs = pull_state(dec, model, shape_cfg, B, dec.max_seq)
    for step in range(2):
        dec.step()
        emitted, counts = dec.results()
        x_gpu = dec.tensor(-1, "x", np.float16).reshape(B, k + 1, shape_cfg.hidden_size).astype(np.float64)
        ctx_gpu = dec.tensor(-1, "ctx", np.int32)
        worst = 0.0
        for b in range(B):
            want, dbg = model.step(seqs[b])
            ref = dbg["hidden"].astype(np.float64)
            per_row = np.abs(x_gpu[b] - ref).max(axis=1) / np.abs(ref).max(axis=1)
            worst = max(worst, float(per_row.max()))
            assert counts[b] == len(want) and emitted[b, :counts[b]].tolist() == want, (step, b)
            assert ctx_gpu[b] == seqs[b]["ctx"]
        assert worst < 1e-2, worst     # a few fp16 roundings of the row's largest element
    dec.close()


def test_step_refuses_to_run_past_the_cache(small):
    """The context lengths advance on the device; the host keeps an upper bound and returns an error instead of
    letting a step drop its newest keys (the reference's KV cache throws when full)."""
    from xinfer_b200 import _lib
    dec, _ = small
    k = dec.k
    room = 3
    dec.reset(dec.max_seq - (room + 2) * (k + 1), seed=1)     # reset itself needs two steps of headroom
    for _ in range(room + 2):
        dec.step()
    torch.cuda.synchronize()
    with pytest.raises(_lib.XInferError) as e:
        dec.step()
    assert e.value.code == _lib.ERR_INVALID_ARGUMENT
    dec.reset(0, seed=1)
    dec.step()                                                # usable again after a reset
    dec.results()


def test_nucleus_sampling_inside_the_step():
    """temperature 0.7 and top_p 0.8: draft tokens come from the head's nucleus, the rule takes the target's probability
    inside the target row's nucleus; the oracle regenerates the uniforms and restates both with the same integer
    weights.  Tokens, counts and contexts must agree, eagerly and from the captured graph, and through generate."""
    import copy
    from xinfer_b200.spec import Shape, SpecDecoder
    shape_cfg = Shape(hidden_size=1024, intermediate_size=2048, num_hidden_layers=4, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=4096 + 512, linear_num_v_heads=6, linear_num_k_heads=2)
    B, k, T, top_p, seed = 2, 3, 0.7, 0.8, 4321
    inv_t = float(np.float32(1.0) / np.float32(T))
    for graph in (False, True):
        dec = SpecDecoder(shape_cfg, batch=B, k=k, max_seq=96, seed=5)
        dec.set_sampling(T, seed)
        dec.set_top_p(top_p)
        dec.reset(20, seed=3)
        model = pull_model(dec, shape_cfg, k)
        seqs = pull_state(dec, model, shape_cfg, B, dec.max_seq)
        stream = torch.cuda.Stream()
        accepted_total = 0
        with torch.cuda.stream(stream):
            for step in range(5):
                if graph and step == 0:
                    dec.capture(stream)
                else:
                    dec.step()
                emitted, counts = dec.results()
                u = oracle.philox_uniform(2 * B * k, seed, step)
                for b in range(B):
                    samp = {"inv_t": inv_t, "top_p": top_p, "u_draft": u[b * k:(b + 1) * k],
                            "u_accept": u[B * k + b * k:B * k + (b + 1) * k]}
                    want, dbg = model.step(seqs[b], None, samp)
                    assert counts[b] == len(want) and emitted[b, :counts[b]].tolist() == want, (graph, step, b, emitted[b], want)
                    accepted_total += dbg["num_accepted"]
        assert accepted_total > 0
        from xinfer_b200 import _lib
        with pytest.raises(_lib.XInferError):
            dec.set_top_p(0.0)
        if graph:
            with pytest.raises(_lib.XInferError):
                dec.set_top_p(0.5)          # refused once the step is captured
        else:
            # generate refuses top_p < 1 without a temperature, and takes it with one
            prompt = np.random.default_rng(2).integers(0, shape_cfg.vocab_size, size=(B, 7)).astype(np.int64)
            with torch.cuda.stream(stream):
                with pytest.raises(_lib.XInferError):
                    dec.generate(prompt, max_new_tokens=6, top_p=0.9)
                out = dec.generate(prompt, max_new_tokens=6, temperature=T, top_p=0.9, seed=7)
            assert all(r.generated_tokens == 6 and r.finish_reason == "length" for r in out)
        dec.close()

