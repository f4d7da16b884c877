"""`.xinfer` artifacts: this repository's writer and C-ABI reader against the format's rules and, when the
reference's own ArtifactWriter / ArtifactReader have been built (oracle/_ref, from the reference tree), against
those - a file written by the reference must read back identically here, and a file written here must pass the
reference's checksum validation and read back identically there.  The GPU part loads an INT4 projection, whole
and as the N-split shards of two ranks, and runs it (converter rules: tools/convert/qwen3_8_27b/convert.py:93-148,
restated as oracle.quantize_int4)."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import oracle
from xinfer_b200 import _lib
from xinfer_b200.artifact import TENSOR_SCALES, TENSOR_WEIGHTS, RAW_BLOB, ArtifactReader, write_artifact


def ref_lib():
    path = os.path.join(os.path.dirname(oracle.__file__), "_ref", "libxinfer_artifact_ref.so")
    if not os.path.exists(path):
        return None
    h = C.CDLL(path)
    h.ref_artifact_write.restype = C.c_int
    h.ref_artifact_read.restype = C.c_int64
    h.ref_artifact_read.argtypes = [C.c_char_p, C.c_int, C.c_char_p, C.c_void_p, C.c_uint64]
    h.ref_artifact_section_count.argtypes = [C.c_char_p]
    return h


def sample_sections(seed=0):
    rng = np.random.default_rng(seed)
    N, K = 96, 512
    w = rng.normal(0, 0.05, size=(N, K)).astype(np.float32)
    packed, scales = oracle.quantize_int4(w)
    norm = (rng.normal(0, 0.02, size=K).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)   # bf16 bits
    secs = [("model.language_model.layers.0.mlp.down_proj.weight", TENSOR_WEIGHTS, packed.tobytes()),
            ("model.language_model.layers.0.mlp.down_proj.weight.scales", TENSOR_SCALES, scales.tobytes()),
            ("model.language_model.layers.0.input_layernorm.weight", RAW_BLOB, norm.tobytes()),
            ("odd.blob", RAW_BLOB, bytes(range(200)) * 3 + b"x"),
            ("empty", RAW_BLOB, b"")]
    meta = json.dumps({"model_name": "tiny", "quant_scheme": "int4_g128_sym", "properties": {"group_size": "128"}})
    return secs, meta, (w, packed, scales, norm, N, K)


def test_writer_reader_roundtrip_and_layout(tmp_path):
    secs, meta, _ = sample_sections()
    path = str(tmp_path / "a.xinfer")
    write_artifact(path, meta, secs)
    r = ArtifactReader(path, verify_file_checksum=True)
    assert r.metadata_json() == meta
    table = r.sections()
    assert [s["name"] for s in table] == [s[0] for s in secs]
    for s, (name, tag, data) in zip(table, secs):
        assert s["type"] == tag and s["size"] == len(data) and s["offset"] % 64 == 0
        assert r.read_section(name) == data
        assert s["checksum"] == (oracle.crc64(data) if data else 0)
    assert r.has_section("odd.blob") and not r.has_section("missing")
    with pytest.raises(KeyError):
        r.read_section("missing")
    r.close()


def test_reader_rejects_damaged_files(tmp_path):
    secs, meta, _ = sample_sections()
    good = str(tmp_path / "g.xinfer")
    write_artifact(good, meta, secs)
    raw = bytearray(open(good, "rb").read())

    def opens(data, verify=True):
        p = str(tmp_path / "d.xinfer")
        open(p, "wb").write(bytes(data))
        try:
            ArtifactReader(p, verify).close()
            return True
        except _lib.XInferError:
            return False

    assert opens(raw)
    assert not opens(raw[:-1])                                   # truncated: size no longer matches the header
    assert not opens(b"YINFER\0\0" + raw[8:])                    # bad magic
    bad = bytearray(raw); bad[-3] ^= 1
    assert not opens(bad)                                        # footer magic
    bad = bytearray(raw); bad[8] = 2
    assert not opens(bad)                                        # format version
    bad = bytearray(raw); bad[300] ^= 0x40                       # a payload byte
    assert not opens(bad, True)                                  # whole-file checksum notices
    assert opens(bad, False)                                     # ...and without it the section's own checksum does:
    p = str(tmp_path / "d.xinfer")
    r = ArtifactReader(p, False)
    hit = [s for s in r.sections() if s["offset"] <= 300 < s["offset"] + s["size"]]
    if hit:
        with pytest.raises(_lib.XInferError) as e:
            r.read_section(hit[0]["name"])
        assert e.value.code == _lib.ERR_CONTRACT
    r.close()
    assert not opens(raw[:40])                                   # smaller than header plus footer


def test_cross_check_with_the_reference_writer_and_reader(tmp_path):
    ref = ref_lib()
    if ref is None:
        pytest.skip("the reference's artifact library has not been built (no reference tree)")
    secs, meta, _ = sample_sections(3)
    ours, theirs = str(tmp_path / "ours.xinfer"), str(tmp_path / "theirs.xinfer")
    write_artifact(ours, meta, secs)
    n = len(secs)
    names = (C.c_char_p * n)(*[s[0].encode() for s in secs])
    types = (C.c_uint32 * n)(*[s[1] for s in secs])
    bufs = [C.create_string_buffer(s[2], max(len(s[2]), 1)) for s in secs]
    datas = (C.c_void_p * n)(*[C.cast(b, C.c_void_p) for b in bufs])
    sizes = (C.c_uint64 * n)(*[len(s[2]) for s in secs])
    assert ref.ref_artifact_write(theirs.encode(), meta.encode(), n, names, types, datas, sizes) == 0
    assert open(ours, "rb").read() == open(theirs, "rb").read()          # byte-identical files
    # the reference's reader accepts our file, checksum included, and reads the same payloads
    assert ref.ref_artifact_section_count(ours.encode()) == n
    for name, _, data in secs:
        buf = np.empty(max(len(data), 1), np.uint8)
        got = ref.ref_artifact_read(ours.encode(), 1, name.encode(), buf.ctypes.data_as(C.c_void_p), len(data))
        if data:
            assert got == len(data) and buf[:got].tobytes() == data
    # our reader accepts the reference's file
    r = ArtifactReader(theirs, True)
    for name, _, data in secs:
        assert r.read_section(name) == data
    r.close()


@pytest.mark.gpu
def test_load_linear_whole_and_as_shards_then_run(tmp_path, cuda):
    import torch
    secs, meta, (w, packed, scales, norm, N, K) = sample_sections(5)
    path = str(tmp_path / "m.xinfer")
    write_artifact(path, meta, secs)
    r = ArtifactReader(path)
    name = "model.language_model.layers.0.mlp.down_proj.weight"
    Wd = torch.empty((N, K // 2), dtype=torch.uint8, device="cuda")
    Sd = torch.empty((N, K // 128), dtype=torch.float16, device="cuda")
    r.load_linear(name, N, K, Wd, Sd)
    assert np.array_equal(Wd.cpu().numpy(), packed) and np.array_equal(Sd.cpu().numpy(), scales)
    # the shards two tensor-parallel ranks would load: contiguous row ranges, no re-packing
    for rank in range(2):
        n0 = rank * (N // 2)
        Wl = torch.empty((N // 2, K // 2), dtype=torch.uint8, device="cuda")
        Sl = torch.empty((N // 2, K // 128), dtype=torch.float16, device="cuda")
        r.load_linear(name, N, K, Wl, Sl, row0=n0, rows=N // 2)
        assert np.array_equal(Wl.cpu().numpy(), packed[n0:n0 + N // 2])
        assert np.array_equal(Sl.cpu().numpy(), scales[n0:n0 + N // 2])
    with pytest.raises(_lib.XInferError):                       # the size checks of the reference's load_linear
        r.load_linear(name, N + 2, K, Wd, Sd)
    with pytest.raises(_lib.XInferError):
        r.load_linear(name, N, K, Wd, Sd, row0=N - 1, rows=2)
    # norm weights: bf16 -> fp32 with the checkpoint's 1 + w convention
    nd = torch.empty(K, dtype=torch.float32, device="cuda")
    r.load_bf16_as_f32("model.language_model.layers.0.input_layernorm.weight", K, nd, add_unit_offset=True)
    want = (norm.astype(np.uint32) << 16).view(np.float32) + np.float32(1.0)
    assert np.array_equal(nd.cpu().numpy(), want)
    # and the loaded projection runs: quantised weights x activations against the oracle
    M = 4
    X = np.random.default_rng(1).normal(size=(M, K)).astype(np.float16)
    Y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    assert cuda.linear_int4(Y, torch.from_numpy(X).cuda(), Wd, Sd, None, M, N, K) == 0
    ref = oracle.linear_int4_f64(X.astype(np.float32), packed, scales)
    assert np.max(np.abs(Y.cpu().numpy() - ref)) <= 1e-4 * max(1.0, float(np.abs(ref).max()))
    r.close()


# ------------------------------------------------------------------ a whole model through the artifact
_LIN = {"gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj", "q_proj": "self_attn.q_proj",
        "k_proj": "self_attn.k_proj", "v_proj": "self_attn.v_proj", "o_proj": "self_attn.o_proj",
        "in_qkv": "linear_attn.in_proj_qkv", "in_z": "linear_attn.in_proj_z", "in_b": "linear_attn.in_proj_b",
        "in_a": "linear_attn.in_proj_a", "out_proj": "linear_attn.out_proj"}
# decoder tensor -> (section, the checkpoint stores w - 1)
_VEC = {"input_norm": ("input_layernorm.weight", True), "post_norm": ("post_attention_layernorm.weight", True),
        "q_norm": ("self_attn.q_norm.weight", True), "k_norm": ("self_attn.k_norm.weight", True),
        "conv_w": ("linear_attn.conv1d.weight", False), "A_log": ("linear_attn.A_log", False),
        "dt_bias": ("linear_attn.dt_bias", False), "gdn_norm": ("linear_attn.norm.weight", False)}


def _bf16_bits(x):
    """fp32 -> bf16 bits, round to nearest even (what a converter stores)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def _bf16_to_f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def _export_layer(dec, idx, prefix, secs):
    """Appends the sections of one decoder layer; rewrites the decoder's fp32 vectors to what the file can hold."""
    full = dec.is_full(idx)
    lins = ["gate", "up", "down"] + (["q_proj", "k_proj", "v_proj", "o_proj"] if full else ["in_qkv", "in_z", "in_b", "in_a", "out_proj"])
    vecs = ["input_norm", "post_norm"] + (["q_norm", "k_norm"] if full else ["conv_w", "A_log", "dt_bias", "gdn_norm"])
    for v in vecs:
        sec, unit = _VEC[v]
        w = dec.tensor(idx, v, np.float32)
        bits = _bf16_bits(w - np.float32(1.0) if unit else w)
        held = _bf16_to_f32(bits) + np.float32(1.0) if unit else _bf16_to_f32(bits)
        dec.write_tensor(idx, v, held.astype(np.float32))
        secs.append((f"{prefix}.{sec}", RAW_BLOB, bits.tobytes()))
    for l in lins:
        secs.append((f"{prefix}.{_LIN[l]}.weight", TENSOR_WEIGHTS, dec.tensor(idx, l + ".w", np.uint8).tobytes()))
        secs.append((f"{prefix}.{_LIN[l]}.weight.scales", TENSOR_SCALES, dec.tensor(idx, l + ".s", np.float16).tobytes()))


@pytest.mark.gpu
def test_decoder_loads_its_weights_from_an_artifact(tmp_path, cuda):
    """A decoder's synthetic weights are written out under the reference loader's section names
    (src/targets/qwen3_8_27b/weights.cpp:358-640), a second decoder built from another seed loads the file, and the
    two then emit the same tokens and hold the same hidden states, bit for bit."""
    import torch
    from xinfer_b200.spec import Shape, SpecDecoder
    shape_cfg = Shape(hidden_size=1024, intermediate_size=2048, num_hidden_layers=4, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=4096, linear_num_v_heads=6, linear_num_k_heads=2)
    a = SpecDecoder(shape_cfg, batch=2, k=3, max_seq=96, seed=5)
    secs = [("model.language_model.embed_tokens.weight", RAW_BLOB, a.tensor(-1, "embed", np.uint16).tobytes())]
    for name, sec in (("final_norm", "model.language_model.norm.weight"), ("mtp_enorm", "mtp.pre_fc_norm_embedding.weight"),
                      ("mtp_hnorm", "mtp.pre_fc_norm_hidden.weight")):
        bits = _bf16_bits(a.tensor(-1, name, np.float32) - np.float32(1.0))
        a.write_tensor(-1, name, (_bf16_to_f32(bits) + np.float32(1.0)).astype(np.float32))
        secs.append((sec, RAW_BLOB, bits.tobytes()))
    for name, sec in (("lm_head", "lm_head.weight"), ("mtp_fc", "mtp.fc.weight")):
        secs.append((sec, TENSOR_WEIGHTS, a.tensor(-1, name + ".w", np.uint8).tobytes()))
        secs.append((sec + ".scales", TENSOR_SCALES, a.tensor(-1, name + ".s", np.float16).tobytes()))
    L = shape_cfg.num_hidden_layers
    for i in range(L):
        _export_layer(a, i, f"model.language_model.layers.{i}", secs)
    _export_layer(a, L, "mtp.layers.0", secs)
    path = str(tmp_path / "model.xinfer")
    write_artifact(path, json.dumps({"format": "xinfer", "note": "synthetic"}), secs)

    b = SpecDecoder(shape_cfg, batch=2, k=3, max_seq=96, seed=77)   # other weights until the file is loaded
    r = ArtifactReader(path)
    b.load_artifact(r)
    for i in list(range(L + 1)):
        for n in ("gate.w", "down.s", "input_norm"):
            assert np.array_equal(a.tensor(i, n, np.uint8), b.tensor(i, n, np.uint8)), (i, n)
    a.reset(30, seed=3)
    b.reset(30, seed=3)
    for step in range(3):
        a.step()
        b.step()
        ea, ca = a.results()
        eb, cb = b.results()
        assert np.array_equal(ea, eb) and np.array_equal(ca, cb), step
        assert np.array_equal(a.tensor(-1, "x", np.uint16), b.tensor(-1, "x", np.uint16)), step
    # a file whose layer kinds do not fit the decoder is refused
    wrong = [(n.replace("layers.0.linear_attn", "layers.0.self_attn_x"), t, d) for n, t, d in secs]
    path2 = str(tmp_path / "wrong.xinfer")
    write_artifact(path2, "{}", wrong)
    r2 = ArtifactReader(path2)
    with pytest.raises(_lib.XInferError):
        b.load_artifact(r2)
    r2.close()
    r.close()
    a.close()
    b.close()
