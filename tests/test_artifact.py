"""The ".pkl4" artifact: oracle pinned to the reference's unit tests, and the C reader / packers
of libpk100.so against the oracle (host code; no GPU needed)."""
import json
import struct

import numpy as np
import pytest

from oracle import artifact as A

VOCAB = [f"p{i}" for i in range(1024)]


# ----------------------------------------------------------------- oracle vs reference tests
def test_oracle_pads_fp16_linear_rows():                       # src/artifact.rs:729-745
    packed = A.encode_fp16_linear([1, 2, 3, 4, 5, 6], 2, 3, 4, 4)
    assert np.frombuffer(packed, "<f2").astype(np.float32).tolist() == [
        1, 2, 3, 0, 4, 5, 6, 0, 0, 0, 0, 0, 0, 0, 0, 0]


def test_oracle_pads_fp32_bias():                               # src/artifact.rs:747-757
    assert np.frombuffer(A.encode_fp32_bias([1.25, -2.5], 2, 4), "<f4").tolist() == [1.25, -2.5, 0.0, 0.0]


def test_oracle_rejects_non_finite():                           # src/artifact.rs:759-763
    with pytest.raises(A.ArtifactInvalid, match="non-finite"):
        A.encode_fp16([float("nan")], "bad")


def test_oracle_align_up():                                     # src/artifact.rs:765-769
    assert A.align_up(257, 256) == 512
    with pytest.raises(A.ArtifactInvalid):
        A.align_up((1 << 64) - 1, 256)


def test_oracle_vocabulary_contract():                          # src/artifact.rs:771-780
    A.validate_vocabulary(["piece"] * 1024, "v2_english")
    with pytest.raises(A.ArtifactInvalid, match="requires 1024"):
        A.validate_vocabulary(["piece"] * 1023, "v2_english")


@pytest.mark.parametrize("profile,tensors,params", [("v2_english", 725, 617_908_374),
                                                    ("v3_multilingual", 723, 627_057_286)])
def test_oracle_manifest_inventory(profile, tensors, params):   # src/weights.rs:656-670
    m = A.manifest(profile)
    assert len(m) == tensors
    assert sum(int(np.prod(shape, dtype=np.int64)) for dtype, shape in m.values() if dtype != "I64") == params


def test_oracle_classes():                                      # src/weights.rs:713-735
    assert A.classify("encoder.layers.12.feed_forward1.linear2.weight") == "ffn"
    assert A.classify("encoder.layers.0.conv.norm.num_batches_tracked") == "counter"
    assert A.classify("encoder.layers.3.conv.norm.running_var") == "sensitive_fp32"
    assert A.classify("encoder.layers.3.conv.depthwise_conv.weight") == "convolution"
    assert A.classify("encoder.layers.3.norm_out.weight") == "other_fp16"


# ----------------------------------------------------------------- C packers vs oracle
def test_c_packers_match_oracle(pk):
    art = pk.artifact
    rng = np.random.default_rng(0)
    # every rounding regime of fp16: normals, subnormals, ties, overflow to infinity, signed zero
    special = np.array([0.0, -0.0, 1.0, -1.0, 65504.0, 65519.9, 65520.0, 1e6, -1e6, 2.0 ** -14, 2.0 ** -24,
                        2.0 ** -25, 2.0 ** -25 * 1.0001, 3 * 2.0 ** -25, 2.0 ** -26, 1.0 + 2.0 ** -11,
                        1.0 + 3 * 2.0 ** -11, 1e-30, 6.0e-8, 6.1e-5], np.float32)
    values = np.concatenate([special, rng.standard_normal(20000).astype(np.float32) *
                             np.exp(rng.uniform(-20, 12, 20000)).astype(np.float32)])
    got = art.encode_fp16(values)
    want = np.frombuffer(A.encode_fp16(values), "<f2")
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))

    w = rng.standard_normal((5, 7)).astype(np.float32)
    got = art.encode_fp16_linear(w, 5, 7, 128, 128)
    want = np.frombuffer(A.encode_fp16_linear(w, 5, 7, 128, 128), "<f2").reshape(128, 128)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    assert art.encode_fp16_linear([1, 2, 3, 4, 5, 6], 2, 3, 4, 4).astype(np.float32).ravel().tolist() == [
        1, 2, 3, 0, 4, 5, 6, 0, 0, 0, 0, 0, 0, 0, 0, 0]
    assert art.encode_fp32_bias([1.25, -2.5], 2, 4).tolist() == [1.25, -2.5, 0.0, 0.0]
    with pytest.raises(art.ArtifactError):
        art.encode_fp16([np.nan])
    with pytest.raises(art.ArtifactError):
        art.encode_fp32_bias([1.0, np.inf], 2, 4)
    with pytest.raises(art.ArtifactError):
        art.encode_fp32_bias([1.0, 2.0], 2, 1)
    assert art.align_up(257, 256) == 512 and art.align_up(0, 4096) == 0 and art.align_up(4096, 4096) == 4096
    with pytest.raises(art.ArtifactError):
        art.align_up((1 << 64) - 1, 256)


# ----------------------------------------------------------------- C reader vs oracle writer
def small_model(rng):
    """A few tensors of every storage class with the checkpoint's names and ranks."""
    def n(*shape, std=0.05):
        return (rng.standard_normal(shape) * std).astype(np.float32)
    return {
        "encoder.layers.0.feed_forward1.linear1.weight": n(200, 72),          # fp16 linear, padded both ways
        "encoder.layers.0.conv.pointwise_conv1.weight": n(256, 128, 1),       # rank-3 linear, no padding
        "encoder.layers.0.conv.depthwise_conv.weight": n(64, 1, 9),           # plain fp16
        "encoder.layers.0.conv.norm.running_var": np.abs(n(64)) + 1.0,         # plain fp32
        "encoder.layers.0.conv.norm.num_batches_tracked": np.zeros((), np.float32),   # counter: dropped
        "encoder.layers.0.norm_out.weight": n(64),
        "encoder.subsampling.layers.0.weight": n(16, 1, 3, 3),                # rank 4, plain fp16
        "encoder.subsampling.linear.weight": n(130, 260),
        "encoder.subsampling.linear.bias": n(130),                            # padded fp32 bias
        "joint.head.weight": n(70, 64),
        "joint.head.bias": n(70),                                             # bias of a linear: padded
        "frontend.window": n(400),
    }


def test_reader_round_trip(pk, tmp_path):
    rng = np.random.default_rng(1)
    tensors = small_model(rng)
    path = tmp_path / "model.pkl4"
    header = A.write(path, tensors, "v2_english", VOCAB)
    want_header, want = A.read(path)
    assert want_header == header

    art = pk.artifact.Artifact(path)
    assert art.field("target") == "sm_89" and art.field("profile") == "v2_english"
    assert art.field("precision_plan") == "fp16" and art.field("source_revision") == header["source_revision"]
    assert art.vocabulary == VOCAB
    assert list(art.records) == [t["name"] for t in header["tensors"]]
    assert "encoder.layers.0.conv.norm.num_batches_tracked" not in art.records
    for rec in header["tensors"]:
        got = art.records[rec["name"]]
        for key in ("storage", "logical_shape", "physical_shape", "offset", "bytes"):
            assert got[key] == rec[key], (rec["name"], key)
        assert got["data"] % 256 == 0
        view = art.tensor(rec["name"])
        assert view.dtype == want[rec["name"]].dtype and view.shape == tuple(rec["logical_shape"])
        assert np.array_equal(view, want[rec["name"]])
        assert art.find(rec["name"]) == header["tensors"].index(rec)
    assert art.find("missing.tensor") == -1
    # storage classes chosen by the plan
    assert art.records["encoder.subsampling.linear.weight"]["physical_shape"] == [256, 384]
    assert art.records["encoder.subsampling.linear.bias"]["storage"] == "sm89_fp32_bias"
    assert art.records["joint.head.bias"]["physical_shape"] == [128]
    assert art.records["encoder.layers.0.conv.norm.running_var"]["storage"] == "fp32"
    assert art.records["encoder.layers.0.conv.pointwise_conv1.weight"]["logical_shape"] == [256, 128]
    # padding is zero
    full = np.frombuffer((pk.artifact.C.c_char * art.records["joint.head.weight"]["bytes"]).from_address(
        art.records["joint.head.weight"]["data"]), np.float16).reshape(128, 128)
    assert not full[70:].any() and not full[:, 64:].any()
    # read_f32: plain FP32 only
    assert np.array_equal(art.read_f32("frontend.window"), tensors["frontend.window"])
    with pytest.raises(pk.artifact.ArtifactError):
        art.read_f32("joint.head.bias")
    art.close()


def _rewrite(path, out, mutate_header=None, mutate_prefix=None, payload_delta=0):
    blob = bytearray(open(path, "rb").read())
    header_bytes = struct.unpack("<Q", blob[16:24])[0]
    header = json.loads(blob[24:24 + header_bytes])
    data_start = A.align_up(24 + header_bytes, 4096)
    payload = bytes(blob[data_start:])
    if mutate_header:
        mutate_header(header)
    encoded = json.dumps(header, separators=(",", ":")).encode()
    prefix = bytearray(A.MAGIC + struct.pack("<IIQ", 2, 0, len(encoded)))
    if mutate_prefix:
        mutate_prefix(prefix)
    new_start = A.align_up(24 + len(encoded), 4096)
    body = bytearray(new_start) + payload
    body[:24] = prefix
    body[24:24 + len(encoded)] = encoded
    if payload_delta > 0:
        body += bytes(payload_delta)
    elif payload_delta < 0:
        body = body[:payload_delta]
    open(out, "wb").write(body)


CASES = [
    ("bad magic", None, lambda p: p.__setitem__(0, ord("X")), 0),
    ("expected schema version 2, got 3", None, lambda p: p.__setitem__(slice(8, 12), struct.pack("<I", 3)), 0),
    ("unsupported prefix flags", None, lambda p: p.__setitem__(slice(12, 16), struct.pack("<I", 1)), 0),
    ("header length 0 is outside", None, lambda p: p.__setitem__(slice(16, 24), struct.pack("<Q", 0)), 0),
    ("payload bytes, file contains", None, None, 256),
    ("payload bytes, file contains", None, None, -2),
    ("header schema is 1", lambda h: h.__setitem__("schema_version", 1), None, 0),
    ("expected sm_89", lambda h: h.__setitem__("target", "sm_90"), None, 0),
    ("profile does not match", lambda h: h.__setitem__("source_revision", "0" * 40), None, 0),
    ("tensor alignment is 128", lambda h: h.__setitem__("tensor_alignment", 128), None, 0),
    ("requires 1024 vocabulary entries", lambda h: h.__setitem__("vocabulary", h["vocabulary"][:1023]), None, 0),
    ("is empty or contains control separators", lambda h: h["vocabulary"].__setitem__(5, "a\tb"), None, 0),
    ("duplicate tensor name", lambda h: h["tensors"][1].__setitem__("name", h["tensors"][0]["name"]), None, 0),
    ("invalid aligned offset", lambda h: h["tensors"][1].__setitem__("offset", h["tensors"][1]["offset"] + 16), None, 0),
    ("invalid aligned offset", lambda h: h["tensors"][2].__setitem__("offset", 0), None, 0),
    ("plain storage cannot change logical shape",
     lambda h: [t for t in h["tensors"] if t["storage"] == "fp32"][0].__setitem__("physical_shape", [1, 1]), None, 0),
    ("invalid sm_89 FP16 linear shapes",
     lambda h: [t for t in h["tensors"] if t["storage"] == "sm89_fp16_linear"][0].__setitem__("physical_shape", [200, 72]),
     None, 0),
    ("invalid sm_89 FP32 bias shapes",
     lambda h: [t for t in h["tensors"] if t["storage"] == "sm89_fp32_bias"][0].__setitem__("physical_shape", [130]),
     None, 0),
    ("bytes, header declares", lambda h: h["tensors"][0].__setitem__("bytes", h["tensors"][0]["bytes"] - 2), None, 0),
    ("last tensor ends at", lambda h: h["tensors"].pop(), None, 0),
    ("unknown storage", lambda h: h["tensors"][0].__setitem__("storage", "int4"), None, 0),
]


@pytest.mark.parametrize("message,mutate_header,mutate_prefix,delta", CASES)
def test_reader_rejects_what_the_reference_rejects(pk, tmp_path, message, mutate_header, mutate_prefix, delta):
    good = tmp_path / "good.pkl4"
    A.write(good, small_model(np.random.default_rng(2)), "v2_english", VOCAB)
    bad = tmp_path / "bad.pkl4"
    _rewrite(good, bad, mutate_header, mutate_prefix, delta)
    with pytest.raises(A.ArtifactInvalid):                    # the oracle agrees that it is invalid
        A.read(bad)
    with pytest.raises(pk.artifact.ArtifactError) as info:
        pk.artifact.Artifact(bad)
    assert info.value.code == pk.artifact.ERR_FORMAT and message in info.value.message


def test_reader_rejects_a_field_given_twice(pk, tmp_path):
    """serde refuses a struct field that occurs twice (src/artifact.rs:30-60, :147); a repeated
    unknown key is ignored like any unknown key."""
    good = tmp_path / "good.pkl4"
    A.write(good, small_model(np.random.default_rng(4)), "v2_english", VOCAB)
    blob = open(good, "rb").read()
    header_bytes = struct.unpack("<Q", blob[16:24])[0]
    doc = blob[24:24 + header_bytes].decode()
    payload = blob[A.align_up(24 + header_bytes, 4096):]

    def rewrite(text, name):
        enc = text.encode()
        body = bytearray(A.align_up(24 + len(enc), 4096)) + payload
        body[:24] = A.MAGIC + struct.pack("<IIQ", 2, 0, len(enc))
        body[24:24 + len(enc)] = enc
        path = tmp_path / name
        open(path, "wb").write(body)
        return path

    assert doc.startswith("{") and '"payload_bytes":' in doc and '"offset":' in doc
    value = json.loads(doc)["payload_bytes"]
    for name, text in (("top.pkl4", '{"payload_bytes":%d,' % value + doc[1:]),
                       ("tensor.pkl4", doc.replace('"offset":', '"offset":0,"offset":', 1))):
        with pytest.raises(pk.artifact.ArtifactError) as info:
            pk.artifact.Artifact(rewrite(text, name))
        assert info.value.code == pk.artifact.ERR_FORMAT and "duplicate field" in info.value.message
    ok = rewrite('{"x_unknown":1,"x_unknown":2,' + doc[1:], "unknown.pkl4")
    assert len(pk.artifact.Artifact(ok).records) > 0


def test_reader_io_errors_and_escapes(pk, tmp_path):
    with pytest.raises(pk.artifact.ArtifactError) as info:
        pk.artifact.Artifact(tmp_path / "absent.pkl4")
    assert info.value.code == pk.artifact.ERR_IO
    short = tmp_path / "short.pkl4"
    short.write_bytes(b"PKL4")
    with pytest.raises(pk.artifact.ArtifactError, match="prefix requires 24"):
        pk.artifact.Artifact(short)
    # JSON escapes and non-ASCII pieces survive the C parser
    vocab = list(VOCAB)
    vocab[0], vocab[1], vocab[2] = "▁the", 'q"uote\\', "\U0001F600"
    path = tmp_path / "escapes.pkl4"
    A.write(path, small_model(np.random.default_rng(3)), "v2_english", vocab)
    blob = open(path, "rb").read()
    assert b"\\u2581" in blob or "▁".encode() in blob
    assert pk.artifact.Artifact(path).vocabulary == vocab
    # the same document written with ASCII-only escapes (surrogate pairs)
    header_bytes = struct.unpack("<Q", blob[16:24])[0]
    header = json.loads(blob[24:24 + header_bytes])
    _rewrite(path, tmp_path / "ascii.pkl4")
    ascii_doc = json.dumps(header, ensure_ascii=True, separators=(", ", ": ")).encode()
    start = A.align_up(24 + len(ascii_doc), 4096)
    body = bytearray(start) + blob[A.align_up(24 + header_bytes, 4096):]
    body[:24] = A.MAGIC + struct.pack("<IIQ", 2, 0, len(ascii_doc))
    body[24:24 + len(ascii_doc)] = ascii_doc
    (tmp_path / "ascii.pkl4").write_bytes(body)
    assert pk.artifact.Artifact(tmp_path / "ascii.pkl4").vocabulary == vocab


def test_model_views_follow_the_manifest(pk, tmp_path):
    """layer / subsampling / decoder dictionaries from an artifact with the manifest's names
    (one encoder block, every tensor at its real shape is too large for a CPU test: the
    linears are checked through their names and logical shapes)."""
    m = A.manifest("v2_english", encoder_layers=1)
    rng = np.random.default_rng(4)
    tensors = {name: (rng.standard_normal(shape) * 0.05).astype(np.float32) for name, (_, shape) in m.items()}
    path = tmp_path / "one_block.pkl4"
    A.write(path, tensors, "v2_english", VOCAB)
    art = pk.artifact.Artifact(path)
    w = art.layer_weights(0)
    f16 = lambda a: np.asarray(a, np.float32).astype(np.float16).astype(np.float32)
    assert w["ff1_w1"].shape == (4096, 1024) and w["ff2_w2"].shape == (1024, 4096)
    assert np.array_equal(w["ff1_w1"], f16(tensors["encoder.layers.0.feed_forward1.linear1.weight"]))
    assert np.array_equal(w["wpos"], f16(tensors["encoder.layers.0.self_attn.relative_k_proj.weight"]))
    assert w["wpw1"].shape == (2048, 1024) and w["dw"].shape == (1024, 9)
    assert np.array_equal(w["dw"], f16(tensors["encoder.layers.0.conv.depthwise_conv.weight"]).reshape(1024, 9))
    assert np.array_equal(w["bn_v"], tensors["encoder.layers.0.conv.norm.running_var"])       # fp32 kept exactly
    assert np.array_equal(w["ln_att_g"], f16(tensors["encoder.layers.0.norm_self_att.weight"]))
    assert set(w) == set(pk.synth.layer_weights(1, 0))
    s = art.subsampling_weights()
    assert set(s) == set(pk.synth.subsampling_weights(1))
    assert s["conv0_w"].shape == (256, 9) and s["pw1_w"].shape == (256, 256) and s["proj_w"].shape == (1024, 4096)
    assert np.array_equal(s["proj_b"], tensors["encoder.subsampling.linear.bias"])
    d = art.decoder_weights(2)
    assert set(d) == set(pk.synth.decoder_weights(1, 2))
    assert d["embedding"].shape == (1025, 640) and d["w_joint"].shape == (1030, 640)
    assert np.array_equal(d["b_hh1"], tensors["decoder.lstm.bias_hh_l1"])
    assert np.array_equal(d["w_ih0"], f16(tensors["decoder.lstm.weight_ih_l0"]))


def test_size_contract_known_answers_through_the_c_abi(pk):
    """estimate_linear / Exl3Layout behind libpk100 (src/packing.rs:168-199, src/exl3.rs:82-95),
    and equal to the oracle's restatement on a sweep of shapes."""
    from oracle import codec
    A = pk.artifact
    fp16 = A.estimate_linear("fp16", 1024, 4096)
    fp8 = A.estimate_linear("fp8_e4m3", 1024, 4096)
    assert fp16["payload_bytes"] + fp16["metadata_bytes"] == 8 * 1024 * 1024
    assert fp8["payload_bytes"] == 4 * 1024 * 1024 and fp8["metadata_bytes"] == 16 * 1024
    assert A.estimate_linear("q4_k", 640, 8198) is None
    q4 = A.estimate_linear("q4_k", 1024, 4096)
    assert q4["payload_bytes"] + q4["metadata_bytes"] == 4096 * 4 * 144
    j = A.estimate_linear("fp8_e4m3", 640, 8198)
    assert (j["padded_in"], j["padded_out"]) == (640, 8320)
    lay = A.exl3_layout(4096, 1024, 4)
    assert lay["trellis_shape"] == [256, 64, 64]
    assert lay["trellis_bytes"] == 2 * 1024 * 1024 and lay["scale_bytes"] == 10 * 1024
    j = A.exl3_layout(640, 8198, 4)
    assert j["padded_in"] == 640 and j["padded_out"] == 8320 and j["trellis_shape"] == [40, 520, 64]
    with pytest.raises(ValueError):
        A.estimate_linear("fp16", 0, 4)
    with pytest.raises(ValueError):
        A.exl3_layout(16, 16, 9)
    for fmt in ("fp16", "fp8_e4m3", "int8", "q4_k", "exl3"):
        for k, n in ((1, 1), (127, 129), (256, 640), (1024, 3072), (4096, 1024), (640, 1030)):
            for bits in ((2, 4, 8) if fmt == "exl3" else (4,)):
                assert A.estimate_linear(fmt, k, n, bits) == codec.estimate_linear(fmt, k, n, bits), (fmt, k, n, bits)
    assert A.exl3_layout(1000, 70, 3) == codec.exl3_layout(1000, 70, 3)
