"""The CPU oracle against committed outputs of the REFERENCE'S OWN KERNELS
(tests/golden/reference_kernels.npz, produced on a B200 by tests/golden/make_golden.py from
the reference's kernels/sm89/*.cu compiled for sm_100a).  Runs without a GPU.
Tolerances as in tests/test_gpu_ref_kernels.py: one fp16 ulp plus fast-math exp for the
floating-point kernels, bit-exact for the quantiser and the token ids."""
import importlib.util
from pathlib import Path

import numpy as np

from oracle import codec, decoder as D, frontend as F, ops as O

HERE = Path(__file__).resolve().parent
spec = importlib.util.spec_from_file_location("make_golden", HERE / "golden" / "make_golden.py")
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)
GOLD = np.load(HERE / "golden" / "reference_kernels.npz")
CASES = make_golden.cases()


def test_layer_norm_and_fixed_quantiser():
    c = CASES["ln"]
    got = GOLD["ln"].astype(np.float32)
    want = O.layer_norm(c["x"], c["g"], c["b"], c["rows"])
    assert np.max(np.abs(got - want)) <= 2.0 ** -7 and np.mean(got != want) < 2e-3
    assert np.array_equal(GOLD["ln_q"], codec.quantize_fp8_fixed(got, 56.0))


def test_ffn_expand_fp8():
    c = CASES["ffn"]
    want = O.linear_fp8(c["xq"], c["wq"], c["ws"], O.FP8_INPUT_SCALE, act=1)[:, ::16]
    assert np.max(np.abs(GOLD["ffn"].astype(np.float32) - want)) <= 4e-3


def test_conv_module_elementwise():
    g, d = CASES["glu"], CASES["dw"]
    glu = GOLD["glu"].astype(np.float32)
    assert np.max(np.abs(glu - O.glu_masked(g["e"], g["rows"], g["valid"]))) <= 4e-3
    want = O.depthwise_bn_silu(glu, d["wdw"], *d["bn"], g["rows"])
    assert np.max(np.abs(GOLD["dw"].astype(np.float32) - want)) <= 4e-3


def test_scalar_attention():
    a = CASES["att"]
    want = O.local_attention(a["q"], a["k"], a["v"], a["pos"], a["u"], a["bv"], a["rows"], a["valid"])
    assert np.max(np.abs(GOLD["att"].astype(np.float32) - want)) <= 3e-3


def test_tdt_decoder_tokens():
    d = CASES["dec"]
    tokens, _, ambiguous = D.tdt_greedy(d["enc"], d["w"], d["frames"])
    n = len(tokens) if ambiguous is None else ambiguous
    ref = GOLD["dec_tokens"]
    assert n > 10 and np.array_equal(ref[:n], tokens[:n])
    if ambiguous is None:
        assert len(ref) == len(tokens)


def test_tdt_decoder_tokens_long_request():
    """The oracle's INT8-cache path against the kernel the reference launches from 1024 frames."""
    d = CASES["dec_long"]
    assert d["frames"] >= D.LONG_REQUEST_FRAMES
    tokens, _, ambiguous = D.tdt_greedy(d["enc"], d["w"], d["frames"], lstm_cache="auto")
    n = len(tokens) if ambiguous is None else ambiguous
    ref = GOLD["dec_long_tokens"]
    assert n >= 15 and np.array_equal(ref[:n], tokens[:n])
    # past the first near-tie the two streams may part for a few tokens, then the encoder
    # frames pull them together again: most positions still agree
    m = min(len(ref), len(tokens))
    assert abs(len(ref) - len(tokens)) <= 3 and np.mean(ref[:m] == tokens[:m]) > 0.85
    # and the long-request kernel is not the short-request kernel
    m = min(len(ref), len(GOLD["dec_long_tokens_fp16"]))
    assert not np.array_equal(ref[:m], GOLD["dec_long_tokens_fp16"][:m])


def test_tdt_decoder_tokens_long_request_kernel_on_short_requests():
    """16 independent 48-frame requests through the reference's INT8-cache kernel: every decision
    before each request's first near-tie must match."""
    d = CASES["dec_long_short"]
    compared = 0
    for i, enc in enumerate(d["enc"]):
        tokens, _, ambiguous = D.tdt_greedy(enc, d["w"], d["frames"], lstm_cache="int8")
        n = len(tokens) if ambiguous is None else ambiguous
        ref = GOLD[f"dec_long_short_{i}"]
        assert np.array_equal(ref[:n], tokens[:n]), i
        if ambiguous is None:
            assert len(ref) == len(tokens), i
        compared += n
    assert compared > 250


def test_tdt_decoder_tokens_long_request_kernel_more_requests():
    """Three further requests through the reference's INT8-cache kernel: the oracle agrees with
    every decision before each request's first near-tie (its trust band, see oracle/decoder.py)."""
    compared = 0
    for i, m in enumerate(CASES["dec_long_more"]):
        tokens, _, ambiguous = D.tdt_greedy(m["enc"], m["w"], m["frames"], lstm_cache="int8")
        n = min(len(tokens) if ambiguous is None else ambiguous, 100)
        ref = GOLD[f"dec_long_more_{i}"]
        assert np.array_equal(ref[:n], tokens[:n]), i
        compared += n
    assert compared > 20


def test_frontend_kernels():
    x = CASES["fe"]["x"]
    frames, valid = F.frame_counts(x.size)
    w512 = F.center_window(F.hann_window())
    want_frames = F.framed(x, w512)
    assert GOLD["fe_frames"].shape == (frames, 512)
    assert np.max(np.abs(GOLD["fe_frames"] - want_frames)) <= 1e-6
    offsets, bins, values = F.sparse_filters(F.triangular_filters())
    want_mel = F.log_mel(GOLD["fe_frames"], offsets, bins, values)
    assert np.max(np.abs(GOLD["fe_mel"] - want_mel)) <= 1e-4
    assert np.max(np.abs(GOLD["fe_norm"] - F.normalize(GOLD["fe_mel"], valid))) <= 1e-5
    assert not GOLD["fe_norm"][valid:].any()


def test_scaled_linears_and_quantisers():
    """pk_sm89_quantize_int8 / _fp8 and the INT8 / FP8 linears (kernels/sm89/linear.cu:325-429,
    :537-560): the contract every INT8 GEMM of this build follows."""
    c = CASES["lin"]
    assert np.array_equal(GOLD["lin_q8"], codec.quantize_int8(c["x"], c["inv8"]))
    assert np.array_equal(GOLD["lin_qf"], codec.quantize_fp8_fixed(c["x"], 56.0))
    w8, w8s = codec.quantize_rows_int8(c["w"])
    for act in (0, 1, 2):
        want = O.linear_int8(GOLD["lin_q8"], w8, w8s, np.float32(1.0 / c["inv8"]), bias=c["bias"], act=act)
        got = GOLD[f"lin_int8_act{act}"].astype(np.float32)
        assert np.max(np.abs(got - want)) <= 2e-3 and np.mean(got != want) < 5e-3, act
    wf, wfs = codec.quantize_rows_fp8(c["w"])
    want = O.linear_fp8(GOLD["lin_qf"], wf, wfs, O.FP8_INPUT_SCALE, bias=c["bias"])
    assert np.max(np.abs(GOLD["lin_fp8"].astype(np.float32) - want)) <= 4e-3


def test_layer_norm_pair_and_dynamic_quantiser():
    c = CASES["lnpair"]
    first, second = GOLD["lnpair_first"].astype(np.float32), GOLD["lnpair_second"].astype(np.float32)
    want1 = O.layer_norm(c["x"], c["g"][0], c["b"][0], c["rows"])
    assert np.max(np.abs(first - want1)) <= 2.0 ** -7 and np.mean(first != want1) < 2e-3
    want2 = O.layer_norm(first, c["g"][1], c["b"][1], c["rows"])
    assert np.max(np.abs(second - want2)) <= 2.0 ** -7 and np.mean(second != want2) < 2e-3
    assert np.array_equal(GOLD["lnpair_second_q"], codec.quantize_fp8_fixed(second, 56.0))
    wq, ws = O.quant_rows_fp8_dynamic(first, c["rows"])
    rows = c["rows"]
    assert np.allclose(GOLD["lndyn_s"][:rows], ws[:rows], rtol=1e-6, atol=0)
    assert np.mean(GOLD["lndyn_q"][:rows] != wq[:rows]) < 2e-3 and not GOLD["lndyn_q"][rows:].any()


def test_subsampling_stack():
    c = CASES["sub"]
    w, mel = c["w"], c["mel"]
    conv0 = codec.f16_round(np.maximum(O._conv_s2(mel[:, :, None], w["conv0_w"].reshape(256, 3, 3), w["conv0_b"]), 0))
    got0 = GOLD["sub_conv0"].astype(np.float32)
    want0 = conv0.reshape(-1, 256)[::7]
    assert got0.shape == want0.shape
    assert np.max(np.abs(got0 - want0)) <= 2e-3 and np.mean(got0 != want0) < 1e-2
    want = O.subsampling(mel, w)
    got = GOLD["sub_out"].astype(np.float32)
    assert got.shape == want.shape == (5, 1024)
    assert np.max(np.abs(got - want)) <= 2e-2
    assert float(np.sqrt(np.mean((got - want) ** 2)) / np.sqrt(np.mean(want ** 2))) <= 2e-3


def test_sparse_2of4_contract():
    """pk_sm89_ffn_contract_fp8_sparse (`mma.sp` on the compressed 2:4 arena, kernels/sm89/encoder.cu:685-713,
    :1087-1095) run on a B200 on the arena the oracle's compressor wrote: equals the oracle's dense sums over
    the pruned values (so the arena layout and the selection rule are the reference's), equals the reference's
    dense kernel on the pruned bytes, and differs from the dense kernel on the unpruned bytes."""
    gold = np.load(HERE / "golden" / "reference_sparse24.npz")
    c = CASES["sparse24"]
    wq, ws = codec.quantize_rows_fp8(c["w"])
    pruned = codec.prune_2of4_e4m3(c["h"])
    want = O.linear_fp8(pruned, wq, ws, np.float32(1.0 / 16.0), residual16=c["x"], alpha=0.5)
    sparse = gold["sparse"].astype(np.float32)
    assert np.max(np.abs(sparse - want)) <= 4e-3
    assert np.max(np.abs(sparse - gold["dense_pruned"].astype(np.float32))) <= 2e-3
    full = O.linear_fp8(c["h"], wq, ws, np.float32(1.0 / 16.0), residual16=c["x"], alpha=0.5)
    assert np.max(np.abs(gold["dense_full"].astype(np.float32) - full)) <= 4e-3
    assert np.max(np.abs(sparse - full)) > 5e-2          # pruning half the activations is visible
