"""GPU parity: tcgen05 GEMM family through pk100_gemm vs the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import codec, ops as O
from tests.util import dev, dev16, host, nrmse

pytestmark = pytest.mark.gpu


def _status(cuda):
    return torch.zeros(1, dtype=torch.int32, device=cuda)


def _f16_case(seed, m, n, k):
    rng = np.random.default_rng(seed)
    x = codec.f16_round(rng.standard_normal((m, k)))
    w = codec.f16_round(rng.standard_normal((n, k)) * 0.02)
    return x, w


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 256, 128), (200, 384, 1024),
                                   (752, 1024, 1024), (33, 640, 1024), (1, 256, 64)])
def test_f16_linear(pk, cuda, m, n, k):
    L = pk.lib
    x, w = _f16_case(m + n, m, n, k)
    st = _status(cuda)
    out = torch.zeros((m, n), dtype=torch.float16, device=cuda)
    pk.ops.gemm(dev16(x), dev16(w), kind=L.KIND_F16, out=out, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0, "a bounded wait expired inside the GEMM"
    want = O.linear_f16(x, w)
    got = host(out)
    # reference gate for FP16 linears: abs <= 0.02 (src/cuda.rs:821-861); ours is tighter
    assert np.max(np.abs(got - want)) <= 4e-3, (np.max(np.abs(got - want)), nrmse(got, want))


def test_f16_linear_reference_bench_operands_bias_residual_relu(pk, cuda):
    # operands of the reference's own linear micro-benchmark (src/cuda.rs:780-818)
    L = pk.lib
    m, n, k = 256, 1024, 1024
    x, w, b = O.reference_bench_operands(m, n, k)
    rng = np.random.default_rng(0)
    res = codec.f16_round(rng.standard_normal((m, n)))
    st = _status(cuda)
    out = dev16(res).clone()
    pk.ops.gemm(dev16(x), dev16(w), kind=L.KIND_F16, out=out, bias=dev(b), act=L.ACT_RELU,
                residual=out, alpha=0.5, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    want = O.linear_f16(x, w, bias=b, act=2, residual16=res, alpha=0.5)
    assert np.max(np.abs(host(out) - want)) <= 4e-3


@pytest.mark.parametrize("m", [750, 128, 77])
def test_fp8_ff_expand_silu(pk, cuda, m):
    # pk_sm89_ffn_expand_fp8_async (kernels/sm89/encoder.cu:1063-1069): fixed 8/448
    # activation scale, per-row weight scales, SiLU, fp16 out
    L = pk.lib
    rng = np.random.default_rng(11)
    x = codec.f16_round(rng.standard_normal((m, 1024)))
    w = codec.f16_round(rng.standard_normal((4096, 1024)) * 0.02)
    xq = codec.quantize_fp8_fixed(x, 56.0)
    wq, ws = codec.quantize_rows_fp8(w)
    st = _status(cuda)
    out = torch.zeros((m, 4096), dtype=torch.float16, device=cuda)
    pk.ops.gemm(dev(xq), dev(wq), kind=L.KIND_E4M3, out=out, row_scale=8.0 / 448.0,
                col_scales=dev(ws), act=L.ACT_SILU, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    want = O.linear_fp8(xq, wq, ws, O.FP8_INPUT_SCALE, act=1)
    got = host(out)
    assert np.max(np.abs(got - want)) <= 4e-3, np.max(np.abs(got - want))


def test_int8_linear_exact_accumulate(pk, cuda):
    # pk_sm89_int8_linear_epilogue contract (kernels/sm89/linear.cu:378-429): the S32
    # accumulator is exact, so an fp32 output with unit scales must match bit for bit
    L = pk.lib
    rng = np.random.default_rng(12)
    m, n, k = 300, 512, 4096
    a = rng.integers(-127, 128, (m, k), dtype=np.int8)
    b = rng.integers(-127, 128, (n, k), dtype=np.int8)
    st = _status(cuda)
    out = torch.zeros((m, n), dtype=torch.float32, device=cuda)
    pk.ops.gemm(dev(a), dev(b), kind=L.KIND_S8, out=out, out_type=L.OUT_F32, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    acc = O.accumulate(a, b)
    assert np.array_equal(host(out), acc.astype(np.float32))


def test_int8_linear_scales_bias_rowscales(pk, cuda):
    L = pk.lib
    rng = np.random.default_rng(13)
    m, n, k = 200, 3072, 1024
    x = codec.f16_round(rng.standard_normal((m, k)))
    w = codec.f16_round(rng.standard_normal((n, k)) * 0.02)
    xq, xs = O.quant_rows_int8_dynamic(x)
    wq, ws = codec.quantize_rows_int8(w)
    bias = (0.1 * rng.standard_normal(n)).astype(np.float32)
    st = _status(cuda)
    out = torch.zeros((m, n), dtype=torch.float16, device=cuda)
    pk.ops.gemm(dev(xq), dev(wq), kind=L.KIND_S8, out=out, row_scales=dev(xs), col_scales=dev(ws),
                bias=dev(bias), status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    want = O.linear_int8(xq, wq, ws, xs, bias=bias)
    assert np.max(np.abs(host(out) - want)) <= 2e-3


def test_fp8_glu_epilogue(pk, cuda):
    # pk_sm89_conv_glu_fp8 (kernels/sm89/encoder.cu:1121-1127): per-row activation
    # scales, value/gate pairing, pad-row mask
    L = pk.lib
    rng = np.random.default_rng(14)
    m, valid = 300, 290
    x = codec.f16_round(rng.standard_normal((m, 1024)))
    w = codec.f16_round(rng.standard_normal((2048, 1024)) * 0.03)
    xq, xs = O.quant_rows_fp8_dynamic(x)
    wq, ws = codec.quantize_rows_fp8(w)
    st = _status(cuda)
    out = torch.zeros((m, 1024), dtype=torch.float16, device=cuda)
    pk.ops.gemm(dev(xq), dev(wq), kind=L.KIND_E4M3, epilogue=L.EPI_GLU, out=out, row_scales=dev(xs),
                col_scales=dev(ws), valid_rows=valid, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    e = O.linear_fp8(xq, wq, ws, xs)
    want = O.glu_masked(e, m, valid)
    got = host(out)
    assert np.all(got[valid:] == 0)
    assert np.max(np.abs(got - want)) <= 4e-3


def test_fp8_residual_in_place(pk, cuda):
    # epilogue 6 (kernels/sm89/encoder.cu:993-999): out = f16(fma(1, v, out))
    L = pk.lib
    rng = np.random.default_rng(15)
    m = 260
    x = codec.f16_round(rng.standard_normal((m, 1024)))
    w = codec.f16_round(rng.standard_normal((1024, 1024)) * 0.02)
    res = codec.f16_round(rng.standard_normal((m, 1024)))
    xq, xs = O.quant_rows_fp8_dynamic(x)
    wq, ws = codec.quantize_rows_fp8(w)
    st = _status(cuda)
    out = dev16(res).clone()
    pk.ops.gemm(dev(xq), dev(wq), kind=L.KIND_E4M3, out=out, row_scales=dev(xs), col_scales=dev(ws),
                residual=out, alpha=1.0, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    want = O.linear_fp8(xq, wq, ws, xs, residual16=res, alpha=1.0)
    assert np.max(np.abs(host(out) - want)) <= 4e-3


@pytest.mark.parametrize("m", [750, 130])
def test_ff_block_config1(pk, cuda, m):
    """Benchmark configuration 1: LN -> FP8 GEMM -> SiLU -> 70 % of the 128x64 tiles
    zeroed -> INT8 GEMM (skipping them) -> x + 0.5 * y."""
    L = pk.lib
    rng = np.random.default_rng(1)
    x = codec.f16_round(rng.standard_normal((m, 1024)))
    gamma, beta = np.ones(1024, np.float32), np.zeros(1024, np.float32)
    w1 = codec.f16_round(rng.standard_normal((4096, 1024)) * 0.02)
    w2 = codec.f16_round(rng.standard_normal((1024, 4096)) * 0.02)
    w1q, w1s = codec.quantize_rows_fp8(w1)
    w2q, w2s = codec.quantize_rows_int8(w2)
    # oracle pass 1: statistics -> tau for 70 % zero tiles
    xq_o = O.ln_quant_fp8_fixed(x, gamma, beta, m)
    _, _, stats = O.ff_expand(xq_o, w1q, w1s, m, 0.0)
    tau = O.calibrate_tau(stats, 0.7)
    want, mid = O.ff_block(x, gamma, beta, w1q, w1s, w2q, w2s, m, tau)
    assert abs(mid["keep"].mean() - 0.3) < 0.04

    xd = dev16(x)
    xq, _ = pk.ops.layer_norm(xd, dev16(gamma), dev16(beta), L.LN_E4M3_FIXED, inv_scale=56.0)
    mt = (m + 127) // 128
    hq = torch.zeros((m, 4096), dtype=torch.int8, device=cuda)
    keep = torch.zeros((mt, 64), dtype=torch.uint8, device=cuda)
    stats_d = torch.zeros((mt, 64), dtype=torch.float32, device=cuda)
    st = _status(cuda)
    pk.ops.gemm(xq, dev(w1q), kind=L.KIND_E4M3, epilogue=L.EPI_SPARSE_OUT, out=hq, out_type=L.OUT_S8,
                out_scale=32.0, row_scale=8.0 / 448.0, col_scales=dev(w1s), tau=float(tau),
                keep_out=keep, stats_out=stats_d, status=st)
    y = xd.clone()
    pk.ops.gemm(hq, dev(w2q), kind=L.KIND_S8, out=y, row_scale=1.0 / 32.0, col_scales=dev(w2s),
                residual=y, alpha=0.5, keep_in=keep, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert np.allclose(host(stats_d), mid["stats"], rtol=2e-3, atol=1e-5)    # tanh.approx: rel 2^-11
    assert np.array_equal(host(keep), mid["keep"])
    # INT8 hidden codes: equal except values sitting on a rounding boundary
    hq_h = host(hq)
    diff = hq_h != mid["hq"]
    assert diff.mean() < 3e-2 and np.max(np.abs(hq_h.astype(int) - mid["hq"].astype(int))) <= 1
    # second GEMM fed with the GPU's own codes is exact up to the fp32 epilogue
    want_gpu_codes = O.ff_contract(hq_h, w2q, w2s, x)
    got = host(y)
    assert np.max(np.abs(got - want_gpu_codes)) <= 2e-3
    assert nrmse(got, want) <= 1e-2


@pytest.mark.parametrize("m,n,k", [(750, 4096, 1024), (130, 1024, 1024), (64, 128, 128)])
def test_w4g128_in_smem_dequant(pk, cuda, m, n, k):
    """Benchmark configuration 0: X fp16 [750,1024] x W INT4 symmetric, g=128 along K, fp16
    scales ~U(0.005,0.02), fp32 accumulate.  The GEMM dequantises the codes in shared memory;
    its result must equal the fp16 GEMM on the pre-dequantised weights bit for bit."""
    L = pk.lib
    rng = np.random.default_rng(0)
    x = codec.f16_round(rng.standard_normal((m, k)))
    codes = rng.integers(-7, 8, (n, k), dtype=np.int8)
    packed = codec.pack_nibbles(codes)
    scales = rng.uniform(0.005, 0.02, (k // 128, n)).astype(np.float16)
    st = _status(cuda)
    out = torch.zeros((m, n), dtype=torch.float16, device=cuda)
    pk.ops.gemm(dev16(x), dev(packed), kind=L.KIND_F16_W4G128, out=out, b_group_scales=dev(scales), n=n,
                status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    want = O.linear_w4g128(x, packed, scales)
    got = host(out)
    assert np.max(np.abs(got - want)) <= 4e-3 * max(1.0, np.abs(want).max() / 4)
    # same operands through the pre-dequantised fp16 path
    w16 = pk.ops.dequant_w4g128(dev(packed), dev(scales))
    assert np.array_equal(host(w16), codec.dequant_int4_g128(packed, scales))
    ref = torch.zeros((m, n), dtype=torch.float16, device=cuda)
    pk.ops.gemm(dev16(x), w16, kind=L.KIND_F16, out=ref, status=st)
    torch.cuda.synchronize()
    assert np.array_equal(got, host(ref))


@pytest.mark.parametrize("kind", ["f16", "e4m3", "s8"])
def test_cta_pair_tiles_match_single_cta_tiles(pk, cuda, kind):
    """256-column tiles can run on CTA pairs (cta_group::2).  Same operands through both paths:
    INT8 must agree bit for bit (exact accumulator), fp kinds within one fp16 ulp; the pair
    result is also checked against the oracle.  M is not a multiple of 256 (odd tile count)."""
    L = pk.lib
    rng = np.random.default_rng(21)
    m, n, k = 4480, 1024, 1024          # 35 row tiles x 4 column tiles = 140... forced to 256-wide below
    x = codec.f16_round(rng.standard_normal((m, k)))
    w = codec.f16_round(rng.standard_normal((2048, k)) * 0.02)
    n = 2048
    res = codec.f16_round(rng.standard_normal((m, n)))
    if kind == "f16":
        a, b, kw, want = dev16(x), dev16(w), dict(kind=L.KIND_F16), O.linear_f16(x, w, residual16=res, alpha=0.5)
    elif kind == "e4m3":
        xq, xs = O.quant_rows_fp8_dynamic(x)
        wq, ws = codec.quantize_rows_fp8(w)
        a, b = dev(xq), dev(wq)
        kw = dict(kind=L.KIND_E4M3, row_scales=dev(xs), col_scales=dev(ws))
        want = O.linear_fp8(xq, wq, ws, xs, residual16=res, alpha=0.5)
    else:
        xq, xs = O.quant_rows_int8_dynamic(x)
        wq, ws = codec.quantize_rows_int8(w)
        a, b = dev(xq), dev(wq)
        kw = dict(kind=L.KIND_S8, row_scales=dev(xs), col_scales=dev(ws))
        want = O.linear_int8(xq, wq, ws, xs, residual16=res, alpha=0.5)
    outs = []
    for pairs in (1, 0):
        L.lib.pk100_set_gemm_cta_pairs(pairs)
        st = _status(cuda)
        out = dev16(res).clone()
        pk.ops.gemm(a, b, out=out, residual=out, alpha=0.5, status=st, **kw)
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        outs.append(host(out))
    L.lib.pk100_set_gemm_cta_pairs(0)
    assert np.max(np.abs(outs[0] - want)) <= 4e-3
    if kind == "s8":
        assert np.array_equal(outs[0], outs[1])
    else:
        assert np.max(np.abs(outs[0] - outs[1])) <= 2e-3


def test_gemm_rejects_bad_arguments(pk, cuda):
    L = pk.lib
    a = torch.zeros((8, 24), dtype=torch.float16, device=cuda)     # k*2 = 48 bytes: ok; n bad below
    b = torch.zeros((40, 24), dtype=torch.float16, device=cuda)
    out = torch.zeros((8, 40), dtype=torch.float16, device=cuda)
    with pytest.raises(L.Pk100Error):
        pk.ops.gemm(a, b, kind=L.KIND_F16, out=out)                 # n % 32 != 0
    a = torch.zeros((8, 20), dtype=torch.float16, device=cuda)     # k*2 = 40 bytes: not /16
    b = torch.zeros((64, 20), dtype=torch.float16, device=cuda)
    out = torch.zeros((8, 64), dtype=torch.float16, device=cuda)
    with pytest.raises(L.Pk100Error):
        pk.ops.gemm(a, b, kind=L.KIND_F16, out=out)


@pytest.mark.parametrize("n", [4096, 1024])
def test_fp8_expand_e4m3_out(pk, cuda, n):
    """The reference's packed FFN chain writes the expand output as E4M3(f16(SiLU(v)) * 16)
    (epilogue 1, kernels/sm89/encoder.cu:1006-1022, pk_sm89_ffn_expand_fp8_packed :1071-1077):
    PK100_OUT_E4M3 with out_scale = 16.  n = 4096 takes the 256-column tiles (staged TMA store of
    64-byte rows), n = 1024 the 128-column tiles (per-thread stores)."""
    L = pk.lib
    rng = np.random.default_rng(31)
    m = 300
    x = codec.f16_round(rng.standard_normal((m, 1024)))
    w = codec.f16_round(rng.standard_normal((n, 1024)) * 0.02)
    xq = codec.quantize_fp8_fixed(x, 56.0)
    wq, ws = codec.quantize_rows_fp8(w)
    st = _status(cuda)
    out = torch.zeros((m, n), dtype=torch.uint8, device=cuda)
    pk.ops.gemm(dev(xq), dev(wq), kind=L.KIND_E4M3, out=out, out_type=L.OUT_E4M3, out_scale=16.0,
                row_scale=8.0 / 448.0, col_scales=dev(ws), act=L.ACT_SILU, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    silu16 = O.linear_fp8(xq, wq, ws, O.FP8_INPUT_SCALE, act=1)          # f16(SiLU(v))
    want = codec.e4m3_encode((silu16 * np.float32(16.0)).astype(np.float32))
    got = host(out)
    # a code differs only where the fp16 value before it differs by an ulp (fast-math exp)
    assert np.mean(got != want) < 2e-2
    d = np.abs(codec.e4m3_decode(got) - codec.e4m3_decode(want))
    assert np.all(d <= 0.125 * np.abs(codec.e4m3_decode(want)) + 2.0 ** -9)


def test_f16_operands_with_silu_glu_and_sparse_out(pk, cuda):
    """The epilogue families on kind::f16 operands (pk_sm89_ffn_expand_async, the reference's fp16
    FF expand with SiLU, kernels/sm89/encoder.cu:427-547; fp16 conv pointwise + GLU)."""
    L = pk.lib
    rng = np.random.default_rng(32)
    m, valid = 260, 250
    x = codec.f16_round(rng.standard_normal((m, 1024)))
    w = codec.f16_round(rng.standard_normal((2048, 1024)) * 0.03)
    st = _status(cuda)
    # SiLU
    out = torch.zeros((m, 2048), dtype=torch.float16, device=cuda)
    pk.ops.gemm(dev16(x), dev16(w), kind=L.KIND_F16, out=out, act=L.ACT_SILU, status=st)
    torch.cuda.synchronize()
    assert np.max(np.abs(host(out) - O.linear_f16(x, w, act=1))) <= 4e-3
    # GLU (+ pad-row mask)
    glu = torch.zeros((m, 1024), dtype=torch.float16, device=cuda)
    pk.ops.gemm(dev16(x), dev16(w), kind=L.KIND_F16, epilogue=L.EPI_GLU, out=glu, valid_rows=valid, status=st)
    torch.cuda.synchronize()
    want = O.glu_masked(O.linear_f16(x, w), m, valid)
    assert np.all(host(glu)[valid:] == 0) and np.max(np.abs(host(glu) - want)) <= 4e-3
    # SPARSE_OUT: SiLU, tile statistic, INT8 codes of the kept tiles
    mt = (m + 127) // 128
    hq = torch.zeros((m, 2048), dtype=torch.int8, device=cuda)
    keep = torch.zeros((mt, 32), dtype=torch.uint8, device=cuda)
    stats = torch.zeros((mt, 32), dtype=torch.float32, device=cuda)
    h32 = O.silu(O.epilogue(O.accumulate(x, w)))
    want_stats = O.tile_stats(h32, m)
    tau = float(np.sort(want_stats.ravel())[int(0.5 * want_stats.size)])
    pk.ops.gemm(dev16(x), dev16(w), kind=L.KIND_F16, epilogue=L.EPI_SPARSE_OUT, out=hq, out_type=L.OUT_S8,
                out_scale=32.0, tau=tau, keep_out=keep, stats_out=stats, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) & 1 == 0
    # N(0, 0.03) weights push a few SiLU values beyond 127 / 32: the clamp is reported (bit 3)
    assert bool(int(st.item()) & 8) == bool(np.max(h32[:m]) * 32.0 > 127.0)
    assert np.allclose(host(stats), want_stats, rtol=2e-3, atol=1e-5)
    near = np.abs(want_stats / tau - 1.0) < 2e-3
    assert np.array_equal(host(keep)[~near], (want_stats >= tau).astype(np.uint8)[~near])
    mask = np.repeat(np.repeat(host(keep), 128, axis=0)[:m], 64, axis=1).astype(bool)
    codes = np.clip(np.rint(h32 * 32.0), -127, 127).astype(np.int8)
    got = host(hq)
    assert not got[~mask].any()
    assert np.max(np.abs(got[mask].astype(int) - codes[mask].astype(int))) <= 1 and np.mean(got[mask] != codes[mask]) < 3e-2


def test_cta_limits_do_not_change_results(pk, cuda):
    """max_ctas (per call) and the process-wide cap shrink the persistent grid; every tile is still
    computed, bit for bit the same."""
    L = pk.lib
    rng = np.random.default_rng(33)
    m, n, k = 700, 1024, 1024
    xq = dev(rng.integers(-127, 128, (m, k), dtype=np.int8))
    wq = dev(rng.integers(-127, 128, (n, k), dtype=np.int8))
    outs = []
    for max_ctas, cap in ((0, 0), (7, 0), (0, 20), (1, 0)):
        L.lib.pk100_set_gemm_cta_cap(cap)
        st = _status(cuda)
        out = torch.zeros((m, n), dtype=torch.float32, device=cuda)
        pk.ops.gemm(xq, wq, kind=L.KIND_S8, out=out, out_type=L.OUT_F32, max_ctas=max_ctas, status=st)
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        outs.append(host(out).copy())
    L.lib.pk100_set_gemm_cta_cap(0)
    assert all(np.array_equal(outs[0], o) for o in outs[1:])
    hits, misses = L.tensor_map_cache_stats()
    assert hits > 0 and misses > 0          # the four calls share their three descriptors


def test_sparse_out_reports_clamped_codes(pk, cuda):
    """|SiLU| * out_scale beyond 127 is clamped, and status bit 3 says so."""
    L = pk.lib
    rng = np.random.default_rng(34)
    m = 128
    x = codec.f16_round(rng.standard_normal((m, 1024)))
    w = codec.f16_round(rng.standard_normal((256, 1024)) * 0.02)
    hq = torch.zeros((m, 256), dtype=torch.int8, device=cuda)
    keep = torch.zeros((1, 4), dtype=torch.uint8, device=cuda)
    for out_scale, clipped in ((32.0, False), (4096.0, True)):
        st = _status(cuda)
        pk.ops.gemm(dev16(x), dev16(w), kind=L.KIND_F16, epilogue=L.EPI_SPARSE_OUT, out=hq, out_type=L.OUT_S8,
                    out_scale=out_scale, tau=0.0, keep_out=keep, status=st)
        torch.cuda.synchronize()
        assert bool(int(st.item()) & 8) == clipped and not int(st.item()) & 1
        assert int(host(hq).max()) == (127 if clipped else int(host(hq).max()))
