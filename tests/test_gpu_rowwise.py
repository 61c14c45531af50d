"""GPU parity: LayerNorm (+fused quantisers), quantisers, weight packers, GLU,
depthwise+BN+SiLU -- CUDA kernels through the C ABI vs the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import codec, ops as O
from tests.util import dev, dev16, host

pytestmark = pytest.mark.gpu


def _rows(seed, m, scale=1.0):
    rng = np.random.default_rng(seed)
    return codec.f16_round(rng.standard_normal((m, 1024)) * scale)


def _affine(seed):
    rng = np.random.default_rng(seed)
    return codec.f16_round(1.0 + 0.1 * rng.standard_normal(1024)), codec.f16_round(0.1 * rng.standard_normal(1024))


def test_quantize_fp8_fixed_bit_exact(pk, cuda):
    # bit-exact contract (src/cuda/quant_benchmark.rs:305-308)
    x = _rows(0, 37, 3.0)
    x[0, :8] = [0.0, -0.0, 500.0, -500.0, 8.0, 1e-4, 0.0179, 65504.0]
    got = host(pk.ops.quantize_fp8_fixed(dev16(x), 56.0))
    assert np.array_equal(got, codec.quantize_fp8_fixed(x, 56.0))
    # ragged tail (elements not a multiple of 8)
    flat = x.reshape(-1)[:1003]
    got = host(pk.ops.quantize_fp8_fixed(dev16(flat), 56.0))
    assert np.array_equal(got, codec.quantize_fp8_fixed(flat, 56.0))


def test_quantize_int8_bit_exact(pk, cuda):
    x = _rows(1, 19, 2.0)
    x[0, :6] = [0.5 / 32, 1.5 / 32, 200.0, -200.0, 2.5 / 32, -0.5 / 32]
    got = host(pk.ops.quantize_int8(dev16(x), 32.0))
    assert np.array_equal(got, codec.quantize_int8(x, 32.0))


def test_empty_inputs_are_accepted(pk, cuda):
    L = pk.lib
    assert L.lib.pk100_quantize_fp8_fixed(None, 1, 1, 0, 1.0) == L.OK
    assert L.lib.pk100_glu_masked(None, 1, 1, 0, 8, 8, None) == L.OK


@pytest.mark.parametrize("fmt", ["e4m3", "s8", "s4_row", "s4_g128"])
def test_weight_packers_bit_exact(pk, cuda, fmt):
    L = pk.lib
    rng = np.random.default_rng(3)
    w = codec.f16_round(rng.standard_normal((96, 1024)) * 0.02)
    w[5] = 0.0                                    # an all-zero row takes scale 1
    wd = dev16(w)
    if fmt == "e4m3":
        q, s = pk.ops.pack_weight_rows(wd, L.PACK_E4M3)
        eq, es = codec.quantize_rows_fp8(w)
    elif fmt == "s8":
        q, s = pk.ops.pack_weight_rows(wd, L.PACK_S8)
        eq, es = codec.quantize_rows_int8(w)
    elif fmt == "s4_row":
        q, s = pk.ops.pack_weight_rows(wd, L.PACK_S4_ROW)
        eq, es = codec.quantize_rows_int4(w)
    else:
        q, s = pk.ops.pack_weight_rows(wd, L.PACK_S4_G128)
        eq, es = codec.quantize_int4_g128(w)
        assert np.array_equal(host(s).astype(np.float16), es)
        assert np.array_equal(host(q), eq)
        back = host(pk.ops.dequant_w4g128(q, s))
        assert np.array_equal(back, codec.dequant_int4_g128(eq, es))
        return
    assert np.array_equal(host(s), es)
    assert np.array_equal(host(q), eq)


def _check_codes(got, want, max_fraction=2e-3):
    """LayerNorm statistics are reduced in a different order on the GPU, so a value
    sitting on a rounding boundary may land on the neighbouring code."""
    got = got.astype(np.int32)
    want = want.astype(np.int32)
    diff = got != want
    assert diff.mean() <= max_fraction, f"{diff.mean():.2e} of codes differ"
    # any differing code is an adjacent code
    g, w = got[diff], want[diff]
    assert np.all(np.abs(g - w) <= 1) or np.all(np.abs((g & 127) - (w & 127)) <= 1)


@pytest.mark.parametrize("rows,valid", [(752, 750), (17, 17), (64, 40)])
def test_layer_norm_modes(pk, cuda, rows, valid):
    L = pk.lib
    x = _rows(10 + rows, rows, 2.0)
    g, b = _affine(4)
    xd, gd, bd = dev16(x), dev16(g), dev16(b)
    want = O.layer_norm(x, g, b, valid)
    y, _ = pk.ops.layer_norm(xd, gd, bd, L.LN_F16, valid_rows=valid)
    y = host(y)
    # tolerance: one fp16 ulp of the normalised value (|y| <= ~8 -> 2^-7)
    assert np.max(np.abs(y - want)) <= 2.0 ** -7
    assert np.mean(y != want) < 2e-3
    assert np.all(y[valid:] == 0)

    q, _ = pk.ops.layer_norm(xd, gd, bd, L.LN_E4M3_FIXED, inv_scale=56.0, valid_rows=valid)
    _check_codes(host(q), codec.quantize_fp8_fixed(want, 56.0))

    q, s = pk.ops.layer_norm(xd, gd, bd, L.LN_E4M3_ROW, valid_rows=valid)
    wq, ws = O.quant_rows_fp8_dynamic(want, valid)
    assert np.allclose(host(s), ws, rtol=2e-3)
    _check_codes(host(q), wq, 2e-2)

    q, s = pk.ops.layer_norm(xd, gd, bd, L.LN_S8_ROW, valid_rows=valid)
    wq, ws = O.quant_rows_int8_dynamic(want, valid)
    assert np.allclose(host(s), ws, rtol=2e-3)
    _check_codes(host(q), wq, 2e-2)


def test_layer_norm_segments_and_ragged_valid(pk, cuda):
    L = pk.lib
    seg_stride, valid = 48, [48, 31, 0]
    x = _rows(20, seg_stride * 3, 1.5)
    g, b = _affine(5)
    sv = torch.tensor(valid, dtype=torch.int32, device=cuda)
    y, _ = pk.ops.layer_norm(dev16(x), dev16(g), dev16(b), L.LN_F16, seg_stride=seg_stride, seg_valid=sv)
    y = host(y)
    for s, v in enumerate(valid):
        blk = slice(s * seg_stride, (s + 1) * seg_stride)
        want = O.layer_norm(x[blk], g, b, v)
        assert np.max(np.abs(y[blk] - want)) <= 2.0 ** -7
        assert np.all(y[blk][v:] == 0)


def test_layer_norm_pair(pk, cuda):
    # kernels/sm89/encoder.cu:128-209: the second norm consumes the ROUNDED first output
    L = pk.lib
    x = _rows(30, 100, 2.0)
    g1, b1 = _affine(6)
    g2, b2 = _affine(7)
    first = O.layer_norm(x, g1, b1, 100)
    second = O.layer_norm(first, g2, b2, 100)
    y1, q2, _ = pk.ops.layer_norm_pair(dev16(x), dev16(g1), dev16(b1), dev16(g2), dev16(b2),
                                       L.LN_E4M3_FIXED, 56.0)
    assert np.max(np.abs(host(y1) - first)) <= 2.0 ** -7
    _check_codes(host(q2), codec.quantize_fp8_fixed(second, 56.0), 2e-2)


def test_glu_masked(pk, cuda):
    rng = np.random.default_rng(8)
    e = codec.f16_round(rng.standard_normal((80, 2048)) * 2.0)
    want = O.glu_masked(e, 80, 61)
    got = host(pk.ops.glu_masked(dev16(e), valid_rows=61))
    assert np.all(got[61:] == 0)
    assert np.max(np.abs(got - want)) <= 4e-3     # fast exp + one fp16 ulp


@pytest.mark.parametrize("seg_stride,valid", [(752, 750), (40, 33)])
def test_depthwise_bn_silu(pk, cuda, seg_stride, valid):
    rng = np.random.default_rng(9)
    segs = 2
    g = codec.f16_round(rng.standard_normal((segs * seg_stride, 1024)))
    for s in range(segs):
        g[s * seg_stride + valid:(s + 1) * seg_stride] = 0
    wdw = codec.f16_round(rng.standard_normal((1024, 9)) * 0.3)
    bn_g = (1 + 0.1 * rng.standard_normal(1024)).astype(np.float32)
    bn_b = (0.1 * rng.standard_normal(1024)).astype(np.float32)
    bn_m = (0.1 * rng.standard_normal(1024)).astype(np.float32)
    bn_v = (1 + 0.2 * rng.random(1024)).astype(np.float32)
    args = [dev16(g), dev16(wdw), dev(bn_g), dev(bn_b), dev(bn_m), dev(bn_v)]
    got, _ = pk.ops.depthwise_bn_silu(*args, quantize=False, seg_stride=seg_stride, valid_rows=valid)
    got = host(got)
    gq, gs = pk.ops.depthwise_bn_silu(*args, quantize=True, seg_stride=seg_stride, valid_rows=valid)
    gq, gs = host(gq), host(gs)
    for s in range(segs):
        blk = slice(s * seg_stride, (s + 1) * seg_stride)
        want = O.depthwise_bn_silu(g[blk], wdw, bn_g, bn_b, bn_m, bn_v, valid)
        assert np.max(np.abs(got[blk] - want)) <= 4e-3
        assert np.all(got[blk][valid:] == 0)
        # fused per-row E4M3 packing of the kernel's own fp16 result is bit exact
        wq, ws = O.quant_rows_fp8_dynamic(got[blk], valid)
        assert np.array_equal(gs[blk], ws)
        assert np.array_equal(gq[blk], wq)
