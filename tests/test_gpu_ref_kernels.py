"""Pins the CPU oracle against the REFERENCE'S OWN KERNELS executed on this GPU
(oracle/_ref/*.cubin, built from the reference checkout by oracle/build_ref.py)."""
import numpy as np
import pytest
import torch

from oracle import codec, decoder as D, ops as O, refkernels as R
from tests.util import dev, dev16, host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_ref():
    if not R.available():
        pytest.skip("oracle/_ref cubins were not built (reference checkout absent at build time)")


def test_layer_norm_and_fixed_quant(cuda):
    rng = np.random.default_rng(0)
    rows, padded = 751, 752
    x = codec.f16_round(rng.standard_normal((padded, 1024)) * 2)
    g = codec.f16_round(1 + 0.1 * rng.standard_normal(1024))
    b = codec.f16_round(0.1 * rng.standard_normal(1024))
    ref = R.layer_norm(dev16(x), dev16(g), dev16(b), rows, padded)
    want = O.layer_norm(x, g, b, rows)
    got = host(ref)
    assert np.max(np.abs(got - want)) <= 2.0 ** -7 and np.mean(got != want) < 2e-3
    # quantiser on identical fp16 input: bit exact against the oracle codec
    q = host(R.quantize_fp8_fixed(ref, 56.0))
    assert np.array_equal(q, codec.quantize_fp8_fixed(got, 56.0))


def test_ffn_expand_fp8(cuda):
    # the legacy mma.sync e4m3 path of the reference running on sm_100a
    rng = np.random.default_rng(1)
    rows = 752
    x = codec.f16_round(rng.standard_normal((rows, 1024)))
    w = codec.f16_round(rng.standard_normal((4096, 1024)) * 0.02)
    xq = codec.quantize_fp8_fixed(x, 56.0)
    wq, ws = codec.quantize_rows_fp8(w)
    ref = host(R.ffn_expand_fp8(dev(xq), dev(wq), dev(ws), rows))
    want = O.linear_fp8(xq, wq, ws, O.FP8_INPUT_SCALE, act=1)
    assert np.max(np.abs(ref - want)) <= 4e-3


def test_fp16_linear_reference_operands(cuda):
    m, n, k = 64, 1024, 1024
    x, w, b = O.reference_bench_operands(m, n, k)
    ref = host(R.fp16_linear(dev16(x), dev16(w), dev(b), None, m, n, k, 1.0, 0.0, 2))
    want = O.linear_f16(x, w, bias=b, act=2)
    assert np.max(np.abs(ref - want)) <= 4e-3        # reference gate is 0.02 (src/cuda.rs:848)


def test_glu_and_depthwise(cuda):
    rng = np.random.default_rng(2)
    rows, padded, valid = 300, 304, 299
    e = codec.f16_round(rng.standard_normal((padded, 2048)) * 2)
    ref = host(R.glu_masked(dev16(e), rows, padded, valid))
    assert np.max(np.abs(ref - O.glu_masked(e, rows, valid))) <= 4e-3
    g = ref
    wdw = codec.f16_round(rng.standard_normal((1024, 9)) * 0.3)
    bn = [(1 + 0.1 * rng.standard_normal(1024)).astype(np.float32), (0.1 * rng.standard_normal(1024)).astype(np.float32),
          (0.1 * rng.standard_normal(1024)).astype(np.float32), (1 + 0.2 * rng.random(1024)).astype(np.float32)]
    ref = host(R.depthwise_bn_silu(dev16(g), dev16(wdw), *[dev(t) for t in bn], rows, padded))
    want = O.depthwise_bn_silu(g, wdw, *bn, rows)
    assert np.max(np.abs(ref - want)) <= 4e-3


def test_scalar_attention(cuda):
    rng = np.random.default_rng(3)
    rows, padded, valid = 300, 304, 300
    q, k, v = [codec.f16_round(rng.standard_normal((padded, 1024))) for _ in range(3)]
    wpos = codec.f16_round(rng.standard_normal((1024, 1024)) * 0.02)
    u = codec.f16_round(rng.standard_normal((8, 128)) * 0.02)
    bv = codec.f16_round(rng.standard_normal((8, 128)) * 0.02)
    pos = O.position_table(wpos)
    ref = host(R.local_attention_scalar(dev16(q), dev16(k), dev16(v), dev16(pos), dev16(u), dev16(bv),
                                        rows, padded, valid))
    want = O.local_attention(q, k, v, pos, u, bv, rows, valid)
    assert np.max(np.abs(ref - want)) <= 3e-3


def test_tdt_decoder_tokens(cuda):
    # token ids must match exactly (src/cuda/decoder.rs:160-179) up to the first decision
    # whose top-2 margin is inside fp32 summation noise
    frames = 120
    w = D.make_decoder_weights(7, layers=2)
    rng = np.random.default_rng(8)
    enc = codec.f16_round(rng.standard_normal((frames, 640)) * 0.5)
    tokens, steps, ambiguous = D.tdt_greedy(enc, w, frames)
    dw = {}
    for key, val in w.items():
        if key == "layers":
            continue
        dw[key] = dev(val) if key.startswith("b_") else dev16(val)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ref = R.tdt_decode(dev16(enc), dw, frames, sms)
    n = len(tokens) if ambiguous is None else ambiguous
    assert n > 20
    assert np.array_equal(ref[:n], tokens[:n])
    if ambiguous is None:
        assert len(ref) == len(tokens)
