"""GPU parity: local relative-position attention vs the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import codec, ops as O
from tests.util import dev16, host

pytestmark = pytest.mark.gpu


def _case(seed, rows):
    rng = np.random.default_rng(seed)
    q = codec.f16_round(rng.standard_normal((rows, 1024)))
    k = codec.f16_round(rng.standard_normal((rows, 1024)))
    v = codec.f16_round(rng.standard_normal((rows, 1024)))
    wpos = codec.f16_round(rng.standard_normal((1024, 1024)) * 0.02)
    u = codec.f16_round(rng.standard_normal((8, 128)) * 0.02)
    bv = codec.f16_round(rng.standard_normal((8, 128)) * 0.02)
    pos = O.position_table(wpos)
    return q, k, v, pos, u, bv


@pytest.mark.parametrize("impl", ["mma", "simple"])
@pytest.mark.parametrize("rows,valid", [(304, 300), (40, 33), (752, 750), (768, 750), (1, 1), (130, 129)])
def test_kernels_match_oracle(pk, cuda, rows, valid, impl):
    q, k, v, pos, u, bv = _case(rows, rows)
    want = O.local_attention(q, k, v, pos, u, bv, rows, valid)
    fn = pk.ops.local_attention if impl == "mma" else pk.ops.local_attention_simple
    got = host(fn(dev16(q), dev16(k), dev16(v), dev16(pos), dev16(u), dev16(bv), valid_rows=valid))
    assert np.all(got[valid:] == 0)
    # tolerance: fp16 output ulp + fp16-rounded probabilities / position scores (mma kernel)
    assert np.max(np.abs(got - want)) <= 3e-3, np.max(np.abs(got - want))


def test_large_scores_do_not_overflow(pk, cuda):
    # queries/keys 4x larger: scores of a few hundred before scaling, softmax nearly one-hot
    q, k, v, pos, u, bv = _case(77, 200)
    q, k = q * 4, k * 4
    want = O.local_attention(q, k, v, pos, u, bv, 200, 200)
    got = host(pk.ops.local_attention(dev16(q), dev16(k), dev16(v), dev16(pos), dev16(u), dev16(bv)))
    assert np.all(np.isfinite(got))
    assert np.max(np.abs(got - want)) <= 2e-2


def test_fused_qkv_strides_and_segments(pk, cuda):
    seg, valid = 272, [272, 150]
    q, k, v, pos, u, bv = _case(5, 2 * seg)
    qkv = np.concatenate([q, k, v], axis=1)
    t = dev16(qkv)
    sv = torch.tensor(valid, dtype=torch.int32, device=cuda)
    for fn in (pk.ops.local_attention, pk.ops.local_attention_simple):
        got = host(fn(t[:, :1024], t[:, 1024:2048], t[:, 2048:], dev16(pos), dev16(u), dev16(bv),
                      seg_stride=seg, seg_valid=sv))
        _check_segments(got, q, k, v, pos, u, bv, seg, valid)


def _check_segments(got, q, k, v, pos, u, bv, seg, valid):
    for s, val in enumerate(valid):
        blk = slice(s * seg, (s + 1) * seg)
        want = O.local_attention(q[blk], k[blk], v[blk], pos, u, bv, seg, val)
        assert np.max(np.abs(got[blk] - want)) <= 3e-3
        assert np.all(got[blk][val:] == 0)


def test_pack_position_heads(pk, cuda):
    rng = np.random.default_rng(6)
    p = codec.f16_round(rng.standard_normal((272, 1024)))
    got = host(pk.ops.pack_position_heads(dev16(p)))
    assert np.array_equal(got, p.reshape(272, 8, 128).transpose(1, 0, 2))


@pytest.mark.parametrize("rows,valid", [(128, 128), (128, 33), (256, 250), (768, 750), (1536, 1411), (384, 1)])
def test_tcgen05_kernel_matches_oracle(pk, cuda, rows, valid):
    """The hot-path kernel (tcgen05.mma, accumulators in tensor memory) against the same oracle and
    tolerance as the mma.sync kernel; pad rows zero; no bounded wait expires."""
    q, k, v, pos, u, bv = _case(1000 + rows + valid, rows)
    want = O.local_attention(q, k, v, pos, u, bv, rows, valid)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    got = host(pk.ops.local_attention_tcgen05(dev16(q), dev16(k), dev16(v), dev16(pos), dev16(u), dev16(bv),
                                              valid_rows=valid, status=st))
    assert int(st.item()) == 0
    assert np.all(got[valid:] == 0) and np.all(np.isfinite(got))
    assert np.max(np.abs(got - want)) <= 3e-3, np.max(np.abs(got - want))


def test_tcgen05_kernel_segments_strides_and_large_scores(pk, cuda):
    seg, valid = 384, [384, 150, 257]
    q, k, v, pos, u, bv = _case(9, 3 * seg)
    qkv = dev16(np.concatenate([q, k, v], axis=1))
    sv = torch.tensor(valid, dtype=torch.int32, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    got = host(pk.ops.local_attention_tcgen05(qkv[:, :1024], qkv[:, 1024:2048], qkv[:, 2048:], dev16(pos), dev16(u),
                                              dev16(bv), seg_stride=seg, seg_valid=sv, status=st))
    assert int(st.item()) == 0
    _check_segments(got, q, k, v, pos, u, bv, seg, valid)
    # it agrees with the mma.sync kernel far inside the oracle tolerance
    other = host(pk.ops.local_attention(qkv[:, :1024], qkv[:, 1024:2048], qkv[:, 2048:], dev16(pos), dev16(u),
                                        dev16(bv), seg_stride=seg, seg_valid=sv))
    assert np.max(np.abs(got - other)) <= 2e-3
    # scores of a few hundred before scaling
    q4, k4 = q[:seg] * 4, k[:seg] * 4
    want = O.local_attention(q4, k4, v[:seg], pos, u, bv, seg, seg)
    big = host(pk.ops.local_attention_tcgen05(dev16(q4), dev16(k4), dev16(v[:seg]), dev16(pos), dev16(u), dev16(bv)))
    assert np.all(np.isfinite(big)) and np.max(np.abs(big - want)) <= 2e-2
    # a stride that is no multiple of 128 is refused (the caller takes the other kernel)
    with pytest.raises(pk.lib.Pk100Error):
        pk.ops.local_attention_tcgen05(dev16(q[:200]), dev16(k[:200]), dev16(v[:200]), dev16(pos), dev16(u), dev16(bv))
