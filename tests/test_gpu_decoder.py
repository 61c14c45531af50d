"""GPU parity: batched TDT greedy decode vs the CPU oracle (itself pinned to the
reference's decoder kernel in test_gpu_ref_kernels.py).  Token ids must match exactly
(src/cuda/decoder.rs:160-179) up to the first decision whose top-2 margin is inside
fp32 summation noise."""
import numpy as np
import pytest
import torch

from oracle import codec, decoder as D
from tests.util import dev16, host

pytestmark = pytest.mark.gpu


def _check(tokens_gpu, count, oracle_tokens, ambiguous):
    n = len(oracle_tokens) if ambiguous is None else ambiguous
    assert np.array_equal(tokens_gpu[:min(n, count)], oracle_tokens[:min(n, count)])
    if ambiguous is None:
        assert count == len(oracle_tokens)
    return n


@pytest.mark.parametrize("kernel", [None, "cluster", "exchange", "barrier"])
@pytest.mark.parametrize("layers", [2, 1])
def test_batched_decode_matches_oracle(pk, cuda, layers, kernel):
    w = D.make_decoder_weights(11 + layers, layers=layers)
    dec = pk.decoder.TdtDecoder(w, cuda)
    seg_stride, frames = 96, [96, 60, 1, 0, 33]
    rng = np.random.default_rng(5)
    enc = codec.f16_round(rng.standard_normal((len(frames) * seg_stride, 640)) * 0.5)
    fr = torch.tensor(frames, dtype=torch.int32, device=cuda)
    tokens, durations, counts = dec.decode(dev16(enc), len(frames), seg_stride, fr, seg_stride * 10,
                                           kernel=kernel)
    torch.cuda.synchronize()
    assert int(dec.status.item()) == 0
    tokens, counts, durations = host(tokens), host(counts), host(durations)
    checked = 0
    for u, f in enumerate(frames):
        want, steps, amb = D.tdt_greedy(enc[u * seg_stride:(u + 1) * seg_stride], w, f)
        checked += _check(tokens[u], int(counts[u]), want, amb)
        if amb is None:
            emitted = [s for s in steps if s[1] != D.BLANK]
            assert [s[2] for s in emitted] == list(durations[u][:len(emitted)])
    assert counts[3] == 0 and checked > 50


def test_encoder_projection_and_full_length(pk, cuda):
    # 60 s worth of frames for two utterances, encoder projection through the fp16 GEMM
    w = D.make_decoder_weights(21, layers=2)
    dec = pk.decoder.TdtDecoder(w, cuda)
    seg_stride, frames = 768, [750, 750]
    rng = np.random.default_rng(6)
    encoded = codec.f16_round(rng.standard_normal((2 * seg_stride, 1024)))
    proj = dec.project(dev16(encoded))
    want_proj = codec.f16_round(
        np.asarray(encoded, np.float64) @ w["w_enc"].astype(np.float64).T + w["b_enc"])
    assert np.max(np.abs(host(proj) - want_proj)) <= 4e-3
    fr = torch.tensor(frames, dtype=torch.int32, device=cuda)
    tokens, _, counts = dec.decode(proj, 2, seg_stride, fr, 7500)
    torch.cuda.synchronize()
    assert int(dec.status.item()) == 0
    gp = host(proj)
    for u in range(2):
        want, _, amb = D.tdt_greedy(gp[u * seg_stride:(u + 1) * seg_stride], w, frames[u])
        n = _check(host(tokens)[u], int(host(counts)[u]), want, amb)
        assert n > 100


def test_decoder_limits(pk, cuda):
    L = pk.lib
    assert L.lib.pk100_tdt_workspace_bytes(9) == 0
    w = D.make_decoder_weights(1, layers=2)
    dec = pk.decoder.TdtDecoder(w, cuda)
    fr = torch.zeros(9, dtype=torch.int32, device=cuda)
    enc = torch.zeros((9 * 8, 640), dtype=torch.float16, device=cuda)
    with pytest.raises(L.Pk100Error):
        dec.decode(enc, 9, 8, fr, 16)


@pytest.mark.parametrize("layers", [1, 2])
def test_eight_utterances_all_kernels_agree(pk, cuda, layers):
    """Full batch width; the cluster, exchange and barrier kernels walk the same decisions."""
    w = D.make_decoder_weights(31, layers=layers)
    dec = pk.decoder.TdtDecoder(w, cuda)
    seg_stride = 128
    frames = [128, 100, 90, 128, 5, 64, 77, 128]
    rng = np.random.default_rng(9)
    enc = dev16(codec.f16_round(rng.standard_normal((8 * seg_stride, 640)) * 0.5))
    fr = torch.tensor(frames, dtype=torch.int32, device=cuda)
    results = []
    for kernel in ("cluster", "exchange", "barrier"):
        t, d, c = dec.decode(enc, 8, seg_stride, fr, 1280, kernel=kernel)
        torch.cuda.synchronize()
        assert int(dec.status.item()) == 0
        results.append((host(t).copy(), host(c).copy()))
    enc_h = host(enc)
    total = 0
    for u in range(8):
        want, _, amb = D.tdt_greedy(enc_h[u * seg_stride:(u + 1) * seg_stride], w, frames[u])
        n = len(want) if amb is None else amb
        for t, c in results:
            assert np.array_equal(t[u][:min(n, c[u])], want[:min(n, c[u])])
            if amb is None:
                assert c[u] == len(want)
        total += n
    assert total > 100
