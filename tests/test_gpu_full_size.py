"""Full-size cases of the benchmark configurations, checked through size-independent
properties and windowed oracle comparisons (the CPU oracle is too slow to run them whole).

  * configuration 2: local relative-position MHSA at T = 45 000 (one hour of audio) inside a
    complete encoder block; a block's receptive field is +-132 rows (attention +-128, depthwise
    +-4), so the oracle is run on 128-aligned windows and compared at their centres;
  * configurations 3 / 4: the 24-block encoder + TDT decode on 60 s utterances: an utterance
    transcribed inside a batch gives exactly the tokens it gives alone, twice in a row."""
import numpy as np
import pytest
import torch

from oracle import codec, ops as O
from tests.util import dev16, host, nrmse

pytestmark = pytest.mark.gpu


def test_one_hour_block_matches_windowed_oracle(pk, cuda):
    t_valid, rows = 45000, 45056                     # 352 tiles of 128 rows
    w = pk.synth.layer_weights(12, 0, randomize_norms=True)
    p = O.prepare_layer(w)
    g = torch.Generator().manual_seed(2)
    x = torch.randn((rows, 1024), generator=g).half()
    x[t_valid:] = 0
    enc = pk.encoder.EncoderLayers(cuda)
    enc.add_layer(w, 0.0, 0.0)                       # dense hidden: windows need no global threshold
    arena, ws = enc.make_workspace(rows)
    a, b = x.to(cuda), torch.zeros((rows, 1024), dtype=torch.float16, device=cuda)
    out = enc.run(a, b, ws, 1, rows, t_valid)
    torch.cuda.synchronize()
    assert enc.status(arena, ws) == 0
    got = host(out)
    assert np.all(got[t_valid:] == 0) and np.all(np.isfinite(got))
    xh = x.float().numpy()
    for start, length in ((0, 512), (22016, 512), (44544, 512)):
        stop = min(start + length, rows)
        valid = min(t_valid, stop) - start
        want = O.encoder_layer(xh[start:stop], p, valid, 0.0, 0.0)
        lo = 0 if start == 0 else 136                # rows whose receptive field lies inside the window
        hi = valid if stop >= t_valid else valid - 136
        assert nrmse(got[start + lo:start + hi], want[lo:hi]) <= 1e-2
        assert np.max(np.abs(got[start + lo:start + hi] - want[lo:hi])) <= 0.15


@pytest.fixture(scope="module")
def full_engine(pk, cuda):
    eng = pk.pipeline.PipelineEngine(cuda, layers=24, decoder_layers=1, seed=4, max_utterances=8, mel_frames=6000)
    mel = torch.from_numpy(np.stack([pk.synth.mel_input(100 + u, 6000) for u in range(8)])).pin_memory()
    eng.mel_dev.copy_(mel)
    eng.calibrate(8)
    return eng, mel


def test_sixty_second_batch_is_batch_invariant_and_deterministic(pk, cuda, full_engine):
    eng, mel = full_engine
    first = eng.transcribe_batch(mel)
    second = eng.transcribe_batch(mel)
    assert eng.status() == 0
    assert all(np.array_equal(x, y) for x, y in zip(first, second))
    assert all(0 < len(t) <= eng.max_tokens and t.min() >= 0 and t.max() < 1024 for t in first)
    # utterances 3 and 5 alone (a batch of two, different slots) decode to the same tokens
    pair = eng.transcribe_batch(mel[[3, 5]].contiguous().pin_memory())
    assert np.array_equal(pair[0], first[3]) and np.array_equal(pair[1], first[5])
    # encoder rows beyond each utterance's 750 frames are zero, rows inside are finite
    eng.mel_dev.copy_(mel)
    encoded = host(eng.encode(8))
    for u in range(8):
        blk = encoded[u * eng.seg_stride:(u + 1) * eng.seg_stride]
        assert np.all(blk[eng.frames_out:] == 0) and np.all(np.isfinite(blk))
        assert np.std(blk[:eng.frames_out]) > 0.1


def test_tile_thresholds_drop_seventy_percent_of_the_tiles(pk, cuda, full_engine):
    eng, mel = full_engine
    eng.mel_dev.copy_(mel)
    eng.sub.run(eng.mel_dev, eng.seg_stride, mel_frames=eng.mel_frames_dev, out=eng.state_a)
    tiles = eng.rows // 128 * 64
    stats = torch.zeros((2 * len(eng.enc.layers), tiles), dtype=torch.float32, device=cuda)
    eng.enc.run(eng.state_a, eng.state_b, eng.ws, 8, eng.seg_stride, eng.frames_out,
                seg_valid=eng.out_frames_dev, tile_stats=stats)
    st = host(stats).reshape(len(eng.enc.layers), 2, -1, 64)
    for l, lw in enumerate(eng.enc.layers):
        for which, tau in ((0, lw.ff1.tau), (1, lw.ff2.tau)):
            zero_fraction = float((st[l, which] < tau).mean())
            assert 0.62 <= zero_fraction <= 0.78, (l, which, zero_fraction)


def test_twenty_four_blocks_match_the_oracle_layer_by_layer(pk, cuda, full_engine):
    """Benchmark configuration 3 at its real depth: one 60 s utterance (T = 750, 768-row segment),
    the benchmarked weights (seed 4) and the calibrated tile thresholds.  Every block's output is
    held to nRMSE <= 1e-2 against the oracle run on the SAME block input (the GPU's own), the
    free-running oracle stack (tile decisions taken from the GPU run: a threshold is a discontinuous
    operator) to the reference's layer-stack gate nRMSE <= 3e-2 (src/cuda/encoder.rs:204-239), and
    the tokens decoded from the GPU's projection of its own encoder output are exact."""
    from oracle import decoder as D
    from tests.test_gpu_encoder import _oracle_layer_same_decisions
    eng, mel = full_engine
    eng.mel_dev.copy_(mel)
    rows, valid = eng.seg_stride, eng.frames_out
    eng.sub.run(eng.mel_dev[:1], eng.seg_stride, mel_frames=eng.mel_frames_dev, out=eng.state_a)
    cur = host(eng.state_a[:rows]).copy()
    cur[valid:] = 0                      # rows past the utterance are "don't care" after subsampling: every consumer masks them
    arena, ws = eng.enc.make_workspace(rows)
    free = cur.copy()
    worst = 0.0
    for l, lw in enumerate(eng.enc.layers):
        p = O.prepare_layer(pk.synth.layer_weights(4, l))
        a, b = dev16(cur), torch.zeros((rows, 1024), dtype=torch.float16, device=cuda)
        stats = torch.zeros((2, rows // 128 * 64), dtype=torch.float32, device=cuda)
        out = host(eng.enc.run(a, b, ws, 1, rows, valid, tile_stats=stats, first=l, count=1)).copy()
        st = host(stats).reshape(2, -1, 64)
        want, _ = _oracle_layer_same_decisions(cur, p, valid, lw.ff1.tau, lw.ff2.tau, st)
        err = nrmse(out[:valid], want[:valid])
        worst = max(worst, err)
        assert err <= 1e-2, (l, err)
        free = O.encoder_layer(free, p, valid, lw.ff1.tau, lw.ff2.tau,
                               keep1=(st[0] >= lw.ff1.tau).astype(np.uint8), keep2=(st[1] >= lw.ff2.tau).astype(np.uint8))
        cur = out
    assert eng.enc.status(arena, ws) == 0
    stack = nrmse(cur[:valid], free[:valid])
    print(f"24 blocks: worst per-layer nRMSE {worst:.2e}, free-running stack nRMSE {stack:.2e}")
    assert stack <= 3e-2
    # one call over the 24 blocks gives the layer-by-layer result bit for bit
    eng.sub.run(eng.mel_dev[:1], eng.seg_stride, mel_frames=eng.mel_frames_dev, out=eng.state_a)
    whole = eng.enc.run(eng.state_a[:rows], eng.state_b[:rows], ws, 1, rows, valid)
    assert np.array_equal(host(whole), cur)
    # tokens: the GPU decoder on the GPU's projection against the oracle decoder on the same rows
    proj = eng.dec.project(whole)
    frames = torch.tensor([valid], dtype=torch.int32, device=cuda)
    tokens, _, counts = eng.dec.decode(proj, 1, rows, frames, eng.max_tokens)
    torch.cuda.synchronize()
    got = host(tokens)[0][:int(host(counts)[0])]
    want_tokens, _, amb = D.tdt_greedy(host(proj)[:valid], pk.synth.decoder_weights(4, 1), valid)
    n = len(want_tokens) if amb is None else amb
    assert n > 20 and np.array_equal(got[:n], want_tokens[:n])
