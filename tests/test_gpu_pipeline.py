"""GPU parity: the whole path (subsampling -> blocks -> projection -> TDT decode) through the
public pipeline API vs the CPU oracle, on a reduced model (2 blocks, short utterances)."""
import numpy as np
import pytest
import torch

from oracle import decoder as D, ops as O, pipeline as P
from tests.util import nrmse

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def engine(pk, cuda):
    eng = pk.pipeline.PipelineEngine(cuda, layers=2, decoder_layers=2, seed=9, max_utterances=3,
                                     mel_frames=1000, randomize_norms=True)
    return eng


def _weights(pk, eng):
    sub_w = pk.synth.subsampling_weights(9)
    layers = [O.prepare_layer(pk.synth.layer_weights(9, l, randomize_norms=True)) for l in range(2)]
    dec_w = pk.synth.decoder_weights(9, 2)
    return sub_w, layers, dec_w


def test_transcribe_batch_matches_oracle(pk, cuda, engine):
    eng = engine
    frames = [1000, 1000, 1000]
    mels = np.stack([pk.synth.mel_input(100 + u, 1000) for u in range(3)])
    mel_host = torch.from_numpy(mels).pin_memory()
    # tile thresholds stay 0 here: the free-running stack is compared as a continuous
    # operator (per-block parity WITH thresholds is covered in test_gpu_encoder.py)
    tokens = eng.transcribe_batch(mel_host)
    assert eng.status() == 0
    sub_w, layers, dec_w = _weights(pk, eng)
    taus = [(eng.enc.layers[l].ff1.tau, eng.enc.layers[l].ff2.tau) for l in range(2)]
    for u in range(3):
        want_tokens, want_enc, amb = P.transcribe(mels[u], sub_w, layers, taus, dec_w)
        # encoder output of the free-running 2-block stack: reference's stack gate
        blk = slice(u * eng.seg_stride, u * eng.seg_stride + eng.frames_out)
        got_proj = eng.enc_proj[blk].float().cpu().numpy()
        want_proj = P.project(want_enc, dec_w)
        assert nrmse(got_proj, want_proj) <= 3e-2
        # token ids: exact on the SAME encoder projection (the GPU's), up to the first
        # decision inside fp32 summation noise
        same_tokens, _, amb2 = D.tdt_greedy(got_proj, dec_w, eng.frames_out)
        n = len(same_tokens) if amb2 is None else amb2
        assert n > 10
        assert np.array_equal(tokens[u][:n], same_tokens[:n])
        if amb2 is None:
            assert len(tokens[u]) == len(same_tokens)


def test_resident_path_is_deterministic_and_ragged_lengths(pk, cuda, engine):
    eng = engine
    frames = [1000, 617, 40]
    mels = np.zeros((3, 1000, 128), np.float32)
    for u, f in enumerate(frames):
        mels[u, :f] = pk.synth.mel_input(200 + u, f)
    mel_host = torch.from_numpy(mels).pin_memory()
    eng.set_lengths(frames)
    eng.mel_dev.copy_(mel_host)
    eng.calibrate(3)                       # 70 % zero tiles from here on
    assert all(l.ff1.tau > 0 and l.ff2.tau > 0 for l in eng.enc.layers)
    a = eng.transcribe_batch(mel_host, frames)
    b = eng.transcribe_batch(mel_host, frames)
    assert all(np.array_equal(x, y) for x, y in zip(a, b))
    # a shorter utterance in a batch decodes like the same utterance alone
    solo = eng.transcribe_batch(torch.from_numpy(np.stack([mels[1]] * 3)).pin_memory(), [617, 617, 617])
    assert np.array_equal(solo[0], a[1])
    # a request without lengths means "all frames": nothing is inherited from the request before
    full = eng.transcribe_batch(mel_host)
    assert tuple(eng.out_frames_host.tolist()) == (eng.frames_out,) * 3
    again = eng.transcribe_batch(mel_host, [1000, 1000, 1000])
    assert all(np.array_equal(x, y) for x, y in zip(full, again))
    # and the schedule changes no token: one group for everything, or two encode groups whose
    # decodes run under the next group's encode (the engine above: one encode pass, a decoder
    # cluster per utterance)
    assert eng.encode_groups == 1 and eng.decode_groups == 3
    for enc_groups, dec_groups in ((1, 1), (2, 2), (2, 3)):
        other = pk.pipeline.PipelineEngine(cuda, layers=2, decoder_layers=2, seed=9, max_utterances=3, mel_frames=1000,
                                           randomize_norms=True, encode_groups=enc_groups, decode_groups=dec_groups)
        for l, lw in enumerate(eng.enc.layers):
            other.enc.set_tau(l, lw.ff1.tau, lw.ff2.tau)
        got = other.transcribe_batch(mel_host, frames)
        assert other.status() == 0 and all(np.array_equal(x, y) for x, y in zip(got, a))
        assert len(other.last_groups) == dec_groups and len(other.last_encode_groups) == enc_groups


def test_streamed_batches_return_what_single_requests_return(pk, cuda, engine):
    """transcribe_stream (batch i + 1 encoded beside the decode of batch i, two alternating sets
    of request buffers) yields, in order, exactly the tokens of one transcribe_batch per batch."""
    eng = engine
    rng = np.random.default_rng(5)
    batches, want = [], []
    for i in range(5):
        n = 1 + i % 3
        frames = [int(f) for f in rng.integers(40, 1001, size=n)]
        mels = np.zeros((n, 1000, 128), np.float32)
        for u, f in enumerate(frames):
            mels[u, :f] = pk.synth.mel_input(300 + 10 * i + u, f)
        batches.append((torch.from_numpy(mels).pin_memory(), frames))
    for mel, frames in batches:
        want.append(eng.transcribe_batch(mel, frames))
    for depth, groups in ((2, 2), (3, 1)):
        got = list(eng.transcribe_stream(iter(batches), decode_groups=groups, depth=depth))
        assert len(got) == len(want) and eng.status() == 0
        for g, w in zip(got, want):
            assert len(g) == len(w) and all(np.array_equal(x, y) for x, y in zip(g, w))
    assert any(len(t) > 0 for batch in got for t in batch)
