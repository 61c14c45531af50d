"""GPU parity of the log-mel frontend: the oracle against the reference's own frontend kernels
on this GPU, then pk100_mel_frontend against the oracle.

Tolerance (stated): the fused kernel runs its 512-point FFT in fp32 (like the reference's cuFFT
plan) while the oracle transforms in double precision: |difference| <= 2e-3 on the normalised
features (unit variance per mel bin), <= 2e-4 on the un-normalised log-mel."""
import numpy as np
import pytest
import torch

from oracle import frontend as F
from oracle import refkernels as R
from tests.util import dev, host

pytestmark = pytest.mark.gpu


def test_oracle_matches_reference_frontend_kernels(cuda):
    if not R.frontend_available():
        pytest.skip("oracle/_ref/frontend.cubin was not built")
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(4000) * 0.3).astype(np.float32)
    frames, valid = F.frame_counts(x.size)
    w512 = F.center_window(F.hann_window())
    offsets, bins, values = F.sparse_filters(F.triangular_filters())
    want_frames = F.framed(x, w512)
    got_frames = host(R.frame_window(dev(x), dev(w512), frames))
    assert np.max(np.abs(got_frames - want_frames)) <= 1e-6            # fp32 vs double pre-emphasis
    # the reference's mel kernel on the oracle's own spectrum (cuFFT is not part of the cubin)
    spec = np.fft.rfft(want_frames.astype(np.float64), axis=1)
    spec2 = np.stack([spec.real, spec.imag], axis=-1).astype(np.float32)
    got_mel = host(R.mel_log_sparse(dev(spec2), dev(offsets), dev(bins), dev(values), frames, float(F.LOG_ZERO_GUARD)))
    want_mel = F.log_mel(want_frames, offsets, bins, values)
    assert np.max(np.abs(got_mel - want_mel)) <= 1e-4
    got_norm = host(R.normalize_mel(dev(want_mel), frames, valid, float(F.NORMALIZE_EPSILON)))
    assert np.max(np.abs(got_norm - F.normalize(want_mel, valid))) <= 1e-5
    assert not got_norm[valid:].any()


def test_fused_frontend_matches_oracle(pk, cuda):
    rng = np.random.default_rng(1)
    lengths = [16000, 1, 159, 160, 161, 320, 5003, 0]
    stride = 16000
    pcm = np.zeros((len(lengths), stride), np.float32)
    for u, n in enumerate(lengths):
        t = np.arange(n, dtype=np.float32)
        pcm[u, :n] = (0.3 * rng.standard_normal(n) + 0.2 * np.sin(t * np.float32(0.05 + 0.01 * u))).astype(np.float32)
    window, filters = F.hann_window(), F.triangular_filters()
    fe = pk.frontend.MelFrontend(window, filters, cuda)
    counts = torch.tensor(lengths, dtype=torch.int32, device=cuda)
    mel, valid = fe.compute(dev(pcm), counts)
    torch.cuda.synchronize()
    mel, valid = host(mel), host(valid)
    assert mel.shape == (len(lengths), stride // 160 + 1, 128)
    for u, n in enumerate(lengths):
        want, want_valid = F.compute(pcm[u, :n], window, filters)
        assert valid[u] == want_valid and pk.frontend.frames_for(n) == want.shape[0]
        assert not mel[u, want_valid:].any()                              # masked frame and padding rows
        if want_valid > 1:
            assert np.max(np.abs(mel[u, :want_valid] - want[:want_valid])) <= 2e-3
        elif want_valid == 1:
            assert not mel[u, 0].any()                                     # one frame: (x - mean) = 0
    # un-normalised log-mel of the long utterance: run with epsilon = 1 and undo the
    # normalisation with the oracle's own statistics
    fe_raw = pk.frontend.MelFrontend(window, filters, cuda, normalize_epsilon=1.0)
    raw, _ = fe_raw.compute(dev(pcm[:1]), counts[:1])
    torch.cuda.synchronize()
    offsets, bins, values = F.sparse_filters(filters)
    whole = F.log_mel(F.framed(pcm[0], F.center_window(window)), offsets, bins, values).astype(np.float64)
    n_valid = F.frame_counts(16000)[1]
    mean, var = whole[:n_valid].mean(axis=0), whole[:n_valid].var(axis=0, ddof=1)
    restored = host(raw)[0, :n_valid].astype(np.float64) * (np.sqrt(var) + 1.0) + mean
    assert np.max(np.abs(restored - whole[:n_valid])) <= 2e-4


def test_frontend_feeds_subsampling_and_rejects_bad_arguments(pk, cuda):
    rng = np.random.default_rng(2)
    pcm = dev((rng.standard_normal((2, 4800)) * 0.3).astype(np.float32))
    counts = torch.tensor([4800, 3000], dtype=torch.int32, device=cuda)
    fe = pk.frontend.MelFrontend(F.hann_window(), F.triangular_filters(), cuda)
    mel, valid = fe.compute(pcm, counts)
    sub = pk.subsampling.Subsampling(pk.synth.subsampling_weights(1), cuda)
    out = sub.run(mel, 8, mel_frames=valid)
    torch.cuda.synchronize()
    rows = pk.subsampling.output_frames(30)
    assert host(valid).tolist() == [30, 18] and rows == 4
    assert np.abs(host(out)[:rows]).max() > 0 and np.all(np.isfinite(host(out)))
    with pytest.raises(pk.lib.Pk100Error):
        fe.compute(pcm, counts, frame_cap=10)                              # 4800 samples need 31 rows


def test_pipeline_from_pcm_equals_pipeline_from_its_own_mel(pk, cuda):
    """PCM entry point = frontend + the mel entry point (same tokens), variable lengths."""
    rng = np.random.default_rng(3)
    eng = pk.pipeline.PipelineEngine(cuda, layers=2, decoder_layers=1, seed=5, max_utterances=2, mel_frames=201)
    eng.attach_frontend(F.hann_window(), F.triangular_filters())
    counts = [32000, 20011]
    pcm = np.zeros((2, 32000), np.float32)
    for u, n in enumerate(counts):
        pcm[u, :n] = (0.3 * rng.standard_normal(n)).astype(np.float32)
    got = eng.transcribe_pcm(torch.from_numpy(pcm), counts)
    mel = host(eng.mel_dev).copy()
    valid = [n // 160 for n in counts]
    for u in range(2):
        want, v = F.compute(pcm[u, :counts[u]], F.hann_window(), F.triangular_filters())
        assert v == valid[u] and np.max(np.abs(mel[u, :v] - want[:v])) <= 2e-3 and not mel[u, v:].any()
    again = eng.transcribe_batch(torch.from_numpy(mel), valid)
    assert all(np.array_equal(a, b) for a, b in zip(got, again)) and sum(len(t) for t in got) > 10
    # a mel request right after a PCM request with short clips does not inherit their lengths:
    # without lengths it covers all 201 frames of the mel it is given
    eng.transcribe_pcm(torch.from_numpy(pcm[:, :8000].copy()), [8000, 4000])
    assert eng.longest_out_frames < eng.frames_out
    full = eng.transcribe_batch(torch.from_numpy(mel))
    assert eng.longest_out_frames == eng.frames_out
    want_full = eng.transcribe_batch(torch.from_numpy(mel), [201, 201])
    assert all(np.array_equal(a, b) for a, b in zip(full, want_full))
