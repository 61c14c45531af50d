"""The frontend oracle against the reference's own unit tests (src/frontend.rs:273-315)."""
import numpy as np

from oracle import frontend as F


def fixture():
    """fixture_frontend (src/frontend.rs:305-314): unit window, one bin per filter."""
    filters = np.zeros((128, 257), np.float32)
    for mel in range(128):
        filters[mel, mel % 257] = 1.0
    return np.ones(400, np.float32), filters


def test_masks_the_extra_centered_frame_at_boundary_lengths():
    window, filters = fixture()
    for samples, frames, valid in [(1, 1, 0), (159, 1, 0), (160, 2, 1), (161, 2, 1), (320, 3, 2)]:
        x = np.sin(np.arange(samples, dtype=np.float32) * np.float32(0.01))
        out, got_valid = F.compute(x, window, filters)
        assert (out.shape[0], got_valid) == (frames, valid)
        assert np.all(np.isfinite(out))
        assert not out[valid:].any()


def test_empty_audio_has_no_frames():
    out, valid = F.compute(np.zeros(0, np.float32), *fixture())
    assert out.shape == (0, 128) and valid == 0


def test_framing_and_normalisation_identities():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(2000).astype(np.float32)
    w512 = F.center_window(F.hann_window())
    assert w512[:56].sum() == 0 and w512[456:].sum() == 0 and w512[56] == 0 and w512[256] == 1.0
    fr = F.framed(x, w512)
    assert fr.shape == (13, 512)
    # frame 2, tap 300 holds sample 2*160 + 300 - 256 with pre-emphasis
    s = 2 * 160 + 300 - 256
    assert fr[2, 300] == np.float32((np.float64(x[s]) - np.float64(np.float32(0.97)) * np.float64(x[s - 1])) *
                                    np.float64(w512[300]))
    assert fr[0, 255] == 0.0                                   # left padding of the centred first frame
    out, valid = F.compute(x, F.hann_window(), F.triangular_filters())
    assert valid == 12 and np.allclose(out[:valid].mean(axis=0), 0, atol=1e-5)
    assert np.allclose(out[:valid].std(axis=0, ddof=1), 1, atol=1e-3)
