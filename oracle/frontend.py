"""CPU restatement of the reference's log-mel frontend.  TEST INFRASTRUCTURE ONLY.

Follows CpuMelFrontend::compute (src/frontend.rs:114-215): centred 512-sample frames every 160
samples (frames = n / 160 + 1, the last one masked: valid = n / 160), pre-emphasis 0.97 in
double precision, windowed value rounded to fp32, DFT in double precision with the spectrum
rounded to fp32, power spectrum, sparse mel filters summed in double, ln(sum + 2^-24) as
fp32, then per-feature normalisation over the valid frames (mean, unbiased variance, double).
Pinned to the reference's unit tests src/frontend.rs:273-300 (frame counts and masked rows at
the boundary lengths 1, 159, 160, 161, 320; empty audio) and, on the GPU, to the reference's
own kernels pk_sm89_frame_window / _mel_log_sparse / _normalize_mel (kernels/sm89/frontend.cu)
through oracle/refkernels.py.  The DFT is numpy's rfft instead of the reference's radix-2
loop: both are double-precision transforms of the same fp32 input, so they agree to ~1e-13
before the rounding to fp32."""
from __future__ import annotations

import numpy as np

N_FFT, HOP, N_MELS, WIN = 512, 160, 128, 400
PREEMPHASIS = np.float32(0.97)
LOG_ZERO_GUARD = np.float32(2.0 ** -24)
NORMALIZE_EPSILON = np.float32(1e-5)


def center_window(window):
    """src/frontend.rs:218-223."""
    window = np.asarray(window, np.float32)
    out = np.zeros(N_FFT, np.float32)
    left = (N_FFT - window.size) // 2
    out[left:left + window.size] = window
    return out


def sparse_filters(mel_filters):
    """Row-wise non-zeros of the [128, 257] bank (src/frontend.rs:84-96)."""
    filters = np.asarray(mel_filters, np.float32).reshape(N_MELS, N_FFT // 2 + 1)
    offsets, bins, values = [0], [], []
    for row in filters:
        nz = np.flatnonzero(row != 0)
        bins.extend(nz.tolist())
        values.extend(row[nz].tolist())
        offsets.append(len(bins))
    return np.asarray(offsets, np.int32), np.asarray(bins, np.int32), np.asarray(values, np.float32)


def frame_counts(samples: int):
    return (samples // HOP + 1, samples // HOP) if samples > 0 else (0, 0)


def framed(samples, window512):
    """fp32 [frames, 512]: pre-emphasised, centred, windowed (src/frontend.rs:133-151)."""
    x = np.asarray(samples, np.float32)
    frames, _ = frame_counts(x.size)
    xd = x.astype(np.float64)
    emph = xd.copy()
    emph[1:] -= np.float64(PREEMPHASIS) * xd[:-1]
    padded = np.zeros(x.size + N_FFT + frames * HOP, np.float64)
    padded[N_FFT // 2:N_FFT // 2 + x.size] = emph
    idx = np.arange(frames)[:, None] * HOP + np.arange(N_FFT)[None, :]
    return (padded[idx] * np.asarray(window512, np.float64)[None, :]).astype(np.float32)


def log_mel(frames_f32, offsets, bins, values, power_in_f32=False):
    """ln(filters . |DFT|^2 + guard) as fp32 [frames, 128] (src/frontend.rs:152-169)."""
    spec = np.fft.rfft(frames_f32.astype(np.float64), axis=1)
    re, im = spec.real.astype(np.float32).astype(np.float64), spec.imag.astype(np.float32).astype(np.float64)
    power = re * re + im * im
    out = np.empty((frames_f32.shape[0], N_MELS), np.float32)
    for mel in range(N_MELS):
        s, e = offsets[mel], offsets[mel + 1]
        acc = power[:, bins[s:e]] @ values[s:e].astype(np.float64) if e > s else np.zeros(power.shape[0])
        out[:, mel] = np.log(acc + np.float64(LOG_ZERO_GUARD)).astype(np.float32)
    return out


def normalize(features, valid_frames):
    """Per mel bin over the valid frames, rows beyond them zero (src/frontend.rs:172-204)."""
    f = np.asarray(features, np.float32)
    out = np.zeros_like(f)
    if valid_frames == 0:
        return out
    v = f[:valid_frames].astype(np.float64)
    mean = v.sum(axis=0) / valid_frames
    var = ((v - mean) ** 2).sum(axis=0) / (valid_frames - 1) if valid_frames > 1 else np.zeros(f.shape[1])
    out[:valid_frames] = ((v - mean) / (np.sqrt(var) + np.float64(NORMALIZE_EPSILON))).astype(np.float32)
    return out


def compute(samples, window, mel_filters):
    """Frame-major [frames, 128] normalised log-mel and the valid frame count."""
    x = np.asarray(samples, np.float32)
    if not np.all(np.isfinite(x)):
        raise ValueError("PCM samples must be finite")
    frames, valid = frame_counts(x.size)
    if frames == 0:
        return np.zeros((0, N_MELS), np.float32), 0
    offsets, bins, values = sparse_filters(mel_filters)
    return normalize(log_mel(framed(x, center_window(window)), offsets, bins, values), valid), valid


def hann_window():
    """Periodic Hann of 400 taps ("window": "hann", src/config.rs:171)."""
    n = np.arange(WIN, dtype=np.float64)
    return (0.5 - 0.5 * np.cos(2.0 * np.pi * n / WIN)).astype(np.float32)


def triangular_filters(seed=0):
    """A synthetic [128, 257] bank of overlapping triangles (the real one ships in the artifact
    as frontend.mel_filters): non-negative, a handful of non-zeros per row."""
    centers = np.linspace(2, 254, N_MELS)
    bins = np.arange(N_FFT // 2 + 1)[None, :]
    width = 2.0 + 6.0 * np.linspace(0, 1, N_MELS)[:, None]
    return np.maximum(0.0, 1.0 - np.abs(bins - centers[:, None]) / width).astype(np.float32) * 0.05
