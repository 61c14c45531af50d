"""Host-side mirror of the reference's GPU frontend driver (src/cuda/frontend.rs:60-316):
window centring, sparse filter bank, device buffers, one call per batch of utterances."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import lib as L

vp = C.c_void_p
N_FFT, HOP, N_MELS = 512, 160, 128


class FrontendWeightsC(C.Structure):
    _fields_ = [("window", vp), ("filter_offsets", vp), ("filter_bins", vp), ("filter_values", vp),
                ("preemphasis", C.c_float), ("log_zero_guard", C.c_float), ("normalize_epsilon", C.c_float)]


L.lib.pk100_mel_frames_for.argtypes = [C.c_int]
L.lib.pk100_mel_frames_for.restype = C.c_int
L.lib.pk100_mel_frontend.argtypes = [vp, C.POINTER(FrontendWeightsC), vp, C.c_int, C.c_longlong, vp, vp, C.c_int, vp]
L.lib.pk100_mel_frontend.restype = C.c_int


def frames_for(samples: int) -> int:
    return L.lib.pk100_mel_frames_for(int(samples))


class MelFrontend:
    """window: the 400-tap analysis window, mel_filters: [128, 257] (the artifact's
    frontend.window / frontend.mel_filters, src/weights.rs:570-573)."""

    def __init__(self, window, mel_filters, device, preemphasis=0.97, log_zero_guard=2.0 ** -24,
                 normalize_epsilon=1e-5):
        self.device = torch.device(device)
        window = np.asarray(window, np.float32)
        if window.size > N_FFT:
            raise ValueError("window must fit the FFT")
        centred = np.zeros(N_FFT, np.float32)
        left = (N_FFT - window.size) // 2
        centred[left:left + window.size] = window                       # src/frontend.rs:218-223
        filters = np.asarray(mel_filters, np.float32).reshape(N_MELS, N_FFT // 2 + 1)
        if not (np.all(np.isfinite(centred)) and np.all(np.isfinite(filters))):
            raise ValueError("window and mel filters must be finite")
        offsets, bins, values = [0], [], []
        for row in filters:                                              # src/cuda/frontend.rs:196-228
            nz = np.flatnonzero(row != 0)
            bins.extend(nz.tolist())
            values.extend(row[nz].tolist())
            offsets.append(len(bins))
        t = lambda a, dt: torch.from_numpy(np.asarray(a, dt)).to(self.device)
        self.t = dict(window=t(centred, np.float32), offsets=t(offsets, np.int32),
                      bins=t(bins if bins else [0], np.int32), values=t(values if values else [0.0], np.float32))
        c = FrontendWeightsC()
        c.window, c.filter_offsets = self.t["window"].data_ptr(), self.t["offsets"].data_ptr()
        c.filter_bins, c.filter_values = self.t["bins"].data_ptr(), self.t["values"].data_ptr()
        c.preemphasis, c.log_zero_guard, c.normalize_epsilon = preemphasis, log_zero_guard, normalize_epsilon
        self.c = c

    def compute(self, samples, sample_counts, frame_cap=None, out=None, valid_frames=None):
        """samples: fp32 CUDA [utterances, stride]; sample_counts: int32 CUDA [utterances].
        Returns (mel fp32 [utterances, frame_cap, 128], valid_frames int32 [utterances])."""
        assert samples.dtype == torch.float32 and samples.is_contiguous() and samples.dim() == 2
        utterances, stride = samples.shape
        frame_cap = stride // HOP + 1 if frame_cap is None else frame_cap
        if out is None:
            out = torch.empty((utterances, frame_cap, N_MELS), dtype=torch.float32, device=self.device)
        if valid_frames is None:
            valid_frames = torch.zeros(utterances, dtype=torch.int32, device=self.device)
        rc = L.lib.pk100_mel_frontend(torch.cuda.current_stream().cuda_stream, C.byref(self.c), samples.data_ptr(),
                                      utterances, stride, sample_counts.data_ptr(), out.data_ptr(), frame_cap,
                                      valid_frames.data_ptr())
        L.check(rc, "pk100_mel_frontend")
        return out, valid_frames
