"""Host-side mirror of the reference's subsampling stage driver
(src/cuda/subsampling.rs:436-804) for a batch of utterances."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import lib as L

vp = C.c_void_p


class SubsamplingWeightsC(C.Structure):
    _fields_ = [(n, vp) for n in ("conv0_w", "conv0_b", "dw1_w", "dw1_b", "pw1_w", "pw1_b", "dw2_w",
                                  "dw2_b", "pw2_w", "pw2_b", "proj_w", "proj_b")]


L.lib.pk100_subsampling_workspace_bytes.argtypes = [C.c_int, C.c_int, C.c_int]
L.lib.pk100_subsampling_workspace_bytes.restype = C.c_longlong
L.lib.pk100_run_subsampling.argtypes = [vp, C.POINTER(SubsamplingWeightsC), vp, C.c_int, C.c_int, vp, vp,
                                        vp, C.c_int, vp]
L.lib.pk100_run_subsampling.restype = C.c_int


class SubsamplingFp8C(C.Structure):
    """Mirror of `pk100_subsampling_fp8`."""
    _fields_ = [(n, vp) for n in ("pw1_q", "pw1_scales", "proj_q", "proj_scales")]


L.lib.pk100_subsampling_fp8_workspace_bytes.argtypes = [C.c_int, C.c_int, C.c_int]
L.lib.pk100_subsampling_fp8_workspace_bytes.restype = C.c_longlong
L.lib.pk100_run_subsampling_fp8.argtypes = [vp, C.POINTER(SubsamplingWeightsC), C.POINTER(SubsamplingFp8C), vp, C.c_int,
                                            C.c_int, vp, vp, vp, C.c_int, vp]
L.lib.pk100_run_subsampling_fp8.restype = C.c_int


def output_frames(mel_frames: int) -> int:
    f = mel_frames
    for _ in range(3):
        f = (f + 1) // 2
    return f


class Subsampling:
    def __init__(self, w, device, precision="fp16"):
        """precision "fp16": every pointwise layer and the projection as fp16 GEMMs (what the reference
        runs below 1024 output frames, and this build's default for every length); "fp8": the
        reference's variant from 1024 output frames on (first pointwise layer and projection as
        E4M3 GEMMs on per-row quantised activations, src/cuda/subsampling.rs:22)."""
        if precision not in ("fp16", "fp8"):
            raise ValueError("precision must be 'fp16' or 'fp8'")
        self.precision = precision
        self.device = torch.device(device)
        self.t = {}
        c = SubsamplingWeightsC()
        for name, _ in SubsamplingWeightsC._fields_:
            t = torch.from_numpy(np.ascontiguousarray(w[name], dtype=np.float32))
            if not (name.startswith("pw") and name.endswith("_b")) and name != "proj_b":
                t = t.to(torch.float16)
            self.t[name] = t.to(self.device)
            setattr(c, name, self.t[name].data_ptr())
        self.c = c
        self.q = None
        if precision == "fp8":
            from . import ops
            q = SubsamplingFp8C()
            for name in ("pw1", "proj"):
                codes, scales = ops.pack_weight_rows(self.t[f"{name}_w"], L.PACK_E4M3)
                self.t[f"{name}_q"], self.t[f"{name}_scales"] = codes, scales
                setattr(q, f"{name}_q", codes.data_ptr())
                setattr(q, f"{name}_scales", scales.data_ptr())
            self.q = q
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._ws = None

    def workspace(self, utterances, frames, seg_stride):
        size = L.lib.pk100_subsampling_workspace_bytes if self.q is None else L.lib.pk100_subsampling_fp8_workspace_bytes
        need = size(utterances, frames, seg_stride)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self._ws

    def run(self, mel, seg_stride, mel_frames=None, out=None):
        """mel: fp32 CUDA [utterances, frames, 128] -> fp16 [utterances*seg_stride, 1024]."""
        utterances, frames, bins = mel.shape
        assert bins == 128 and mel.dtype == torch.float32 and mel.is_contiguous()
        ws = self.workspace(utterances, frames, seg_stride)
        if out is None:
            out = torch.empty((utterances * seg_stride, 1024), dtype=torch.float16, device=self.device)
        args = (mel.data_ptr(), utterances, frames, None if mel_frames is None else mel_frames.data_ptr(),
                ws.data_ptr(), out.data_ptr(), seg_stride, self.status.data_ptr())
        stream = torch.cuda.current_stream().cuda_stream
        if self.q is None:
            L.check(L.lib.pk100_run_subsampling(stream, C.byref(self.c), *args), "pk100_run_subsampling")
        else:
            L.check(L.lib.pk100_run_subsampling_fp8(stream, C.byref(self.c), C.byref(self.q), *args),
                    "pk100_run_subsampling_fp8")
        return out
