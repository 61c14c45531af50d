"""Host-side mirror of the reference's decoder stage driver
(src/cuda/decoder.rs: DecoderWeights :227-271, launch_decode :274-353,
decode_tokens :210-225) for a batch of utterances."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import lib as L
from . import ops

vp = C.c_void_p
HIDDEN = 640
MAX_UTTERANCES = 8
LONG_REQUEST_FRAMES = 1024      # FP8_MIN_FRAMES, src/cuda/decoder.rs:15


class DecoderWeightsC(C.Structure):
    _fields_ = [("layers", C.c_int), ("embedding", vp), ("w_ih", vp * 2), ("w_hh", vp * 2),
                ("b_ih", vp * 2), ("b_hh", vp * 2), ("w_pred", vp), ("b_pred", vp),
                ("w_joint", vp), ("b_joint", vp)]


L.lib.pk100_tdt_workspace_bytes.argtypes = [C.c_int]
L.lib.pk100_tdt_workspace_bytes.restype = C.c_longlong
L.lib.pk100_tdt_rounds_offset.argtypes = [C.c_int]
L.lib.pk100_tdt_rounds_offset.restype = C.c_longlong
L.lib.pk100_tdt_cluster_capacity.argtypes = [C.c_int]
L.lib.pk100_tdt_cluster_capacity.restype = C.c_int
L.lib.pk100_tdt_decode.argtypes = [vp, C.POINTER(DecoderWeightsC), vp, C.c_int, C.c_int, vp, vp, vp, vp,
                                   vp, C.c_int, vp]
L.lib.pk100_tdt_decode.restype = C.c_int
for _name in ("pk100_tdt_decode_barrier", "pk100_tdt_decode_cluster", "pk100_tdt_decode_exchange",
              "pk100_tdt_decode_long", "pk100_tdt_decode_long_cluster", "pk100_tdt_decode_long_barrier",
              "pk100_tdt_decode_auto"):
    getattr(L.lib, _name).argtypes = L.lib.pk100_tdt_decode.argtypes
    getattr(L.lib, _name).restype = C.c_int


class TdtDecoder:
    """Decoder tensors on one GPU.  `w` maps names to numpy arrays: embedding [1025,640],
    w_ih{l} / w_hh{l} [2560,640], b_ih{l} / b_hh{l} [2560], w_pred [640,640], b_pred,
    w_joint [1030,640], b_joint, w_enc [640,1024], b_enc (fp16 values for matrices, fp32
    biases); w["layers"] = 1 or 2."""

    def __init__(self, w, device):
        self.device = torch.device(device)
        self.layers = int(w["layers"])
        self.t = {}
        for key, val in w.items():
            if key == "layers":
                continue
            t = torch.from_numpy(np.ascontiguousarray(val, dtype=np.float32))
            if not key.startswith("b_"):
                t = t.to(torch.float16)
            self.t[key] = t.to(self.device)
        c = DecoderWeightsC()
        c.layers = self.layers
        c.embedding = self.t["embedding"].data_ptr()
        for l in range(self.layers):
            c.w_ih[l] = self.t[f"w_ih{l}"].data_ptr()
            c.w_hh[l] = self.t[f"w_hh{l}"].data_ptr()
            c.b_ih[l] = self.t[f"b_ih{l}"].data_ptr()
            c.b_hh[l] = self.t[f"b_hh{l}"].data_ptr()
        c.w_pred, c.b_pred = self.t["w_pred"].data_ptr(), self.t["b_pred"].data_ptr()
        c.w_joint, c.b_joint = self.t["w_joint"].data_ptr(), self.t["b_joint"].data_ptr()
        self.c = c
        self.workspace = torch.zeros(L.lib.pk100_tdt_workspace_bytes(MAX_UTTERANCES), dtype=torch.uint8,
                                     device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def last_rounds(self, utterances, scratch=None):
        """Lockstep rounds of the last cluster / exchange decode of `utterances` sequences
        (synchronises: reads one int from the workspace)."""
        off = int(L.lib.pk100_tdt_rounds_offset(utterances))
        workspace = self.workspace if scratch is None else scratch[0]
        return int(workspace[off:off + 4].view(torch.int32).item())

    def project(self, encoded, out=None):
        """enc_proj = f16(encoded . W_enc^T + b_enc) (src/cuda/decoder.rs:298-313)."""
        rows = encoded.shape[0]
        if out is None:
            out = torch.empty((rows, HIDDEN), dtype=torch.float16, device=self.device)
        return ops.gemm(encoded, self.t["w_enc"], kind=L.KIND_F16, out=out, bias=self.t["b_enc"])

    def make_scratch(self):
        """A further (workspace, status) pair, for a decode that runs beside another one on a second
        stream: concurrent calls must not share either."""
        return (torch.zeros_like(self.workspace), torch.zeros(1, dtype=torch.int32, device=self.device))

    def decode(self, enc_proj, utterances, seg_stride, frames, max_tokens, tokens=None, durations=None,
               counts=None, barrier_kernel=False, kernel=None, lstm_cache="fp16", scratch=None):
        """frames: int32 CUDA tensor [utterances].  Returns (tokens, durations, counts) CUDA tensors.
        kernel: None (the library's choice), "cluster", "exchange" or "barrier".
        lstm_cache: "fp16" = the numerics of the reference's short-request kernel, "int8" = those of
        its kernel for requests of 1024 frames or more (cluster or barrier kernel), "auto" = the
        reference's rule per utterance (src/cuda/decoder.rs:88; two launches)."""
        if tokens is None:
            tokens = torch.zeros((utterances, max_tokens), dtype=torch.int32, device=self.device)
        if durations is None:
            durations = torch.zeros((utterances, max_tokens), dtype=torch.int32, device=self.device)
        if counts is None:
            counts = torch.zeros(utterances, dtype=torch.int32, device=self.device)
        if barrier_kernel:
            kernel = "barrier"
        if lstm_cache == "auto":
            if kernel is not None:
                raise ValueError("lstm_cache='auto' chooses its own kernels")
            name = "pk100_tdt_decode_auto"
        elif lstm_cache == "int8":
            if kernel not in (None, "cluster", "barrier"):
                raise ValueError("the long-request numerics exist in the cluster and barrier kernels")
            name = "pk100_tdt_decode_long" + ("_" + kernel if kernel else "")
        elif lstm_cache == "fp16":
            name = "pk100_tdt_decode" + ("_" + kernel if kernel else "")
        else:
            raise ValueError(f"lstm_cache: {lstm_cache!r}")
        fn = getattr(L.lib, name)
        workspace, status = (self.workspace, self.status) if scratch is None else scratch
        rc = fn(torch.cuda.current_stream().cuda_stream, C.byref(self.c),
                                    enc_proj.data_ptr(), utterances, seg_stride, frames.data_ptr(),
                                    workspace.data_ptr(), tokens.data_ptr(), durations.data_ptr(),
                                    counts.data_ptr(), max_tokens, status.data_ptr())
        L.check(rc, name)
        return tokens, durations, counts
