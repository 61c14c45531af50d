"""Host-side mirror of the reference's encoder stage driver
(src/cuda/encoder.rs: LayerWeights :530-601, QuantizedFfnWeights :361-422,
cache_position_projections :441-482, run_layers :484-528).

Owns the packed per-layer weights (torch CUDA tensors = device memory) and calls
the C-ABI sequencer `pk100_run_layers`.  All arithmetic runs in libpk100.so.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from . import lib as L
from . import ops

vp, f32 = C.c_void_p, C.c_float
POSITION_ROWS = 257
POSITION_ROWS_PADDED = 272
ATT_LEFT = 128


class FfWeights(C.Structure):
    _fields_ = [("ln_gamma", vp), ("ln_beta", vp), ("w1", vp), ("w1_scales", vp), ("w2", vp),
                ("w2_scales", vp), ("tau", f32)]


class LayerWeights(C.Structure):
    _fields_ = [("ff1", FfWeights), ("ln_att_gamma", vp), ("ln_att_beta", vp), ("wqkv", vp),
                ("wqkv_scales", vp), ("position", vp), ("bias_u", vp), ("bias_v", vp), ("wo_f16", vp),
                ("wo_codes", vp), ("wo_group_scales", vp),
                ("ln_conv_gamma", vp), ("ln_conv_beta", vp), ("wpw1", vp), ("wpw1_scales", vp),
                ("dw_weight", vp), ("bn_gamma", vp), ("bn_beta", vp), ("bn_mean", vp), ("bn_var", vp),
                ("wpw2", vp), ("wpw2_scales", vp), ("ff2", FfWeights), ("ln_out_gamma", vp),
                ("ln_out_beta", vp)]


class Workspace(C.Structure):
    _fields_ = [("q8", vp), ("row_scales", vp), ("hidden8", vp), ("keep", vp), ("qkv", vp),
                ("att", vp), ("glu", vp), ("dw8", vp), ("dw_scales", vp), ("status", vp),
                ("profile_events", C.POINTER(vp)), ("profile_events_len", C.c_int)]


L.lib.pk100_encoder_workspace_bytes.argtypes = [C.c_int]
L.lib.pk100_encoder_workspace_bytes.restype = C.c_longlong
L.lib.pk100_encoder_workspace_carve.argtypes = [vp, C.c_int, C.POINTER(Workspace)]
L.lib.pk100_encoder_workspace_carve.restype = C.c_int
L.lib.pk100_run_layers.argtypes = [vp, C.POINTER(LayerWeights), C.c_int, vp, vp, C.POINTER(Workspace),
                                   C.c_int, C.c_int, C.c_int, vp, vp, C.c_int, C.POINTER(vp)]
L.lib.pk100_run_layers.restype = C.c_int


def relative_position_encoding() -> np.ndarray:
    """Sinusoid table [272, 1024]: row j encodes relative position 128 - j (rows >= 257
    are zero positions), sin at even and cos at odd features, evaluated in float64 and
    rounded to fp16 (src/cuda/encoder.rs:2038-2054)."""
    factor = -(math.log(10000.0) / 1024)
    freq = np.exp(2.0 * np.arange(512, dtype=np.float64) * factor)
    out = np.zeros((POSITION_ROWS_PADDED, 1024), dtype=np.float32)
    for j in range(POSITION_ROWS_PADDED):
        pos = float(ATT_LEFT - j) if j < POSITION_ROWS else 0.0
        out[j, 0::2] = np.sin(pos * freq)
        out[j, 1::2] = np.cos(pos * freq)
    return out.astype(np.float16)


class EncoderLayers:
    """Packed weights of n layers on one GPU + the launch of `pk100_run_layers`."""

    def __init__(self, device, out_proj_resident="f16"):
        """`out_proj_resident`: how the INT4 group-128 attention output projection lives on the GPU.
        "f16" (default): the codes are expanded once at load to the fp16 values the fused kernel
        would produce (2 MB per layer) and the projection runs as a plain fp16 tcgen05 GEMM;
        "int4": the codes stay packed (0.5 MB per layer) and the GEMM dequantises them in shared
        memory.  Both give the same bits; on a 180 GB part the expanded form is the faster one
        (21.7 vs 34.5 us at 6144 rows)."""
        if out_proj_resident not in ("f16", "int4"):
            raise ValueError("out_proj_resident must be 'f16' or 'int4'")
        self.out_proj_resident = out_proj_resident
        self.device = torch.device(device)
        self.tensors = []          # keeps device memory alive
        self.layers = []           # list[LayerWeights]
        self._sinus = torch.from_numpy(relative_position_encoding()).to(self.device)

    def _dev16(self, a):
        t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.float16).to(self.device)
        self.tensors.append(t)
        return t

    def _dev32(self, a):
        t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(self.device)
        self.tensors.append(t)
        return t

    def _keep(self, *ts):
        self.tensors.extend(ts)
        return ts

    def _ff(self, w, ff, tau):
        w1q, w1s = self._keep(*ops.pack_weight_rows(self._dev16(w[f"{ff}_w1"]), L.PACK_E4M3))
        w2q, w2s = self._keep(*ops.pack_weight_rows(self._dev16(w[f"{ff}_w2"]), L.PACK_S8))
        return FfWeights(self._dev16(w[f"ln_{ff}_g"]).data_ptr(), self._dev16(w[f"ln_{ff}_b"]).data_ptr(),
                         w1q.data_ptr(), w1s.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), float(tau))

    def add_layer(self, w, tau1=0.0, tau2=0.0):
        """Packs one layer's fp16 tensors on the GPU (load-time work; the reference does the
        FFN part on the CPU and the rest inside every request)."""
        lw = LayerWeights()
        lw.ff1 = self._ff(w, "ff1", tau1)
        lw.ff2 = self._ff(w, "ff2", tau2)
        wqkv = self._dev16(np.concatenate([w["wq"], w["wk"], w["wv"]], axis=0))
        q, s = self._keep(*ops.pack_weight_rows(wqkv, L.PACK_S8))
        lw.wqkv, lw.wqkv_scales = q.data_ptr(), s.data_ptr()
        codes, gs = self._keep(*ops.pack_weight_rows(self._dev16(w["wo"]), L.PACK_S4_G128))
        (wo16,) = self._keep(ops.dequant_w4g128(codes, gs))
        lw.wo_f16 = wo16.data_ptr()
        if self.out_proj_resident == "int4":
            lw.wo_codes, lw.wo_group_scales = codes.data_ptr(), gs.data_ptr()
        else:
            lw.wo_codes, lw.wo_group_scales = None, None
        # position table: sinusoid . Wpos^T (fp16 linear), head-major
        proj = torch.empty((POSITION_ROWS_PADDED, 1024), dtype=torch.float16, device=self.device)
        ops.gemm(self._sinus, self._dev16(w["wpos"]), kind=L.KIND_F16, out=proj)
        (pos,) = self._keep(ops.pack_position_heads(proj))
        lw.position = pos.data_ptr()
        lw.bias_u, lw.bias_v = self._dev16(w["bias_u"]).data_ptr(), self._dev16(w["bias_v"]).data_ptr()
        for name in ("att", "conv", "out"):
            setattr(lw, f"ln_{name}_gamma", self._dev16(w[f"ln_{name}_g"]).data_ptr())
            setattr(lw, f"ln_{name}_beta", self._dev16(w[f"ln_{name}_b"]).data_ptr())
        q, s = self._keep(*ops.pack_weight_rows(self._dev16(w["wpw1"]), L.PACK_E4M3))
        lw.wpw1, lw.wpw1_scales = q.data_ptr(), s.data_ptr()
        q, s = self._keep(*ops.pack_weight_rows(self._dev16(w["wpw2"]), L.PACK_E4M3))
        lw.wpw2, lw.wpw2_scales = q.data_ptr(), s.data_ptr()
        lw.dw_weight = self._dev16(w["dw"]).data_ptr()
        lw.bn_gamma, lw.bn_beta = self._dev32(w["bn_g"]).data_ptr(), self._dev32(w["bn_b"]).data_ptr()
        lw.bn_mean, lw.bn_var = self._dev32(w["bn_m"]).data_ptr(), self._dev32(w["bn_v"]).data_ptr()
        self.layers.append(lw)
        return lw

    def set_tau(self, layer, tau1=None, tau2=None):
        if tau1 is not None:
            self.layers[layer].ff1.tau = float(tau1)
        if tau2 is not None:
            self.layers[layer].ff2.tau = float(tau2)

    def make_workspace(self, rows):
        nbytes = L.lib.pk100_encoder_workspace_bytes(rows)
        arena = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        ws = Workspace()
        L.check(L.lib.pk100_encoder_workspace_carve(arena.data_ptr(), rows, C.byref(ws)), "workspace_carve")
        return arena, ws

    def run(self, state_a, state_b, ws, segments, seg_stride, valid_rows, seg_valid=None,
            tile_stats=None, attention_impl=0, first=0, count=None):
        """Runs layers [first, first+count) in place; returns the tensor holding the result."""
        count = len(self.layers) - first if count is None else count
        arr = (LayerWeights * count)(*self.layers[first:first + count])
        out = vp()
        rc = L.lib.pk100_run_layers(
            torch.cuda.current_stream().cuda_stream, arr, count, state_a.data_ptr(), state_b.data_ptr(),
            C.byref(ws), segments, seg_stride, valid_rows,
            None if seg_valid is None else seg_valid.data_ptr(),
            None if tile_stats is None else tile_stats.data_ptr(), attention_impl, C.byref(out))
        L.check(rc, "pk100_run_layers")
        return state_a if out.value == state_a.data_ptr() else state_b

    def status(self, ws_arena, ws):
        """Non-zero when a bounded wait expired inside a GEMM."""
        off = ws.status - ws_arena.data_ptr()
        return int(ws_arena[off:off + 4].view(torch.int32).item())


def tau_for_zero_fraction(stats: np.ndarray, zero_fraction: float = 0.7, window: float = 0.03) -> float:
    """Threshold that leaves about `zero_fraction` of the tiles below it.  Among the cuts
    within +-`window` of the target the one with the widest relative gap between
    neighbouring order statistics is used (tau = midpoint of that gap): a threshold that
    no tile sits close to, so the kept-tile bitmap is stable under rounding noise."""
    s = np.sort(np.asarray(stats, dtype=np.float32).ravel())
    lo = max(1, int(round((zero_fraction - window) * s.size)))
    hi = min(s.size - 1, int(round((zero_fraction + window) * s.size)))
    if hi < lo:
        return 0.0 if zero_fraction <= 0 else float("inf")
    cuts = np.arange(lo, hi + 1)
    a, b = s[cuts - 1].astype(np.float64), s[cuts].astype(np.float64)
    best = int(cuts[int(np.argmax((b - a) / np.maximum(b, 1e-30)))])
    return float((np.float64(s[best - 1]) + np.float64(s[best])) * 0.5)


def calibrate_tile_thresholds(enc: EncoderLayers, x0: torch.Tensor, ws, segments, seg_stride,
                              valid_rows, seg_valid=None, zero_fraction=0.7, attention_impl=0):
    """Sets every FF module's tau so that `zero_fraction` of its 128x64 hidden tiles fall
    below it on the calibration batch `x0` ([rows,1024] fp16).  Layer by layer: run the
    layer with tau = 0 recording tile statistics, fix ff1's tau, run again for ff2's.
    Returns the encoder output for x0 with the final thresholds."""
    rows = x0.shape[0]
    tiles = (rows + 127) // 128 * 64
    stats = torch.zeros((2, tiles), dtype=torch.float32, device=x0.device)
    # tiles that only contain padding rows never carry data: leave them out of the percentile
    live = np.ones((rows + 127) // 128, dtype=bool)
    if segments > 1 or valid_rows < seg_stride or seg_valid is not None:
        valid = (seg_valid.cpu().numpy() if seg_valid is not None else np.full(segments, valid_rows))
        rowmask = np.zeros(((rows + 127) // 128) * 128, dtype=bool)
        for s in range(segments):
            rowmask[s * seg_stride:s * seg_stride + int(valid[s])] = True
        live = rowmask.reshape(-1, 128).any(axis=1)
    cur = x0.clone()
    other = torch.empty_like(cur)
    for i in range(len(enc.layers)):
        saved = cur.clone()
        for which in (1, 2):
            cur.copy_(saved)
            enc.set_tau(i, **{f"tau{which}": 0.0})
            enc.run(cur, other, ws, segments, seg_stride, valid_rows, seg_valid, stats,
                    attention_impl, first=i, count=1)
            torch.cuda.synchronize()
            st = stats[which - 1].cpu().numpy().reshape(-1, 64)[live]
            enc.set_tau(i, **{f"tau{which}": tau_for_zero_fraction(st, zero_fraction)})
        cur.copy_(saved)
        out = enc.run(cur, other, ws, segments, seg_stride, valid_rows, seg_valid, None,
                      attention_impl, first=i, count=1)
        if out is other:
            cur, other = other, cur
    return cur
