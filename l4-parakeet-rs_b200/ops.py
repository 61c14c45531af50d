"""torch-tensor convenience wrappers around the C ABI.

torch supplies device memory and the current stream; every computation happens
inside libpk100.so.  Tensors must be CUDA and contiguous where stated.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import lib as L

EPS = 1e-5


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t, dtype=None):
    if not t.is_cuda:
        raise L.Pk100Error("libpk100 operates on CUDA tensors only (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"expected {dtype}, got {t.dtype}")
    return t


def gemm(a, b, *, kind, out, epilogue=L.EPI_LINEAR, row_scales=None, row_scale=1.0,
         col_scales=None, bias=None, act=L.ACT_NONE, residual=None, alpha=1.0, valid_rows=0,
         out_type=L.OUT_F16, out_scale=1.0, tau=0.0, keep_out=None, stats_out=None, keep_in=None,
         status=None, max_ctas=0, n=None, b_group_scales=None):
    """D = epilogue(A . B^T); see `pk100_gemm` in include/pk100.h."""
    _need(a), _need(b), _need(out)
    m, k = a.shape
    nn = b.shape[0] if n is None else n
    args = L.GemmArgs(
        kind=kind, epilogue=epilogue, m=m, n=nn, k=k,
        a=a.data_ptr(), lda=a.stride(0), b=b.data_ptr(), ldb=b.stride(0),
        row_scales=None if row_scales is None else row_scales.data_ptr(), row_scale=row_scale,
        col_scales=None if col_scales is None else col_scales.data_ptr(),
        bias=None if bias is None else bias.data_ptr(), act=act,
        residual=None if residual is None else residual.data_ptr(),
        ld_res=0 if residual is None else residual.stride(0), alpha=alpha, valid_rows=valid_rows,
        out=out.data_ptr(), ld_out=out.stride(0), out_type=out_type, out_scale=out_scale, tau=tau,
        keep_out=None if keep_out is None else keep_out.data_ptr(),
        stats_out=None if stats_out is None else stats_out.data_ptr(),
        keep_in=None if keep_in is None else keep_in.data_ptr(),
        status=None if status is None else status.data_ptr(), max_ctas=max_ctas,
        b_group_scales=None if b_group_scales is None else b_group_scales.data_ptr())
    L.check(L.lib.pk100_gemm(_stream(), C.byref(args)), "pk100_gemm")
    return out


def layer_norm(x, gamma, beta, mode=L.LN_F16, inv_scale=0.0, seg_stride=None, valid_rows=None,
               seg_valid=None, out=None, scales=None):
    _need(x, torch.float16)
    rows = x.shape[0]
    seg_stride = rows if seg_stride is None else seg_stride
    valid_rows = seg_stride if valid_rows is None else valid_rows
    if out is None:
        out = torch.empty((rows, 1024), device=x.device,
                          dtype=torch.float16 if mode == L.LN_F16 else
                          (torch.int8 if mode in (L.LN_S8_ROW, L.LN_S4_ROW) else torch.uint8))
    if scales is None and mode in (L.LN_E4M3_ROW, L.LN_S8_ROW, L.LN_S4_ROW):
        scales = torch.empty(rows, device=x.device, dtype=torch.float32)
    L.check(L.lib.pk100_layer_norm(_stream(), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(out),
                                   _ptr(scales), mode, inv_scale, rows, seg_stride, valid_rows,
                                   _ptr(seg_valid), EPS), "pk100_layer_norm")
    return out, scales


def layer_norm_pair(x, gamma, beta, next_gamma, next_beta, next_mode, next_inv_scale=0.0,
                    seg_stride=None, valid_rows=None, seg_valid=None, out=None, next_out=None,
                    next_scales=None):
    _need(x, torch.float16)
    rows = x.shape[0]
    seg_stride = rows if seg_stride is None else seg_stride
    valid_rows = seg_stride if valid_rows is None else valid_rows
    if out is None:
        out = torch.empty_like(x)
    if next_out is None:
        next_out = torch.empty((rows, 1024), device=x.device,
                               dtype=torch.float16 if next_mode == L.LN_F16 else
                               (torch.int8 if next_mode in (L.LN_S8_ROW, L.LN_S4_ROW) else torch.uint8))
    if next_scales is None and next_mode in (L.LN_E4M3_ROW, L.LN_S8_ROW, L.LN_S4_ROW):
        next_scales = torch.empty(rows, device=x.device, dtype=torch.float32)
    L.check(L.lib.pk100_layer_norm_pair(
        _stream(), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(out), _ptr(next_gamma), _ptr(next_beta),
        _ptr(next_out), _ptr(next_scales), next_mode, next_inv_scale, rows, seg_stride, valid_rows,
        _ptr(seg_valid), EPS), "pk100_layer_norm_pair")
    return out, next_out, next_scales


def quantize_fp8_fixed(x, inverse_scale):
    _need(x, torch.float16)
    out = torch.empty(x.shape, device=x.device, dtype=torch.uint8)
    L.check(L.lib.pk100_quantize_fp8_fixed(_stream(), _ptr(x), _ptr(out), x.numel(), inverse_scale),
            "pk100_quantize_fp8_fixed")
    return out


def quantize_int8(x, inverse_scale):
    _need(x, torch.float16)
    out = torch.empty(x.shape, device=x.device, dtype=torch.int8)
    L.check(L.lib.pk100_quantize_int8(_stream(), _ptr(x), _ptr(out), inverse_scale, x.numel()),
            "pk100_quantize_int8")
    return out


def pack_weight_rows(w, fmt):
    """fp16 [n, k] -> (packed, scales) ; S4_G128 returns fp16 group scales [k/128, n]."""
    _need(w, torch.float16)
    n, k = w.shape
    dev = w.device
    if fmt in (L.PACK_E4M3, L.PACK_S8):
        packed = torch.empty((n, k), device=dev, dtype=torch.uint8 if fmt == L.PACK_E4M3 else torch.int8)
    else:
        packed = torch.empty((n, k // 2), device=dev, dtype=torch.uint8)
    scales = torch.empty(n, device=dev, dtype=torch.float32) if fmt != L.PACK_S4_G128 else None
    gscales = torch.empty((k // 128, n), device=dev, dtype=torch.float16) if fmt == L.PACK_S4_G128 else None
    L.check(L.lib.pk100_pack_weight_rows(_stream(), _ptr(w), n, k, w.stride(0), fmt, _ptr(packed),
                                         _ptr(scales), _ptr(gscales)), "pk100_pack_weight_rows")
    return packed, (gscales if fmt == L.PACK_S4_G128 else scales)


def dequant_w4g128(codes, group_scales):
    n, k2 = codes.shape
    out = torch.empty((n, k2 * 2), device=codes.device, dtype=torch.float16)
    L.check(L.lib.pk100_dequant_w4g128(_stream(), _ptr(codes), _ptr(group_scales), n, k2 * 2,
                                       _ptr(out)), "pk100_dequant_w4g128")
    return out


def glu_masked(e, seg_stride=None, valid_rows=None, seg_valid=None):
    _need(e, torch.float16)
    rows = e.shape[0]
    seg_stride = rows if seg_stride is None else seg_stride
    valid_rows = seg_stride if valid_rows is None else valid_rows
    out = torch.empty((rows, 1024), device=e.device, dtype=torch.float16)
    L.check(L.lib.pk100_glu_masked(_stream(), _ptr(e), _ptr(out), rows, seg_stride, valid_rows,
                                   _ptr(seg_valid)), "pk100_glu_masked")
    return out


def unpack_s4(packed):
    """Packed INT4 codes [..., n/2] (low nibble = even index) -> INT8 codes [..., n]."""
    out = torch.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=torch.int8, device=packed.device)
    L.check(L.lib.pk100_unpack_s4(_stream(), _ptr(packed), _ptr(out), packed.numel()), "pk100_unpack_s4")
    return out


def prune_2of4_e4m3(dense):
    """E4M3 bytes [rows, cols] with the two smaller magnitudes of every quartet zeroed
    (the values the reference's 2:4-sparse FF2 multiplies, kernels/sm89/encoder.cu:685-713)."""
    rows, cols = dense.shape
    out = torch.empty_like(dense)
    L.check(L.lib.pk100_prune_2of4_e4m3(_stream(), _ptr(dense), _ptr(out), rows, cols), "pk100_prune_2of4_e4m3")
    return out


def compress_2of4_e4m3(dense):
    """The reference's compressed FF2 activation arena: data [rows, cols/2] + metadata [rows, cols/8], flat."""
    rows, cols = dense.shape
    out = torch.empty(rows * cols * 5 // 8, dtype=torch.uint8, device=dense.device)
    L.check(L.lib.pk100_compress_2of4_e4m3(_stream(), _ptr(dense), _ptr(out), rows, cols), "pk100_compress_2of4_e4m3")
    return out


def decompress_2of4_e4m3(flat, rows, cols):
    out = torch.empty((rows, cols), dtype=torch.uint8, device=flat.device)
    L.check(L.lib.pk100_decompress_2of4_e4m3(_stream(), _ptr(flat), _ptr(out), rows, cols),
            "pk100_decompress_2of4_e4m3")
    return out


def depthwise_bn_silu(g, wdw, bn_gamma, bn_beta, bn_mean, bn_var, quantize=False, seg_stride=None,
                      valid_rows=None, seg_valid=None):
    _need(g, torch.float16)
    rows = g.shape[0]
    seg_stride = rows if seg_stride is None else seg_stride
    valid_rows = seg_stride if valid_rows is None else valid_rows
    segments = rows // seg_stride
    out = torch.empty((rows, 1024), device=g.device, dtype=torch.uint8 if quantize else torch.float16)
    scales = torch.empty(rows, device=g.device, dtype=torch.float32) if quantize else None
    L.check(L.lib.pk100_depthwise_bn_silu(
        _stream(), _ptr(g), _ptr(wdw), _ptr(bn_gamma), _ptr(bn_beta), _ptr(bn_mean), _ptr(bn_var),
        _ptr(out), _ptr(scales), int(quantize), segments, seg_stride, valid_rows, _ptr(seg_valid),
        EPS), "pk100_depthwise_bn_silu")
    return out, scales


def local_attention(q, k, v, pos, bias_u, bias_v, seg_stride=None, valid_rows=None,
                    seg_valid=None, out=None):
    """Tensor-core local relative-position attention (the hot-path kernel)."""
    rows = q.shape[0]
    seg_stride = rows if seg_stride is None else seg_stride
    valid_rows = seg_stride if valid_rows is None else valid_rows
    if out is None:
        out = torch.empty((rows, 1024), device=q.device, dtype=torch.float16)
    L.check(L.lib.pk100_local_relpos_attention(
        _stream(), _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(pos),
        _ptr(bias_u), _ptr(bias_v), _ptr(out), out.stride(0), rows // seg_stride, seg_stride,
        valid_rows, _ptr(seg_valid)), "pk100_local_relpos_attention")
    return out


def local_attention_tcgen05(q, k, v, pos, bias_u, bias_v, seg_stride=None, valid_rows=None,
                            seg_valid=None, out=None, status=None):
    """The tcgen05 kernel (128 queries per CTA, accumulators in tensor memory); seg_stride % 128 == 0."""
    rows = q.shape[0]
    seg_stride = rows if seg_stride is None else seg_stride
    valid_rows = seg_stride if valid_rows is None else valid_rows
    if out is None:
        out = torch.empty((rows, 1024), device=q.device, dtype=torch.float16)
    L.check(L.lib.pk100_local_relpos_attention_tcgen05(
        _stream(), _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(pos),
        _ptr(bias_u), _ptr(bias_v), _ptr(out), out.stride(0), rows // seg_stride, seg_stride,
        valid_rows, _ptr(seg_valid), _ptr(status)), "pk100_local_relpos_attention_tcgen05")
    return out


def local_attention_simple(q, k, v, pos, bias_u, bias_v, seg_stride=None, valid_rows=None,
                           seg_valid=None, out=None):
    rows = q.shape[0]
    seg_stride = rows if seg_stride is None else seg_stride
    valid_rows = seg_stride if valid_rows is None else valid_rows
    if out is None:
        out = torch.empty((rows, 1024), device=q.device, dtype=torch.float16)
    L.check(L.lib.pk100_local_relpos_attention_simple(
        _stream(), _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(pos),
        _ptr(bias_u), _ptr(bias_v), _ptr(out), out.stride(0), rows // seg_stride, seg_stride,
        valid_rows, _ptr(seg_valid)), "pk100_local_relpos_attention_simple")
    return out


def pack_position_heads(p):
    out = torch.empty((8, 272, 128), device=p.device, dtype=torch.float16)
    L.check(L.lib.pk100_pack_position_heads(_stream(), _ptr(p), _ptr(out)), "pk100_pack_position_heads")
    return out
