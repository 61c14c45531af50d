"""Launches the reference's own kernels (oracle/_ref/*.cubin) on the GPU.

TEST INFRASTRUCTURE.  Restates the launch geometry of the reference's Rust host
(src/cuda/encoder.rs launch_* helpers, src/cuda/decoder.rs:274-353) through the
CUDA driver API (cuda-python), the same way cudarc does there: cuModuleLoadData
+ cuModuleGetFunction("pk_sm89_*") + cuLaunchKernel with positional arguments.
torch provides device memory only.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch
from cuda.bindings import driver as cu

REF_DIR = Path(__file__).resolve().parent / "_ref"


def available() -> bool:
    return all((REF_DIR / f"{u}.cubin").exists() for u in ("linear", "encoder", "decoder"))


def _ok(res):
    err = res[0]
    if err != cu.CUresult.CUDA_SUCCESS:
        raise RuntimeError(f"CUDA driver error {err}")
    return res[1] if len(res) == 2 else res[1:]


class Module:
    def __init__(self, unit: str):
        torch.cuda.init()
        torch.zeros(1, device="cuda")                      # make the primary context current
        data = (REF_DIR / f"{unit}.cubin").read_bytes()
        self.module = _ok(cu.cuModuleLoadData(data))
        self.functions = {}

    def fn(self, name: str):
        if name not in self.functions:
            self.functions[name] = _ok(cu.cuModuleGetFunction(self.module, name.encode()))
        return self.functions[name]

    def launch(self, name, grid, block, smem, args, cooperative=False):
        """args: list of torch tensors (device pointer), None (null pointer), int or float."""
        vals, types = [], []
        for a in args:
            if a is None:
                vals.append(0); types.append(C.c_void_p)
            elif isinstance(a, torch.Tensor):
                vals.append(a.data_ptr()); types.append(C.c_void_p)
            elif isinstance(a, float):
                vals.append(a); types.append(C.c_float)
            else:
                vals.append(int(a)); types.append(C.c_int)
        f = self.fn(name)
        if smem > 48 * 1024:
            _ok(cu.cuFuncSetAttribute(
                f, cu.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, smem))
        stream = torch.cuda.current_stream().cuda_stream
        g = tuple(grid) + (1,) * (3 - len(grid))
        b = tuple(block) + (1,) * (3 - len(block))
        launch = cu.cuLaunchCooperativeKernel if cooperative else cu.cuLaunchKernel
        if cooperative:
            _ok(launch(f, g[0], g[1], g[2], b[0], b[1], b[2], smem, stream, (tuple(vals), tuple(types))))
        else:
            _ok(launch(f, g[0], g[1], g[2], b[0], b[1], b[2], smem, stream, (tuple(vals), tuple(types)), 0))


_modules = {}


def module(unit: str) -> Module:
    if unit not in _modules:
        _modules[unit] = Module(unit)
    return _modules[unit]


def _cdiv(a, b):
    return (a + b - 1) // b


# ---- encoder.cu -----------------------------------------------------------

def layer_norm(x, gamma, beta, rows, padded_rows, eps=1e-5):
    """launch_norm (src/cuda/encoder.rs:1361-1391): grid padded_rows x 256."""
    out = torch.empty_like(x)
    module("encoder").launch("pk_sm89_layer_norm", (padded_rows,), (256,), 0,
                             [x, gamma, beta, out, rows, padded_rows, float(eps)])
    return out


def quantize_fp8_fixed(x, inverse_scale):
    """launch_quantize_fp8 (src/cuda/encoder.rs:1267-1291)."""
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    n = x.numel()
    module("encoder").launch("pk_sm89_quantize_fp8_fixed", (_cdiv(n, 256),), (256,), 0,
                             [x, out, n, float(inverse_scale)])
    return out


def ffn_expand_fp8(xq, wq, w_scales, rows):
    """launch_ffn_expand_fp8 (src/cuda/encoder.rs:1322-1358): grid (32, ceil(rows/128)) x 256,
    32768 B dynamic shared memory, input_scale 8/448, dynamic_scale 0."""
    out = torch.zeros((rows, 4096), dtype=torch.float16, device=xq.device)
    module("encoder").launch("pk_sm89_ffn_expand_fp8_async", (32, _cdiv(rows, 128)), (256,), 32768,
                             [xq, wq, w_scales, w_scales, out, rows, 8.0 / 448.0, 0])
    return out


def layer_norm_quantize_int4_dynamic(x, gamma, beta, rows, padded_rows, eps=1e-5):
    """launch_norm_quantize_fp8 with pk_sm89_layer_norm_quantize_int4_dynamic (src/cuda/encoder.rs:1029-1039):
    packed INT4 codes [padded_rows, 512] and fp32 row scales."""
    out = torch.zeros((padded_rows, 512), dtype=torch.uint8, device=x.device)
    scales = torch.zeros(padded_rows, dtype=torch.float32, device=x.device)
    module("encoder").launch("pk_sm89_layer_norm_quantize_int4_dynamic", (padded_rows,), (256,), 0,
                             [x, gamma, beta, out, scales, rows, padded_rows, float(eps)])
    return out, scales


def ffn_expand_int4_sparse(xq_packed, x_scales, wq_packed, w_scales, rows):
    """launch_ffn_expand_fp8 with pk_sm89_ffn_expand_int4_sparse and dynamic row scales
    (src/cuda/encoder.rs:1040-1050, :1322-1358): INT4 x INT4 `mma m16n8k64 s4`, SiLU -> fp16 -> x 16 -> E4M3,
    2:4 compression.  Returns the arena as flat bytes: data [rows, 2048] then metadata [rows, 512]."""
    out = torch.zeros(rows * 2560, dtype=torch.uint8, device=xq_packed.device)
    module("encoder").launch("pk_sm89_ffn_expand_int4_sparse", (32, _cdiv(rows, 128)), (256,), 32768,
                             [xq_packed, wq_packed, w_scales, x_scales, out, rows, 8.0 / 448.0, 1])
    return out


def ffn_contract_fp8(hq, wq, w_scales, x16, rows, sparse=False):
    """launch_ffn_contract_fp8 (src/cuda/encoder.rs:1128-1202) without its weight re-quantisation:
    pk_sm89_ffn_contract_fp8 on dense E4M3 activations [rows, 4096], or (sparse) pk_sm89_ffn_contract_fp8_sparse
    on the 2:4-compressed arena (data [rows, 2048] + metadata [rows, 512], `mma.sp`); both add
    0.5 * acc / 16 * w_scale to the fp16 state [rows, 1024] in place.  Grid (8, ceil(rows/128)) x 256."""
    out = x16.clone()
    if sparse:
        module("encoder").launch("pk_sm89_ffn_contract_fp8_sparse", (8, _cdiv(rows, 128)), (256,),
                                 2 * (128 * 32 + 128 * 64 + 128 * 8), [hq, wq, w_scales, out, rows, 4096])
    else:
        module("encoder").launch("pk_sm89_ffn_contract_fp8", (8, _cdiv(rows, 128)), (256,),
                                 2 * (128 * 64 + 128 * 64), [hq, wq, w_scales, out, rows])
    return out


def layer_norm_pair(x, gamma, beta, next_gamma, next_beta, rows, padded_rows, inverse_scale=0.0, eps=1e-5):
    """launch_norm_pair (src/cuda/encoder.rs:1394-1433): grid padded_rows x 256.  Returns the fp16
    first output and the second output: fp16 when inverse_scale == 0, else E4M3 bytes."""
    out = torch.empty_like(x)
    if inverse_scale != 0.0:
        nxt = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    else:
        nxt = torch.empty_like(x)
    module("encoder").launch("pk_sm89_layer_norm_pair", (padded_rows,), (256,), 0,
                             [x, gamma, beta, out, next_gamma, next_beta, nxt, rows, padded_rows,
                              float(eps), float(inverse_scale)])
    return out, nxt


def layer_norm_quantize_fp8_dynamic(x, gamma, beta, rows, padded_rows, eps=1e-5):
    """launch_norm_quantize_fp8 (src/cuda/encoder.rs:1436-1468): E4M3 bytes + per-row scales."""
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scales = torch.zeros(padded_rows, dtype=torch.float32, device=x.device)
    module("encoder").launch("pk_sm89_layer_norm_quantize_fp8_dynamic", (padded_rows,), (256,), 0,
                             [x, gamma, beta, out, scales, rows, padded_rows, float(eps)])
    return out, scales


def glu_masked(e, rows, padded_rows, valid_rows):
    """launch_glu_arena (src/cuda/encoder.rs:1965-1997)."""
    out = torch.empty((padded_rows, 1024), dtype=torch.float16, device=e.device)
    module("encoder").launch("pk_sm89_glu_masked", (_cdiv(padded_rows * 1024, 256),), (256,), 0,
                             [e, out, rows, padded_rows, valid_rows])
    return out


def depthwise_bn_silu(g, wdw, bn_g, bn_b, bn_m, bn_v, rows, padded_rows, eps=1e-5):
    """launch_depthwise_arena (src/cuda/encoder.rs:1999-2036): grid ceil(padded/8)*4 x 256."""
    out = torch.empty((padded_rows, 1024), dtype=torch.float16, device=g.device)
    module("encoder").launch("pk_sm89_depthwise_batchnorm_silu", (_cdiv(padded_rows, 8) * 4,), (256,), 0,
                             [g, wdw, bn_g, bn_b, bn_m, bn_v, out, rows, padded_rows, float(eps)])
    return out


def local_attention_scalar(q, k, v, pos, u, bv, rows, padded_rows, valid_rows):
    """pk_sm89_local_relpos_attention (src/cuda/encoder.rs:1925-1961 geometry
    (padded_rows, 8) x 32)."""
    out = torch.empty((padded_rows, 1024), dtype=torch.float16, device=q.device)
    module("encoder").launch("pk_sm89_local_relpos_attention", (padded_rows, 8), (32,), 0,
                             [q, k, v, pos, u, bv, out, rows, padded_rows, valid_rows, 128, 128])
    return out


# ---- linear.cu ------------------------------------------------------------

def fp16_linear(x, w, bias, residual, m, n, k, output_scale=1.0, residual_scale=0.0, activation=0):
    """launch_linear_view (src/cuda.rs:698-768): grid (n/32, ceil(m/32)) x 64."""
    out = torch.zeros((m, n), dtype=torch.float16, device=x.device)
    module("linear").launch("pk_sm89_fp16_linear_epilogue", (n // 32, _cdiv(m, 32)), (64,), 0,
                            [x, w, bias, residual, out, m, n, k, float(output_scale),
                             float(residual_scale), activation])
    return out


def _scaled_linear(name, xq, wq, w_scales, bias, m, n, k, input_scale, activation):
    """pk_sm89_fp8_linear_epilogue / pk_sm89_int8_linear_epilogue (kernels/sm89/linear.cu:325-429) as the
    quantisation benchmarks launch them (src/cuda/quant_benchmark.rs): one warp per 16 x 8 output
    tile, grid (n/32, m/16) x 128; m % 16 == 0, n % 32 == 0, k % 32 == 0, bias required."""
    assert m % 16 == 0 and n % 32 == 0 and k % 32 == 0
    out = torch.zeros((m, n), dtype=torch.float16, device=xq.device)
    module("linear").launch(name, (n // 32, m // 16), (128,), 0,
                            [xq, wq, w_scales, bias, out, m, n, k, float(input_scale), activation])
    return out


def fp8_linear(xq, wq, w_scales, bias, m, n, k, input_scale, activation=0):
    return _scaled_linear("pk_sm89_fp8_linear_epilogue", xq, wq, w_scales, bias, m, n, k, input_scale, activation)


def int8_linear(xq, wq, w_scales, bias, m, n, k, input_scale, activation=0):
    return _scaled_linear("pk_sm89_int8_linear_epilogue", xq, wq, w_scales, bias, m, n, k, input_scale, activation)


def quantize_fp8(x, inverse_scale):
    """pk_sm89_quantize_fp8 (kernels/sm89/linear.cu:537-547)."""
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    n = x.numel()
    module("linear").launch("pk_sm89_quantize_fp8", (_cdiv(n, 256),), (256,), 0, [x, out, float(inverse_scale), n])
    return out


def quantize_int8(x, inverse_scale):
    """pk_sm89_quantize_int8 (kernels/sm89/linear.cu:549-560)."""
    out = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    n = x.numel()
    module("linear").launch("pk_sm89_quantize_int8", (_cdiv(n, 256),), (256,), 0, [x, out, float(inverse_scale), n])
    return out


# ---- subsampling.cu -------------------------------------------------------

def subsampling_available() -> bool:
    return (REF_DIR / "subsampling.cubin").exists()


def subsample_first(mel, weight, bias, frames):
    """launch_first (src/cuda/subsampling.rs) on the whole utterance as one tile: mel fp32
    [frames, 128] -> fp16 [ceil(frames/2) * 64, 256] (row = frame * 64 + feature), ReLU fused."""
    f_out, feat = _cdiv(frames, 2), 64
    out = torch.zeros((f_out * feat, 256), dtype=torch.float16, device=mel.device)
    module("subsampling").launch("pk_sm89_subsample_first", (_cdiv(feat, 8), f_out), (256,), 0,
                                 [mel, weight, bias, out, frames, 0, f_out, feat])
    return out


def subsample_depthwise(x, weight, bias, in_frames, in_features, pad_rows_to=16):
    """launch_depthwise: fp16 [in_frames * in_features, 256] -> [ceil/2 frames * ceil/2 features, 256];
    the row count is padded (zero rows) to a multiple of 16 for the pointwise linear that follows."""
    f_out, feat = _cdiv(in_frames, 2), _cdiv(in_features, 2)
    rows = _cdiv(f_out * feat, pad_rows_to) * pad_rows_to
    out = torch.zeros((rows, 256), dtype=torch.float16, device=x.device)
    module("subsampling").launch("pk_sm89_subsample_depthwise", (_cdiv(feat, 8), f_out), (256,), 0,
                                 [x, weight, bias, out, 0, in_frames, in_features, 0, f_out, feat])
    return out


def subsample_depthwise_fp8(x, weight, bias, in_frames, in_features, pad_rows_to=16):
    """launch of pk_sm89_subsample_depthwise_fp8 (src/cuda/subsampling.rs:583-608): the depthwise conv with
    its output rounded to fp16, then quantised per row (256 channels) to E4M3 with scale absmax / 448.
    Returns (bytes [rows, 256], fp32 scales [rows]); rows padded with zero bytes / zero scales."""
    f_out, feat = _cdiv(in_frames, 2), _cdiv(in_features, 2)
    rows = _cdiv(f_out * feat, pad_rows_to) * pad_rows_to
    out = torch.zeros((rows, 256), dtype=torch.uint8, device=x.device)
    scales = torch.zeros(rows, dtype=torch.float32, device=x.device)
    module("subsampling").launch("pk_sm89_subsample_depthwise_fp8", (_cdiv(feat, 8), f_out), (256,), 0,
                                 [x, weight, bias, out, 0, in_frames, in_features, 0, f_out, feat, scales])
    return out, scales


def quantize_rows_fp8(x16, width):
    """pk_sm89_quantize_rows256 / pk_sm89_quantize_ffn_contract (kernels/sm89/encoder.cu:1150-1180): one CTA per
    row of 256 or 4096 fp16 values -> E4M3 bytes and the fp32 scale absmax / 448 (0 -> 1)."""
    rows = x16.shape[0]
    out = torch.empty((rows, width), dtype=torch.uint8, device=x16.device)
    scales = torch.empty(rows, dtype=torch.float32, device=x16.device)
    name = {256: "pk_sm89_quantize_rows256", 4096: "pk_sm89_quantize_ffn_contract"}[width]
    module("encoder").launch(name, (rows,), (256,), 0, [x16, out, scales])
    return out, scales


def subsample_linear_fp8(xq, x_scales, wq, w_scales, bias, rows, projection=False):
    """pk_sm89_subsample_pointwise_fp8 (K = N = 256, + bias, ReLU) or pk_sm89_subsample_projection_fp8
    (K = 4096, N = 1024, + bias): E4M3 x E4M3 with per-row activation scales (kernels/sm89/encoder.cu:1105-1119;
    launches src/cuda/subsampling.rs:613-630, :757-775: grid (N/128, ceil(rows/128)) x 256, 32768 B)."""
    n = 1024 if projection else 256
    out = torch.zeros((rows, n), dtype=torch.float16, device=xq.device)
    name = "pk_sm89_subsample_projection_fp8" if projection else "pk_sm89_subsample_pointwise_fp8"
    module("encoder").launch(name, (n // 128, _cdiv(rows, 128)), (256,), 32768,
                             [xq, wq, w_scales, x_scales, bias, out, rows])
    return out


def subsample_flatten(x, frames, padded_frames, features, valid_frames):
    """launch_flatten: [frames * features, 256] -> [padded_frames, 256 * features], column =
    channel * features + feature; rows >= valid_frames are zero."""
    out = torch.empty((padded_frames, 256 * features), dtype=torch.float16, device=x.device)
    total = padded_frames * 256 * features
    module("subsampling").launch("pk_sm89_subsample_flatten", (_cdiv(total, 256),), (256,), 0,
                                 [x, out, frames, padded_frames, features, 0, valid_frames])
    return out


def subsampling(mel, w, frames):
    """run_subsampling (src/cuda/subsampling.rs:436-804) for a request that fits one tile, fp16 path:
    first conv, two (depthwise, pointwise + ReLU) stages, flatten, projection.  `w`: device
    tensors named as in pk100_subsampling_weights.  Returns (stages, output [ceil(frames/8), 1024])."""
    stages = {}
    f1, f2, f3 = _cdiv(frames, 2), _cdiv(_cdiv(frames, 2), 2), _cdiv(_cdiv(_cdiv(frames, 2), 2), 2)
    x = subsample_first(mel, w["conv0_w"], w["conv0_b"], frames)
    stages["conv0"] = x
    x = subsample_depthwise(x, w["dw1_w"], w["dw1_b"], f1, 64)
    stages["dw1"] = x
    x = fp16_linear(x, w["pw1_w"], w["pw1_b"], None, x.shape[0], 256, 256, 1.0, 0.0, 2)
    stages["pw1"] = x
    x = subsample_depthwise(x, w["dw2_w"], w["dw2_b"], f2, 32)
    stages["dw2"] = x
    x = fp16_linear(x, w["pw2_w"], w["pw2_b"], None, x.shape[0], 256, 256, 1.0, 0.0, 2)
    stages["pw2"] = x
    padded = _cdiv(f3, 16) * 16
    flat = subsample_flatten(x, f3, padded, 16, f3)
    stages["flat"] = flat
    out = fp16_linear(flat, w["proj_w"], w["proj_b"], None, padded, 1024, 4096)
    return stages, out[:f3]


def subsampling_fp8(mel, w, frames):
    """run_subsampling for a request of 1024 output frames or more, restated on one tile (the FP8 branches
    of src/cuda/subsampling.rs:551-630 and :718-775): the first depthwise stage quantised per row with an
    E4M3 pointwise layer, the second stage in fp16, the flattened rows quantised per row and projected in
    E4M3.  Weights are quantised per row by the reference's own kernels, as it does in every request."""
    stages = {}
    f1, f2, f3 = _cdiv(frames, 2), _cdiv(_cdiv(frames, 2), 2), _cdiv(_cdiv(_cdiv(frames, 2), 2), 2)
    x = subsample_first(mel, w["conv0_w"], w["conv0_b"], frames)
    xq, xs = subsample_depthwise_fp8(x, w["dw1_w"], w["dw1_b"], f1, 64, pad_rows_to=128)
    stages["dw1_q"], stages["dw1_s"] = xq, xs
    wq, ws = quantize_rows_fp8(w["pw1_w"], 256)
    x = subsample_linear_fp8(xq, xs, wq, ws, w["pw1_b"], xq.shape[0])
    stages["pw1"] = x
    x = subsample_depthwise(x, w["dw2_w"], w["dw2_b"], f2, 32)
    x = fp16_linear(x, w["pw2_w"], w["pw2_b"], None, x.shape[0], 256, 256, 1.0, 0.0, 2)
    stages["pw2"] = x
    padded = _cdiv(f3, 128) * 128
    flat = subsample_flatten(x, f3, padded, 16, f3)
    fq, fs = quantize_rows_fp8(flat, 4096)
    stages["flat_q"], stages["flat_s"] = fq, fs
    pq, ps = quantize_rows_fp8(w["proj_w"], 4096)
    out = subsample_linear_fp8(fq, fs, pq, ps, w["proj_b"], padded, projection=True)
    return stages, out[:f3]


# ---- decoder.cu -----------------------------------------------------------

def tdt_decode(enc_proj, w, frames, sms):
    """launch_decode (src/cuda/decoder.rs:274-353), short-request kernel: cooperative
    grid 3*SMs x 128 (the reference sizes it with L4_SMS = 58 -> 174 CTAs; any grid
    that is co-resident works).  `w` holds the decoder tensors."""
    dev = enc_proj.device
    workspace = torch.zeros(9360 + 16 + 2088, dtype=torch.float32, device=dev)
    control = torch.zeros(8, dtype=torch.int32, device=dev)
    tokens = torch.zeros(frames * 10 + 16, dtype=torch.int32, device=dev)
    count = torch.zeros(1, dtype=torch.int32, device=dev)
    grid = min(3 * 58, 3 * sms)
    module("decoder").launch(
        "pk_sm89_tdt_persistent_v2", (grid,), (128,), 0,
        [enc_proj, w["embedding"], w["w_ih0"], w["w_hh0"], w["b_ih0"], w["b_hh0"], w["w_ih1"],
         w["w_hh1"], w["b_ih1"], w["b_hh1"], w["w_pred"], w["b_pred"], w["w_joint"], w["b_joint"],
         None, workspace, control, tokens, count, frames], cooperative=True)
    torch.cuda.synchronize()
    n = int(count.item())
    return tokens[:n].cpu().numpy()


def tdt_decode_long(enc_proj, w, frames):
    """launch_decode (src/cuda/decoder.rs:274-353) for a request of 1024 frames or more: the
    fp16 input table (launch_input_table, :355-383) and the INT8-cache kernel on a
    cooperative grid of 160 CTAs x 128 threads (:317-321)."""
    dev = enc_proj.device
    table = fp16_linear(w["embedding"][:1024].contiguous(), w["w_ih0"], None, None, 1024, 2560, 640)
    workspace = torch.zeros(9360 + 16 + 2088, dtype=torch.float32, device=dev)
    control = torch.zeros(9, dtype=torch.int32, device=dev)
    tokens = torch.zeros(frames * 10 + 16, dtype=torch.int32, device=dev)
    count = torch.zeros(1, dtype=torch.int32, device=dev)
    module("decoder").launch(
        "pk_sm89_tdt_persistent_fp8_ih", (160,), (128,), 0,
        [enc_proj, w["embedding"], w["w_ih0"], w["w_hh0"], w["b_ih0"], w["b_hh0"], w["w_ih1"],
         w["w_hh1"], w["b_ih1"], w["b_hh1"], w["w_pred"], w["b_pred"], w["w_joint"], w["b_joint"],
         table, workspace, control, tokens, count, frames], cooperative=True)
    torch.cuda.synchronize()
    n = int(count.item())
    return tokens[:n].cpu().numpy()


# ---- frontend.cu -----------------------------------------------------------

def frontend_available() -> bool:
    return (REF_DIR / "frontend.cubin").exists()


def frame_window(samples, window512, frames, preemphasis=0.97):
    """pk_sm89_frame_window as run_frontend launches it (src/cuda/frontend.rs:262-279)."""
    out = torch.empty((frames, 512), dtype=torch.float32, device=samples.device)
    module("frontend").launch("pk_sm89_frame_window", (_cdiv(frames * 512, 256),), (256,), 0,
                              [samples, window512, out, samples.numel(), frames, 0, float(preemphasis)])
    return out


def mel_log_sparse(spectrum, offsets, bins, values, frames, log_zero_guard):
    """pk_sm89_mel_log_sparse (src/cuda/frontend.rs:283-300); spectrum: float2 [frames, 257]."""
    out = torch.empty((frames, 128), dtype=torch.float32, device=spectrum.device)
    module("frontend").launch("pk_sm89_mel_log_sparse", (frames,), (128,), 0,
                              [spectrum, offsets, bins, values, out, frames, 0, float(log_zero_guard)])
    return out


def normalize_mel(features, frames, valid_frames, epsilon):
    """pk_sm89_normalize_mel (src/cuda/frontend.rs:303-315), in place on a copy."""
    out = features.clone()
    module("frontend").launch("pk_sm89_normalize_mel", (128,), (256,), 0, [out, frames, valid_frames, float(epsilon)])
    return out
