"""ctypes binding of libpk100.so (the C ABI declared in include/pk100.h).

The library is the product: there is no fallback.  Importing this module raises
if the shared object has not been built (`python l4-parakeet-rs_b200/build.py`).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libpk100.so"

if not LIB_PATH.exists():
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python {HERE / 'build.py'}` "
        "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")

lib = C.CDLL(str(LIB_PATH))

vp, i32, f32, i64 = C.c_void_p, C.c_int, C.c_float, C.c_longlong


class GemmArgs(C.Structure):
    """Mirror of `pk100_gemm_args` (include/pk100.h)."""
    _fields_ = [
        ("kind", i32), ("epilogue", i32), ("m", i32), ("n", i32), ("k", i32),
        ("a", vp), ("lda", i32), ("b", vp), ("ldb", i32),
        ("row_scales", vp), ("row_scale", f32), ("col_scales", vp), ("bias", vp),
        ("act", i32), ("residual", vp), ("ld_res", i32), ("alpha", f32), ("valid_rows", i32),
        ("out", vp), ("ld_out", i32), ("out_type", i32), ("out_scale", f32),
        ("tau", f32), ("keep_out", vp), ("stats_out", vp), ("keep_in", vp),
        ("status", vp), ("max_ctas", i32), ("b_group_scales", vp),
    ]


# name -> argument types (every function returns int)
SIGNATURES = {
    "pk100_gemm": [vp, C.POINTER(GemmArgs)],
    "pk100_layer_norm": [vp, vp, vp, vp, vp, vp, i32, f32, i32, i32, i32, vp, f32],
    "pk100_layer_norm_pair": [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, f32, i32, i32, i32, vp, f32],
    "pk100_quantize_fp8_fixed": [vp, vp, vp, i64, f32],
    "pk100_quantize_int8": [vp, vp, vp, f32, i64],
    "pk100_pack_weight_rows": [vp, vp, i32, i32, i32, i32, vp, vp, vp],
    "pk100_dequant_w4g128": [vp, vp, vp, i32, i32, vp],
    "pk100_glu_masked": [vp, vp, vp, i32, i32, i32, vp],
    "pk100_depthwise_bn_silu": [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, f32],
    "pk100_local_relpos_attention_simple": [vp, vp, i32, vp, i32, vp, i32, vp, vp, vp, vp, i32,
                                            i32, i32, i32, vp],
    "pk100_local_relpos_attention": [vp, vp, i32, vp, i32, vp, i32, vp, vp, vp, vp, i32,
                                     i32, i32, i32, vp],
    "pk100_local_relpos_attention_tcgen05": [vp, vp, i32, vp, i32, vp, i32, vp, vp, vp, vp, i32,
                                             i32, i32, i32, vp, vp],
    "pk100_pack_position_heads": [vp, vp, vp],
    "pk100_unpack_s4": [vp, vp, vp, i64],
    "pk100_prune_2of4_e4m3": [vp, vp, vp, i32, i32],
    "pk100_compress_2of4_e4m3": [vp, vp, vp, i32, i32],
    "pk100_decompress_2of4_e4m3": [vp, vp, vp, i32, i32],
    # struct-taking entry points: argtypes are completed in encoder.py / decoder.py
    "pk100_encoder_workspace_bytes": None,
    "pk100_encoder_workspace_carve": None,
    "pk100_run_layers": None,
    "pk100_tdt_workspace_bytes": None,
    "pk100_tdt_rounds_offset": None,
    "pk100_tdt_cluster_capacity": None,
    "pk100_tdt_decode": None,
    "pk100_tdt_decode_barrier": None,
    "pk100_tdt_decode_cluster": None,
    "pk100_tdt_decode_exchange": None,
    "pk100_tdt_decode_static": None,
    "pk100_tdt_decode_long": None,
    "pk100_tdt_decode_long_cluster": None,
    "pk100_tdt_decode_long_barrier": None,
    "pk100_tdt_decode_auto": None,
    "pk100_artifact_open": None,
    "pk100_artifact_close": None,
    "pk100_artifact_tensor_count": None,
    "pk100_artifact_tensor_at": None,
    "pk100_artifact_find": None,
    "pk100_artifact_vocabulary_size": None,
    "pk100_artifact_vocabulary_at": None,
    "pk100_artifact_field": None,
    "pk100_artifact_read_f32": None,
    "pk100_encode_fp16": None,
    "pk100_encode_fp16_linear": None,
    "pk100_encode_fp32_bias": None,
    "pk100_align_up": None,
    "pk100_estimate_linear": None,
    "pk100_exl3_layout": None,
    "pk100_mel_frames_for": None,
    "pk100_mel_frontend": None,
    "pk100_subsampling_workspace_bytes": None,
    "pk100_run_subsampling": None,
    "pk100_subsampling_fp8_workspace_bytes": None,
    "pk100_run_subsampling_fp8": None,
    "pk100_launch_count": None,
}

for _name, _argtypes in SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here = header / library mismatch
    if _argtypes is not None:
        _fn.argtypes = _argtypes
    _fn.restype = i32
lib.pk100_launch_count.restype = i64
lib.pk100_launch_count.argtypes = []
lib.pk100_set_gemm_cta_pairs.restype = None
lib.pk100_set_gemm_cta_pairs.argtypes = [i32]
lib.pk100_set_gemm_cta_cap.restype = None
lib.pk100_set_gemm_cta_cap.argtypes = [i32]
lib.pk100_set_dependent_launch.restype = None
lib.pk100_set_dependent_launch.argtypes = [i32]
lib.pk100_tensor_map_cache_stats.restype = None
lib.pk100_tensor_map_cache_stats.argtypes = [C.POINTER(i64), C.POINTER(i64)]


def tensor_map_cache_stats():
    hits, misses = i64(0), i64(0)
    lib.pk100_tensor_map_cache_stats(C.byref(hits), C.byref(misses))
    return int(hits.value), int(misses.value)

# enums (include/pk100.h)
OK, ERR_NULL, ERR_SHAPE, ERR_ALIGN, ERR_UNSUPPORTED, ERR_DRIVER, ERR_LIMIT = 0, -1, -2, -3, -4, -5, -6
KIND_F16, KIND_E4M3, KIND_S8, KIND_F16_W4G128 = 0, 1, 2, 3
OUT_F16, OUT_F32, OUT_E4M3, OUT_S8 = 0, 1, 2, 3
ACT_NONE, ACT_SILU, ACT_RELU = 0, 1, 2
EPI_LINEAR, EPI_GLU, EPI_SPARSE_OUT = 0, 1, 2
LN_F16, LN_E4M3_FIXED, LN_E4M3_ROW, LN_S8_ROW, LN_S4_ROW = 0, 1, 2, 3, 4
PACK_E4M3, PACK_S8, PACK_S4_ROW, PACK_S4_G128 = 0, 1, 2, 3


class Pk100Error(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        kind = "argument" if rc < 0 else "CUDA"
        raise Pk100Error(f"{what}: {kind} error {rc}")
