// Host sequencer of the FastConformer block: issues the kernels of one layer in
// stream order, with no synchronisation and no allocation.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "pk100_internal.h"

namespace {

constexpr int kWidth = 1024;
constexpr int kFf = 4096;
constexpr float kFp8InputInv = 56.0f;             // activations are stored as E4M3(x * 56)
constexpr float kFp8InputScale = 8.0f / 448.0f;
constexpr float kHiddenInv = 32.0f;               // FF hidden activations as INT8(x * 32)
constexpr float kHiddenScale = 1.0f / 32.0f;
constexpr float kEps = 1e-5f;

long long align256(long long v) { return (v + 255) / 256 * 256; }

struct Geometry {
    int rows, segments, seg_stride, valid_rows;
    const int* seg_valid;
};

#define PK_TRY(expr)                 \
    do {                             \
        const int rc__ = (expr);     \
        if (rc__ != PK100_OK) return rc__; \
    } while (0)

int gemm_base(pk100_gemm_args& a, int kind, int m, int n, int k, const void* x, const void* w) {
    a = pk100_gemm_args{};
    a.kind = kind;
    a.epilogue = PK100_EPI_LINEAR;
    a.m = m; a.n = n; a.k = k;
    a.a = x; a.lda = k;
    a.b = w; a.ldb = k;
    a.row_scale = 1.0f;
    a.alpha = 1.0f;
    a.out_type = PK100_OUT_F16;
    a.out_scale = 1.0f;
    return PK100_OK;
}

// LN (already applied) -> FP8 expand + SiLU + tile threshold -> INT8 contract, x += 0.5*y
int ff_module(void* stream, const pk100_ff_weights& w, void* x, const pk100_encoder_workspace& ws,
              const Geometry& g, float* stats, int profile_slot) {
    pk100_gemm_args a;
    const bool timed = ws.profile_events != nullptr && 2 * profile_slot + 1 < ws.profile_events_len;
    if (timed) cudaEventRecord(static_cast<cudaEvent_t>(ws.profile_events[2 * profile_slot]),
                               static_cast<cudaStream_t>(stream));
    gemm_base(a, PK100_KIND_E4M3, g.rows, kFf, kWidth, ws.q8, w.w1);
    a.epilogue = PK100_EPI_SPARSE_OUT;
    a.row_scale = kFp8InputScale;
    a.col_scales = w.w1_scales;
    a.out = ws.hidden8; a.ld_out = kFf; a.out_type = PK100_OUT_S8; a.out_scale = kHiddenInv;
    a.tau = w.tau; a.keep_out = ws.keep; a.stats_out = stats; a.status = ws.status;
    PK_TRY(pk100_gemm(stream, &a));
    if (timed) cudaEventRecord(static_cast<cudaEvent_t>(ws.profile_events[2 * profile_slot + 1]),
                               static_cast<cudaStream_t>(stream));

    gemm_base(a, PK100_KIND_S8, g.rows, kWidth, kFf, ws.hidden8, w.w2);
    a.row_scale = kHiddenScale;
    a.col_scales = w.w2_scales;
    a.residual = x; a.ld_res = kWidth; a.alpha = 0.5f;
    a.out = x; a.ld_out = kWidth;
    a.keep_in = ws.keep; a.status = ws.status;
    return pk100_gemm(stream, &a);
}

}  // namespace

extern "C" long long pk100_encoder_workspace_bytes(int rows) {
    if (rows <= 0) return 0;
    const long long r = rows;
    const long long tiles = (r + 127) / 128;
    return align256(r * 1024) + align256(r * 4) + align256(r * 4096) + align256(tiles * 64) +
           align256(r * 3072 * 2) + align256(r * 1024 * 2) + align256(r * 1024 * 2) +
           align256(r * 1024) + align256(r * 4) + 256;
}

extern "C" int pk100_encoder_workspace_carve(void* base, int rows, pk100_encoder_workspace* out) {
    if (!base || !out) return PK100_ERR_NULL;
    if (rows <= 0) return PK100_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(base) & 255u) return PK100_ERR_ALIGN;
    const long long r = rows;
    const long long tiles = (r + 127) / 128;
    char* p = static_cast<char*>(base);
    auto take = [&p](long long bytes) { char* cur = p; p += align256(bytes); return cur; };
    out->q8 = take(r * 1024);
    out->row_scales = reinterpret_cast<float*>(take(r * 4));
    out->hidden8 = take(r * 4096);
    out->keep = reinterpret_cast<uint8_t*>(take(tiles * 64));
    out->qkv = take(r * 3072 * 2);
    out->att = take(r * 1024 * 2);
    out->glu = take(r * 1024 * 2);
    out->dw8 = take(r * 1024);
    out->dw_scales = reinterpret_cast<float*>(take(r * 4));
    out->status = reinterpret_cast<int*>(take(4));
    out->profile_events = nullptr;
    out->profile_events_len = 0;
    return PK100_OK;
}

extern "C" int pk100_run_layers(void* stream, const pk100_layer_weights* layers, int n_layers,
                                void* state_a, void* state_b, const pk100_encoder_workspace* wsp,
                                int segments, int seg_stride, int valid_rows, const int* seg_valid,
                                float* tile_stats, int attention_impl, void** output) {
    if (!layers || !state_a || !state_b || !wsp) return PK100_ERR_NULL;
    if (n_layers < 0 || segments < 0 || seg_stride <= 0) return PK100_ERR_SHAPE;
    const pk100_encoder_workspace& ws = *wsp;
    if (!ws.q8 || !ws.row_scales || !ws.hidden8 || !ws.keep || !ws.qkv || !ws.att || !ws.glu ||
        !ws.dw8 || !ws.dw_scales)
        return PK100_ERR_NULL;
    Geometry g{segments * seg_stride, segments, seg_stride, valid_rows, seg_valid};
    void* x = state_a;
    void* other = state_b;
    if (output) *output = x;
    if (g.rows == 0 || n_layers == 0) return PK100_OK;
    const long long stats_stride = static_cast<long long>((g.rows + 127) / 128) * 64;

    for (int i = 0; i < n_layers; ++i) {
        const pk100_layer_weights& w = layers[i];
        float* stats1 = tile_stats ? tile_stats + (2LL * i) * stats_stride : nullptr;
        float* stats2 = tile_stats ? tile_stats + (2LL * i + 1) * stats_stride : nullptr;
        pk100_gemm_args a;

        // ---- feed-forward module 1 (its LayerNorm was fused into the previous block's output norm)
        if (i == 0) {
            PK_TRY(pk100_layer_norm(stream, x, w.ff1.ln_gamma, w.ff1.ln_beta, ws.q8, nullptr,
                                    PK100_LN_E4M3_FIXED, kFp8InputInv, g.rows, seg_stride,
                                    valid_rows, seg_valid, kEps));
        }
        PK_TRY(ff_module(stream, w.ff1, x, ws, g, stats1, 2 * i));

        // ---- self-attention
        PK_TRY(pk100_layer_norm(stream, x, w.ln_att_gamma, w.ln_att_beta, ws.q8, ws.row_scales,
                                PK100_LN_S8_ROW, 0.0f, g.rows, seg_stride, valid_rows, seg_valid,
                                kEps));
        gemm_base(a, PK100_KIND_S8, g.rows, 3 * kWidth, kWidth, ws.q8, w.wqkv);
        a.row_scales = ws.row_scales;
        a.col_scales = w.wqkv_scales;
        a.out = ws.qkv; a.ld_out = 3 * kWidth; a.status = ws.status;
        PK_TRY(pk100_gemm(stream, &a));
        {
            const __half* qkv = static_cast<const __half*>(ws.qkv);
            if (attention_impl == 1) {
                PK_TRY(pk100_local_relpos_attention_simple(
                    stream, qkv, 3 * kWidth, qkv + kWidth, 3 * kWidth, qkv + 2 * kWidth, 3 * kWidth,
                    w.position, w.bias_u, w.bias_v, ws.att, kWidth, segments, seg_stride, valid_rows,
                    seg_valid));
            } else if (attention_impl == 0 && seg_stride % 128 == 0) {
                PK_TRY(pk100_local_relpos_attention_tcgen05(
                    stream, qkv, 3 * kWidth, qkv + kWidth, 3 * kWidth, qkv + 2 * kWidth, 3 * kWidth,
                    w.position, w.bias_u, w.bias_v, ws.att, kWidth, segments, seg_stride, valid_rows,
                    seg_valid, ws.status));
            } else {
                PK_TRY(pk100_local_relpos_attention(
                    stream, qkv, 3 * kWidth, qkv + kWidth, 3 * kWidth, qkv + 2 * kWidth, 3 * kWidth,
                    w.position, w.bias_u, w.bias_v, ws.att, kWidth, segments, seg_stride, valid_rows,
                    seg_valid));
            }
        }
        if (w.wo_codes != nullptr) {
            gemm_base(a, PK100_KIND_F16_W4G128, g.rows, kWidth, kWidth, ws.att, w.wo_codes);
            a.ldb = kWidth / 2;
            a.b_group_scales = w.wo_group_scales;
        } else {
            gemm_base(a, PK100_KIND_F16, g.rows, kWidth, kWidth, ws.att, w.wo_f16);
        }
        a.residual = x; a.ld_res = kWidth; a.out = x; a.ld_out = kWidth; a.status = ws.status;
        PK_TRY(pk100_gemm(stream, &a));

        // ---- convolution module
        PK_TRY(pk100_layer_norm(stream, x, w.ln_conv_gamma, w.ln_conv_beta, ws.q8, ws.row_scales,
                                PK100_LN_E4M3_ROW, 0.0f, g.rows, seg_stride, valid_rows, seg_valid,
                                kEps));
        gemm_base(a, PK100_KIND_E4M3, g.rows, 2 * kWidth, kWidth, ws.q8, w.wpw1);
        a.epilogue = PK100_EPI_GLU;
        a.row_scales = ws.row_scales;
        a.col_scales = w.wpw1_scales;
        a.out = ws.glu; a.ld_out = kWidth; a.status = ws.status;
        // the pad mask is per utterance: handled by the depthwise kernel's row bound, and the
        // LayerNorm above already zero-filled pad rows, so GLU(0, 0) = 0 there
        PK_TRY(pk100_gemm(stream, &a));
        PK_TRY(pk100_depthwise_bn_silu(stream, ws.glu, w.dw_weight, w.bn_gamma, w.bn_beta, w.bn_mean,
                                       w.bn_var, ws.dw8, ws.dw_scales, 1, segments, seg_stride,
                                       valid_rows, seg_valid, kEps));
        gemm_base(a, PK100_KIND_E4M3, g.rows, kWidth, kWidth, ws.dw8, w.wpw2);
        a.row_scales = ws.dw_scales;
        a.col_scales = w.wpw2_scales;
        a.residual = x; a.ld_res = kWidth; a.out = x; a.ld_out = kWidth; a.status = ws.status;
        PK_TRY(pk100_gemm(stream, &a));

        // ---- feed-forward module 2
        PK_TRY(pk100_layer_norm(stream, x, w.ff2.ln_gamma, w.ff2.ln_beta, ws.q8, nullptr,
                                PK100_LN_E4M3_FIXED, kFp8InputInv, g.rows, seg_stride, valid_rows,
                                seg_valid, kEps));
        PK_TRY(ff_module(stream, w.ff2, x, ws, g, stats2, 2 * i + 1));

        // ---- output norm, fused with the next block's first norm
        if (i + 1 < n_layers) {
            const pk100_layer_weights& nx = layers[i + 1];
            PK_TRY(pk100_layer_norm_pair(stream, x, w.ln_out_gamma, w.ln_out_beta, other,
                                         nx.ff1.ln_gamma, nx.ff1.ln_beta, ws.q8, nullptr,
                                         PK100_LN_E4M3_FIXED, kFp8InputInv, g.rows, seg_stride,
                                         valid_rows, seg_valid, kEps));
        } else {
            PK_TRY(pk100_layer_norm(stream, x, w.ln_out_gamma, w.ln_out_beta, other, nullptr,
                                    PK100_LN_F16, 0.0f, g.rows, seg_stride, valid_rows, seg_valid,
                                    kEps));
        }
        void* t = x; x = other; other = t;
        if (output) *output = x;
    }
    return PK100_OK;
}
