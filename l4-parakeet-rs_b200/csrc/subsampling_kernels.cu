// 8x depthwise-striding convolution subsampling (mel [frames,128] -> [frames/8, 1024])
// for a batch of utterances.  The convolutions are channel-parallel kernels (thread =
// channel, coalesced over the 256 channels), the first two fused so that the largest
// intermediate never reaches HBM; the two pointwise layers and
// the 4096 -> 1024 projection are tcgen05 GEMMs (pk100_gemm).  Semantics follow
// kernels/sm89/subsampling.cu:11-226 and the host tiling of
// src/cuda/subsampling.rs:436-804 (without its 256-frame tiles: the whole batch is
// processed at once).
#include <cuda_fp16.h>
#include <stdint.h>

#include "pk100_internal.h"

namespace pk100 {

constexpr int kChannels = 256;
constexpr int kMelBins = 128;
constexpr int kGroup = 8;

__device__ __forceinline__ int frames_of(const int* per_utt, int utt, int uniform) {
    return per_utt != nullptr ? per_utt[utt] : uniform;
}

// First two stages in one kernel: conv 3x3 s2 (1 -> 256 channels) + bias + ReLU, rounded to fp16,
// feeding the depthwise conv 3x3 s2 + bias.  The intermediate [frames/2, 64, 256] tensor (98 KB per
// output frame, 786 MB for 8 x 60 s) stays in registers instead of making a round trip through HBM.
// One CTA per output frame f2: thread = channel; the 7 mel rows 4*f2-3 .. 4*f2+3 are staged in shared
// memory with one zero column on each side; each thread walks the 64 intermediate features of the 3
// intermediate rows 2*f2-1 .. 2*f2+1 and scatters them into its 32 outputs.  The accumulation order of
// both convolutions (bias, then taps row by row, out-of-range taps skipped) is the reference's
// (kernels/sm89/subsampling.cu:11-179), so fusing changes no bit of the result.
// in [utt][in_stride frames][128] fp32 -> out [utt][out_cap][32][256] fp16
__global__ void __launch_bounds__(256)
subsample_first_fused_kernel(const float* __restrict__ in, const __half* __restrict__ w0,
                             const __half* __restrict__ b0, const __half* __restrict__ w1,
                             const __half* __restrict__ b1, __half* __restrict__ out, int in_stride,
                             int in_frames_uniform, const int* __restrict__ in_frames_per_utt, int out_cap) {
    __shared__ __align__(8) float smel[7][kMelBins + 4];      // column t of the mel row sits at index t + 1
    const int ch = threadIdx.x;
    const int f2 = blockIdx.x, utt = blockIdx.y;
    const int in_frames = frames_of(in_frames_per_utt, utt, in_frames_uniform);
    const int f1_frames = (in_frames + 1) / 2;
    const int f2_frames = (f1_frames + 1) / 2;
    if (f2 >= f2_frames) return;
    const float* src = in + static_cast<size_t>(utt) * in_stride * kMelBins;
    for (int i = ch; i < 7 * (kMelBins + 4); i += 256) {
        const int row = i / (kMelBins + 4), p = i % (kMelBins + 4);
        const int f = 4 * f2 - 3 + row, t = p - 1;
        (&smel[0][0])[i] = (f >= 0 && f < in_frames && t >= 0 && t < kMelBins)
            ? src[static_cast<size_t>(f) * kMelBins + t] : 0.0f;
    }
    float wa[9], wb[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) {
        wa[i] = __half2float(w0[ch * 9 + i]);
        wb[i] = __half2float(w1[ch * 9 + i]);
    }
    const float bias0 = __half2float(b0[ch]), bias1 = __half2float(b1[ch]);
    float sums[32];
#pragma unroll
    for (int m = 0; m < 32; ++m) sums[m] = bias1;
    __syncthreads();
#pragma unroll
    for (int kf = 0; kf < 3; ++kf) {
        const int f1 = 2 * f2 + kf - 1;
        if (f1 < 0 || f1 >= f1_frames) continue;             // padding row of the depthwise conv
        // mel rows of this intermediate row: 2*f1 - 1 + a = smel row 2*kf + a; rows outside the
        // utterance are skipped like in the separate kernel
        bool row_ok[3];
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const int f = 2 * f1 + a - 1;
            row_ok[a] = f >= 0 && f < in_frames;
        }
        // sliding 3-wide windows of the three mel rows: (c0, c1, c2) = columns 2*m1 - 1 .. 2*m1 + 1
        float c0[3], c1[3];
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            c0[a] = smel[2 * kf + a][0];
            c1[a] = smel[2 * kf + a][1];
        }
#pragma unroll
        for (int m1 = 0; m1 < 64; ++m1) {
            float acc = bias0;
#pragma unroll
            for (int a = 0; a < 3; ++a) {
                const float2 nx = *reinterpret_cast<const float2*>(&smel[2 * kf + a][2 * m1 + 2]);
                if (row_ok[a]) {
                    if (m1 > 0) acc = fmaf(c0[a], wa[a * 3 + 0], acc);      // column -1 is padding
                    acc = fmaf(c1[a], wa[a * 3 + 1], acc);
                    acc = fmaf(nx.x, wa[a * 3 + 2], acc);                   // column 2*m1 + 1 <= 127
                }
                c0[a] = nx.x;
                c1[a] = nx.y;
            }
            const float v = __half2float(__float2half_rn(fmaxf(acc, 0.0f)));
            // intermediate feature m1 is tap kt of output m2 with m1 = 2*m2 + kt - 1
            if (m1 % 2 == 0) {
                sums[m1 / 2] = fmaf(v, wb[kf * 3 + 1], sums[m1 / 2]);
            } else {
                sums[(m1 - 1) / 2] = fmaf(v, wb[kf * 3 + 2], sums[(m1 - 1) / 2]);
                if ((m1 + 1) / 2 < 32) sums[(m1 + 1) / 2] = fmaf(v, wb[kf * 3 + 0], sums[(m1 + 1) / 2]);
            }
        }
    }
    __half* dst = out + (static_cast<size_t>(utt) * out_cap + f2) * 32 * kChannels + ch;
#pragma unroll
    for (int m = 0; m < 32; ++m) dst[m * kChannels] = __float2half_rn(sums[m]);
}

// depthwise conv 3x3, stride 2, pad 1, + bias (no activation).
// in [utt][in_cap][in_feats][256] -> out [utt][out_cap][in_feats/2][256]
__global__ void __launch_bounds__(256)
subsample_depthwise_kernel(const __half* __restrict__ in, const __half* __restrict__ w,
                           const __half* __restrict__ b, __half* __restrict__ out, int in_cap,
                           int in_feats, int out_cap, int mel_frames_uniform,
                           const int* __restrict__ mel_frames_per_utt, int in_level) {
    const int ch = threadIdx.x;
    const int out_feats = in_feats / 2;
    const int feat0 = blockIdx.x * kGroup;
    const int of = blockIdx.y;
    const int utt = blockIdx.z;
    int in_frames = frames_of(mel_frames_per_utt, utt, mel_frames_uniform);
    for (int l = 0; l < in_level; ++l) in_frames = (in_frames + 1) / 2;
    const int out_frames = (in_frames + 1) / 2;
    if (of >= out_frames || feat0 >= out_feats) return;
    float wk[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) wk[i] = __half2float(w[ch * 9 + i]);
    const float bias = __half2float(b[ch]);
    float sums[kGroup];
#pragma unroll
    for (int g = 0; g < kGroup; ++g) sums[g] = bias;
    const __half* src = in + static_cast<size_t>(utt) * in_cap * in_feats * kChannels + ch;
#pragma unroll
    for (int kf = 0; kf < 3; ++kf) {
        const int f = of * 2 + kf - 1;
        if (f < 0 || f >= in_frames) continue;
#pragma unroll
        for (int kt = 0; kt < 3; ++kt) {
#pragma unroll
            for (int g = 0; g < kGroup; ++g) {
                const int t = (feat0 + g) * 2 + kt - 1;
                if (feat0 + g < out_feats && t >= 0 && t < in_feats)
                    sums[g] = fmaf(__half2float(src[(static_cast<size_t>(f) * in_feats + t) * kChannels]),
                                   wk[kf * 3 + kt], sums[g]);
            }
        }
    }
    __half* dst = out + ((static_cast<size_t>(utt) * out_cap + of) * out_feats + feat0) * kChannels + ch;
#pragma unroll
    for (int g = 0; g < kGroup; ++g)
        if (feat0 + g < out_feats) dst[g * kChannels] = __float2half_rn(sums[g]);
}

// [utt][cap][16][256] -> rows [utt*seg_stride + frame][channel*16 + feature]; rows at or
// beyond the utterance's output length are zero (kernels/sm89/subsampling.cu:202-226).
__global__ void __launch_bounds__(256)
subsample_flatten_kernel(const __half* __restrict__ in, __half* __restrict__ out, int in_cap,
                         int seg_stride, int mel_frames_uniform,
                         const int* __restrict__ mel_frames_per_utt) {
    __shared__ __half tile[16][kChannels + 2];
    const int frame = blockIdx.x, utt = blockIdx.y, tid = threadIdx.x;
    int valid = frames_of(mel_frames_per_utt, utt, mel_frames_uniform);
    for (int l = 0; l < 3; ++l) valid = (valid + 1) / 2;
    __half* dst = out + (static_cast<size_t>(utt) * seg_stride + frame) * 4096;
    if (frame >= valid) {
        for (int i = tid; i < 4096 / 8; i += 256) reinterpret_cast<uint4*>(dst)[i] = make_uint4(0, 0, 0, 0);
        return;
    }
    const __half* src = in + (static_cast<size_t>(utt) * in_cap + frame) * 16 * kChannels;
#pragma unroll
    for (int f = 0; f < 16; ++f) tile[f][tid] = src[f * kChannels + tid];
    __syncthreads();
    for (int i = tid; i < 4096; i += 256) dst[i] = tile[i % 16][i / 16];
}

}  // namespace pk100

using namespace pk100;

namespace {
long long up256(long long v) { return (v + 255) / 256 * 256; }
struct Caps { int f1, f2, f3; };
Caps caps(int frames) {
    Caps c;
    c.f1 = (frames + 1) / 2;
    c.f2 = (c.f1 + 1) / 2;
    c.f3 = (c.f2 + 1) / 2;
    return c;
}
}  // namespace

extern "C" long long pk100_subsampling_workspace_bytes(int utterances, int frames, int seg_stride) {
    if (utterances <= 0 || frames <= 0 || seg_stride <= 0) return 0;
    const Caps c = caps(frames);
    const long long u = utterances;
    return 2 * up256(u * c.f2 * 32 * 256 * 2) +
           2 * up256(u * c.f3 * 16 * 256 * 2) + up256(u * seg_stride * 4096LL * 2) + 256;
}

extern "C" long long pk100_subsampling_fp8_workspace_bytes(int utterances, int frames, int seg_stride) {
    if (utterances <= 0 || frames <= 0 || seg_stride <= 0) return 0;
    const Caps c = caps(frames);
    const long long u = utterances;
    return pk100_subsampling_workspace_bytes(utterances, frames, seg_stride) +
           up256(u * c.f2 * 32 * 256) + up256(u * c.f2 * 32 * 4) + up256(u * seg_stride * 4096LL) + up256(u * seg_stride * 4);
}

static int run_subsampling(void* stream_v, const pk100_subsampling_weights* w, const pk100_subsampling_fp8* q,
                           const float* mel, int utterances, int frames, const int* mel_frames, void* workspace,
                           void* output, int seg_stride, int* status);

extern "C" int pk100_run_subsampling(void* stream_v, const pk100_subsampling_weights* w,
                                     const float* mel, int utterances, int frames,
                                     const int* mel_frames, void* workspace, void* output,
                                     int seg_stride, int* status) {
    return run_subsampling(stream_v, w, nullptr, mel, utterances, frames, mel_frames, workspace, output, seg_stride,
                           status);
}

extern "C" int pk100_run_subsampling_fp8(void* stream_v, const pk100_subsampling_weights* w,
                                         const pk100_subsampling_fp8* q, const float* mel, int utterances,
                                         int frames, const int* mel_frames, void* workspace, void* output,
                                         int seg_stride, int* status) {
    if (!q || !q->pw1_q || !q->pw1_scales || !q->proj_q || !q->proj_scales) return PK100_ERR_NULL;
    return run_subsampling(stream_v, w, q, mel, utterances, frames, mel_frames, workspace, output, seg_stride, status);
}

static int run_subsampling(void* stream_v, const pk100_subsampling_weights* w, const pk100_subsampling_fp8* q,
                           const float* mel, int utterances, int frames, const int* mel_frames, void* workspace,
                           void* output, int seg_stride, int* status) {
    if (!w || !mel || !workspace || !output) return PK100_ERR_NULL;
    if (!w->conv0_w || !w->conv0_b || !w->dw1_w || !w->dw1_b || !w->pw1_w || !w->pw1_b || !w->dw2_w ||
        !w->dw2_b || !w->pw2_w || !w->pw2_b || !w->proj_w || !w->proj_b)
        return PK100_ERR_NULL;
    if (utterances == 0) return PK100_OK;
    if (utterances < 0 || frames <= 0) return PK100_ERR_SHAPE;
    const Caps c = caps(frames);
    if (seg_stride < c.f3) return PK100_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return PK100_ERR_ALIGN;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const long long u = utterances;
    char* p = static_cast<char*>(workspace);
    auto take = [&p](long long bytes) { char* cur = p; p += up256(bytes); return cur; };
    __half* s2 = reinterpret_cast<__half*>(take(u * c.f2 * 32 * 256 * 2));
    __half* s3 = reinterpret_cast<__half*>(take(u * c.f2 * 32 * 256 * 2));
    __half* s4 = reinterpret_cast<__half*>(take(u * c.f3 * 16 * 256 * 2));
    __half* s5 = reinterpret_cast<__half*>(take(u * c.f3 * 16 * 256 * 2));
    __half* flat = reinterpret_cast<__half*>(take(u * seg_stride * 4096LL * 2));
    take(256);                                              // (slack counted by the fp16 size function)
    // E4M3 variant: quantised rows of the first depthwise output and of the flattened features
    uint8_t* q2 = q ? reinterpret_cast<uint8_t*>(take(u * c.f2 * 32 * 256)) : nullptr;
    float* q2_scales = q ? reinterpret_cast<float*>(take(u * c.f2 * 32 * 4)) : nullptr;
    uint8_t* qflat = q ? reinterpret_cast<uint8_t*>(take(u * seg_stride * 4096LL)) : nullptr;
    float* qflat_scales = q ? reinterpret_cast<float*>(take(u * seg_stride * 4)) : nullptr;

    subsample_first_fused_kernel<<<dim3(c.f2, utterances), 256, 0, stream>>>(
        mel, static_cast<const __half*>(w->conv0_w), static_cast<const __half*>(w->conv0_b),
        static_cast<const __half*>(w->dw1_w), static_cast<const __half*>(w->dw1_b), s2, frames, frames,
        mel_frames, c.f2);
    int rc = pk100_launch_status();
    if (rc != PK100_OK) return rc;

    pk100_gemm_args a{};
    a.kind = PK100_KIND_F16; a.epilogue = PK100_EPI_LINEAR;
    a.m = static_cast<int>(u * c.f2 * 32); a.n = 256; a.k = 256;
    a.a = s2; a.lda = 256; a.b = w->pw1_w; a.ldb = 256;
    a.row_scale = 1.0f; a.alpha = 1.0f; a.bias = w->pw1_b; a.act = PK100_ACT_RELU;
    a.out = s3; a.ld_out = 256; a.out_type = PK100_OUT_F16; a.out_scale = 1.0f; a.status = status;
    if (q != nullptr) {
        // per-row E4M3 of the fp16 depthwise output (absmax / 448), E4M3 x E4M3 pointwise layer
        if ((rc = pk100_pack_weight_rows(stream, s2, a.m, 256, 256, PK100_PACK_E4M3, q2, q2_scales, nullptr)) != PK100_OK)
            return rc;
        pk100_gemm_args f = a;
        f.kind = PK100_KIND_E4M3; f.a = q2; f.b = q->pw1_q; f.row_scales = q2_scales; f.col_scales = q->pw1_scales;
        if ((rc = pk100_gemm(stream, &f)) != PK100_OK) return rc;
    } else if ((rc = pk100_gemm(stream, &a)) != PK100_OK) {
        return rc;
    }

    subsample_depthwise_kernel<<<dim3(16 / kGroup, c.f3, utterances), 256, 0, stream>>>(
        s3, static_cast<const __half*>(w->dw2_w), static_cast<const __half*>(w->dw2_b), s4, c.f2, 32,
        c.f3, frames, mel_frames, 2);
    if ((rc = pk100_launch_status()) != PK100_OK) return rc;

    a.m = static_cast<int>(u * c.f3 * 16);
    a.a = s4; a.b = w->pw2_w; a.bias = w->pw2_b; a.out = s5;
    if ((rc = pk100_gemm(stream, &a)) != PK100_OK) return rc;

    subsample_flatten_kernel<<<dim3(seg_stride, utterances), 256, 0, stream>>>(
        s5, flat, c.f3, seg_stride, frames, mel_frames);
    if ((rc = pk100_launch_status()) != PK100_OK) return rc;

    a.m = static_cast<int>(u * seg_stride); a.n = 1024; a.k = 4096;
    a.a = flat; a.lda = 4096; a.b = w->proj_w; a.ldb = 4096; a.bias = w->proj_b; a.act = PK100_ACT_NONE;
    a.out = output; a.ld_out = 1024;
    if (q != nullptr) {
        if ((rc = pk100_pack_weight_rows(stream, flat, a.m, 4096, 4096, PK100_PACK_E4M3, qflat, qflat_scales,
                                         nullptr)) != PK100_OK)
            return rc;
        a.kind = PK100_KIND_E4M3; a.a = qflat; a.b = q->proj_q; a.row_scales = qflat_scales;
        a.col_scales = q->proj_scales;
    }
    return pk100_gemm(stream, &a);
}
