// Local relative-position multi-head attention (window +-128) for sm_100a.
//
//   score[q,k] = ((Q_q + u_h) . K_k + (Q_q + v_h) . P_h[128 - q + k]) / sqrt(128)
//   keys k in [max(0, q-128), min(valid-1, q+128)] of the query's own utterance,
//   fp32 softmax with max subtraction, ctx = sum_k p . V_k, fp16 output;
//   rows at or beyond the utterance's valid length are written as zero.
//
// `local_attention_simple_kernel` is the plain fp32 CUDA-core statement of the
// operator (one warp per query and head); `local_attention_mma_kernel` is the
// tensor-core version used on the hot path.
#include <cuda_fp16.h>
#include <float.h>
#include <stdint.h>

#include "pk100_internal.h"

namespace pk100 {

constexpr int kHeads = 8;
constexpr int kHeadWidth = 128;
constexpr int kLeft = 128;
constexpr int kRight = 128;
constexpr int kBand = kLeft + kRight + 1;          // 257
constexpr int kPositionRowsPadded = 272;
constexpr float kSoftmaxScale = 0.08838834764831845f;

struct AttnParams {
    const __half* q; int ldq;
    const __half* k; int ldk;
    const __half* v; int ldv;
    const __half* pos;        // [8, 272, 128] head-major
    const __half* bias_u;     // [8, 128]
    const __half* bias_v;     // [8, 128]
    __half* out; int ldo;
    int segments, seg_stride, valid_rows;
    const int* seg_valid;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off /= 2) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off /= 2) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

// grid: (ceil(seg_stride / 8), heads, segments); block: 8 warps = 8 queries.
__global__ void __launch_bounds__(256)
local_attention_simple_kernel(const AttnParams p) {
    __shared__ float s_qu[8][kHeadWidth];
    __shared__ float s_qv[8][kHeadWidth];
    __shared__ float s_score[8][kBand + 7];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int head = blockIdx.y, seg = blockIdx.z;
    const int q_local = blockIdx.x * 8 + warp;
    if (q_local >= p.seg_stride) return;
    const int valid = p.seg_valid != nullptr ? p.seg_valid[seg] : p.valid_rows;
    const size_t base = static_cast<size_t>(seg) * p.seg_stride;
    __half* out_row = p.out + (base + q_local) * p.ldo + head * kHeadWidth;
    if (q_local >= valid) {
        *reinterpret_cast<uint2*>(out_row + lane * 4) = make_uint2(0, 0);
        return;
    }
    const __half* q_row = p.q + (base + q_local) * p.ldq + head * kHeadWidth;
    for (int d = lane; d < kHeadWidth; d += 32) {
        const float qv = __half2float(q_row[d]);
        s_qu[warp][d] = qv + __half2float(p.bias_u[head * kHeadWidth + d]);
        s_qv[warp][d] = qv + __half2float(p.bias_v[head * kHeadWidth + d]);
    }
    __syncwarp();
    const int first_key = max(0, q_local - kLeft);
    const int last_key = min(valid - 1, q_local + kRight);
    const int count = last_key - first_key + 1;
    float mx = -FLT_MAX;
    for (int slot = lane; slot < count; slot += 32) {
        const int key = first_key + slot;
        const int pos_row = kLeft - q_local + key;
        const __half* k_row = p.k + (base + key) * p.ldk + head * kHeadWidth;
        const __half* p_row = p.pos + (static_cast<size_t>(head) * kPositionRowsPadded + pos_row) * kHeadWidth;
        float acc = 0.0f;
#pragma unroll 4
        for (int d = 0; d < kHeadWidth; d += 8) {
            const uint4 kr = *reinterpret_cast<const uint4*>(k_row + d);
            const uint4 pr = *reinterpret_cast<const uint4*>(p_row + d);
            const __half2* kh = reinterpret_cast<const __half2*>(&kr);
            const __half2* ph = reinterpret_cast<const __half2*>(&pr);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 kf = __half22float2(kh[i]);
                const float2 pf = __half22float2(ph[i]);
                acc = fmaf(s_qu[warp][d + 2 * i], kf.x, acc);
                acc = fmaf(s_qv[warp][d + 2 * i], pf.x, acc);
                acc = fmaf(s_qu[warp][d + 2 * i + 1], kf.y, acc);
                acc = fmaf(s_qv[warp][d + 2 * i + 1], pf.y, acc);
            }
        }
        acc *= kSoftmaxScale;
        s_score[warp][slot] = acc;
        mx = fmaxf(mx, acc);
    }
    mx = warp_max(mx);
    float denom = 0.0f;
    for (int slot = lane; slot < count; slot += 32) {
        const float e = __expf(s_score[warp][slot] - mx);
        s_score[warp][slot] = e;
        denom += e;
    }
    denom = warp_sum(denom);
    __syncwarp();
    const float inv = 1.0f / denom;
    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int slot = 0; slot < count; ++slot) {
        const float w = s_score[warp][slot] * inv;
        const uint2 raw = *reinterpret_cast<const uint2*>(
            p.v + (base + first_key + slot) * p.ldv + head * kHeadWidth + lane * 4);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
        const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
        c[0] = fmaf(w, a.x, c[0]);
        c[1] = fmaf(w, a.y, c[1]);
        c[2] = fmaf(w, b.x, c[2]);
        c[3] = fmaf(w, b.y, c[3]);
    }
    uint2 raw;
    __half2* h = reinterpret_cast<__half2*>(&raw);
    h[0] = __floats2half2_rn(c[0], c[1]);
    h[1] = __floats2half2_rn(c[2], c[3]);
    *reinterpret_cast<uint2*>(out_row + lane * 4) = raw;
}

// [272, 1024] -> head-major [8, 272, 128].
__global__ void pack_position_heads_kernel(const __half* __restrict__ in, __half* __restrict__ out) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= kPositionRowsPadded * kHeads * kHeadWidth) return;
    const int position = idx / (kHeads * kHeadWidth);
    const int feature = idx % (kHeads * kHeadWidth);
    const int head = feature / kHeadWidth, dim = feature % kHeadWidth;
    out[(static_cast<size_t>(head) * kPositionRowsPadded + position) * kHeadWidth + dim] = in[idx];
}

}  // namespace pk100

using namespace pk100;

static int check_attn(const void* q, const void* k, const void* v, const void* pos, const void* u,
                      const void* bv, const void* out, int ldq, int ldk, int ldv, int ldo,
                      int segments, int seg_stride) {
    if (!q || !k || !v || !pos || !u || !bv || !out) return PK100_ERR_NULL;
    if (segments < 0 || seg_stride <= 0) return PK100_ERR_SHAPE;
    if (ldq < 1024 || ldk < 1024 || ldv < 1024 || ldo < 1024) return PK100_ERR_SHAPE;
    if ((ldq | ldk | ldv | ldo) % 8 != 0) return PK100_ERR_SHAPE;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                           reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(pos) |
                           reinterpret_cast<uintptr_t>(out);
    if (bits & 15u) return PK100_ERR_ALIGN;
    return PK100_OK;
}

extern "C" int pk100_local_relpos_attention_simple(
    void* stream, const void* query, int ldq, const void* key, int ldk, const void* value, int ldv,
    const void* position, const void* bias_u, const void* bias_v, void* output, int ldo,
    int segments, int seg_stride, int valid_rows, const int* seg_valid) {
    const int rc = check_attn(query, key, value, position, bias_u, bias_v, output, ldq, ldk, ldv,
                              ldo, segments, seg_stride);
    if (rc != PK100_OK) return rc;
    if (segments == 0) return PK100_OK;
    AttnParams p{static_cast<const __half*>(query), ldq, static_cast<const __half*>(key), ldk,
                 static_cast<const __half*>(value), ldv, static_cast<const __half*>(position),
                 static_cast<const __half*>(bias_u), static_cast<const __half*>(bias_v),
                 static_cast<__half*>(output), ldo, segments, seg_stride, valid_rows, seg_valid};
    dim3 grid((seg_stride + 7) / 8, kHeads, segments);
    local_attention_simple_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return pk100_launch_status();
}

extern "C" int pk100_pack_position_heads(void* stream, const void* input, void* output) {
    if (!input || !output) return PK100_ERR_NULL;
    const int total = kPositionRowsPadded * kHeads * kHeadWidth;
    pack_position_heads_kernel<<<(total + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(input), static_cast<__half*>(output));
    return pk100_launch_status();
}
