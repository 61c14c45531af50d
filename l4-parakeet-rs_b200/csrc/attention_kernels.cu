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

// ---------------------------------------------------------------------------
// Tensor-core version.  One CTA = 4 warps = 64 consecutive queries of one head of
// one utterance (16 queries per warp).
//   phase 1  QP[q][j] = Q_q . P_h[j] + v_h . P_h[j] for the 272 position rows,
//            kept in shared memory as fp16 (the "relative shift" then is a plain
//            gather: key k of query q uses column j = 128 - q + k);
//   phase 2  flash-style loop over 32-key blocks of the 320-key union window:
//            S = Q . K^T (mma.sync m16n8k16, fp32 accumulate) + u_h . K_k + QP gather,
//            online softmax in fp32, O += P . V with P rounded to fp16.
// Operand tiles are staged with cp.async into padded (272-byte pitch) shared memory
// and read with ldmatrix; K/V (and the P_h blocks of phase 1) are double-buffered.
constexpr int kQTile = 64;
constexpr int kKeyBlock = 32;
constexpr int kPitch = kHeadWidth + 8;           // halves per shared-memory row
constexpr int kQpPitch = 280;                    // halves per QP row (272 used)
constexpr int kKeyBlocks = (kQTile + kLeft + kRight + kKeyBlock - 1) / kKeyBlock;   // 10
constexpr int kPosBlocks = (kPositionRowsPadded + kKeyBlock - 1) / kKeyBlock;         // 9

struct AttnSmem {
    // The Q tile is only read once, into register fragments, before the first QP value is
    // written: both live in the same bytes (71.6 KB per CTA -> 3 CTAs per SM instead of 2).
    union {
        __half q[kQTile][kPitch];
        __half qp[kQTile][kQpPitch];
    };
    __half kv[2][2][kKeyBlock][kPitch];          // [buffer][0 = K / P block, 1 = V]
    float uk[2][kKeyBlock];
    float bias_u[kHeadWidth];
    float bias_v[kHeadWidth];
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    const int bytes = valid ? 16 : 0;            // src-size 0 -> the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const unsigned*>(&h);
}

// Stage `rows` x 128 halves starting at row `first` of a [*, ld] matrix; rows outside
// [0, limit) are zero-filled.
__device__ __forceinline__ void stage_rows(__half (*dst)[kPitch], const __half* src, size_t ld,
                                           int first, int rows, int limit, int tid) {
    for (int c = tid; c < rows * 16; c += 128) {
        const int r = c / 16, part = c % 16;
        const int row = first + r;
        const bool ok = row >= 0 && row < limit;
        cp_async16(&dst[r][part * 8], src + static_cast<size_t>(ok ? row : 0) * ld + part * 8, ok);
    }
}

// Dot product of 32 consecutive fp32 bias values with 32 consecutive halves of a staged row
// (16-byte shared-memory loads).
__device__ __forceinline__ float dot32(const float* bias, const __half* row) {
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + i * 8);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
        const float4 b0 = *reinterpret_cast<const float4*>(bias + i * 8);
        const float4 b1 = *reinterpret_cast<const float4*>(bias + i * 8 + 4);
        const float2 x0 = __half22float2(h[0]), x1 = __half22float2(h[1]);
        const float2 x2 = __half22float2(h[2]), x3 = __half22float2(h[3]);
        acc = fmaf(b0.x, x0.x, acc); acc = fmaf(b0.y, x0.y, acc);
        acc = fmaf(b0.z, x1.x, acc); acc = fmaf(b0.w, x1.y, acc);
        acc = fmaf(b1.x, x2.x, acc); acc = fmaf(b1.y, x2.y, acc);
        acc = fmaf(b1.z, x3.x, acc); acc = fmaf(b1.w, x3.y, acc);
    }
    return acc;
}

__global__ void __launch_bounds__(128, 3) local_attention_mma_kernel(const AttnParams p) {
    extern __shared__ __align__(16) uint8_t attn_smem_raw[];
    AttnSmem& sm = *reinterpret_cast<AttnSmem*>(attn_smem_raw);
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int g = lane / 4, t = lane % 4;
    const int head = blockIdx.y, seg = blockIdx.z;
    const int q0 = blockIdx.x * kQTile;
    const int valid = p.seg_valid != nullptr ? p.seg_valid[seg] : p.valid_rows;
    const size_t base = static_cast<size_t>(seg) * p.seg_stride;
    const int rows_here = min(kQTile, p.seg_stride - q0);

    if (q0 >= valid) {                       // whole tile is padding: zero-fill and leave
        for (int c = tid; c < rows_here * 16; c += 128)
            *reinterpret_cast<uint4*>(p.out + (base + q0 + c / 16) * p.ldo + head * kHeadWidth + (c % 16) * 8) =
                make_uint4(0, 0, 0, 0);
        return;
    }

    const __half* qg = p.q + base * p.ldq + head * kHeadWidth;
    const __half* kg = p.k + base * p.ldk + head * kHeadWidth;
    const __half* vg = p.v + base * p.ldv + head * kHeadWidth;
    const __half* pg = p.pos + static_cast<size_t>(head) * kPositionRowsPadded * kHeadWidth;

    // ---- stage Q, the biases and the first position block
    stage_rows(sm.q, qg, p.ldq, q0, kQTile, valid, tid);
    stage_rows(sm.kv[0][0], pg, kHeadWidth, 0, kKeyBlock, kPositionRowsPadded, tid);
    cp_async_commit();
    for (int d = tid; d < kHeadWidth; d += 128) {
        sm.bias_u[d] = __half2float(p.bias_u[head * kHeadWidth + d]);
        sm.bias_v[d] = __half2float(p.bias_v[head * kHeadWidth + d]);
    }
    cp_async_wait<0>();
    __syncthreads();

    // Q fragments of this warp's 16 queries stay in registers for both phases
    unsigned qf[8][4];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
        ldmatrix_x4(qf[ks], &sm.q[warp * 16 + lane % 16][ks * 16 + (lane / 16) * 8]);

    // ---- phase 1: QP = Q . P^T + v . P
    for (int blk = 0; blk < kPosBlocks; ++blk) {
        const int buf = blk & 1;
        if (blk + 1 < kPosBlocks) {
            stage_rows(sm.kv[buf ^ 1][0], pg, kHeadWidth, (blk + 1) * kKeyBlock, kKeyBlock,
                       kPositionRowsPadded, tid);
            cp_async_commit();
        }
        // v . P_j for the 32 rows of this block: 4 threads per row
        {
            const int r = tid / 4, part = tid % 4;
            float acc = dot32(sm.bias_v + part * 32, &sm.kv[buf][0][r][part * 32]);
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (part == 0) sm.uk[buf][r] = acc;
        }
        float s[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
            for (int jp = 0; jp < 2; ++jp) {
                unsigned b[4];
                ldmatrix_x4(b, &sm.kv[buf][0][jp * 16 + (lane / 16) * 8 + lane % 8][ks * 16 + ((lane / 8) % 2) * 8]);
                mma_16816(s[2 * jp], qf[ks], b[0], b[1]);
                mma_16816(s[2 * jp + 1], qf[ks], b[2], b[3]);
            }
        }
        __syncthreads();                     // uk[buf] (v.P) is complete
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = blk * kKeyBlock + j * 8 + 2 * t;
            if (col < kPositionRowsPadded) {
                const float v0 = sm.uk[buf][j * 8 + 2 * t], v1 = sm.uk[buf][j * 8 + 2 * t + 1];
                *reinterpret_cast<unsigned*>(&sm.qp[warp * 16 + g][col]) = pack2(s[j][0] + v0, s[j][1] + v1);
                *reinterpret_cast<unsigned*>(&sm.qp[warp * 16 + g + 8][col]) = pack2(s[j][2] + v0, s[j][3] + v1);
            }
        }
        cp_async_wait<0>();
        __syncthreads();                     // next block landed; this block's readers are done
    }

    // ---- phase 2: keys [q0-128, q0+63+128] in blocks of 32
    const int key_first = q0 - kLeft;
    auto stage_kv = [&](int blk, int buf) {
        stage_rows(sm.kv[buf][0], kg, p.ldk, key_first + blk * kKeyBlock, kKeyBlock, valid, tid);
        stage_rows(sm.kv[buf][1], vg, p.ldv, key_first + blk * kKeyBlock, kKeyBlock, valid, tid);
        cp_async_commit();
    };
    // skip blocks that lie entirely outside [0, valid)
    int blk_begin = 0, blk_end = kKeyBlocks;
    while (blk_begin < blk_end && key_first + (blk_begin + 1) * kKeyBlock <= 0) ++blk_begin;
    while (blk_end > blk_begin && key_first + (blk_end - 1) * kKeyBlock >= valid) --blk_end;

    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY};
    float row_sum[2] = {0.0f, 0.0f};
    constexpr float kLog2e = 1.4426950408889634f;
    const float scale2 = kSoftmaxScale * kLog2e;
    const int qw = warp * 16;                // first query of this warp inside the tile

    stage_kv(blk_begin, blk_begin & 1);
    for (int blk = blk_begin; blk < blk_end; ++blk) {
        const int buf = blk & 1;
        cp_async_wait<0>();
        __syncthreads();                     // block `blk` landed; previous block's readers are done
        if (blk + 1 < blk_end) stage_kv(blk + 1, buf ^ 1);
        // u . K_k for this block's keys
        {
            const int r = tid / 4, part = tid % 4;
            float acc = dot32(sm.bias_u + part * 32, &sm.kv[buf][0][r][part * 32]);
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (part == 0) sm.uk[buf][r] = acc;
        }
        // band of this warp: j = 32*blk + c - q_local must intersect [0, 256]
        const bool warp_live = (kKeyBlock * blk + kKeyBlock - 1 - qw >= 0) &&
                               (kKeyBlock * blk - (qw + 15) <= kBand - 1);
        float s[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;
        if (warp_live) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
                for (int jp = 0; jp < 2; ++jp) {
                    unsigned b[4];
                    ldmatrix_x4(b, &sm.kv[buf][0][jp * 16 + (lane / 16) * 8 + lane % 8][ks * 16 + ((lane / 8) % 2) * 8]);
                    mma_16816(s[2 * jp], qf[ks], b[0], b[1]);
                    mma_16816(s[2 * jp + 1], qf[ks], b[2], b[3]);
                }
            }
        }
        __syncthreads();                     // uk[buf] complete
        if (warp_live) {
            float blk_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int c = j * 8 + 2 * t + (e & 1);
                    const int ql = qw + g + (e >> 1) * 8;
                    const int jj = kKeyBlock * blk + c - ql;
                    const int key = key_first + kKeyBlock * blk + c;
                    float v = -INFINITY;
                    if (jj >= 0 && jj < kBand && key >= 0 && key < valid && q0 + ql < valid)
                        v = (s[j][e] + sm.uk[buf][c] + __half2float(sm.qp[ql][jj])) * scale2;
                    s[j][e] = v;
                    blk_max[e >> 1] = fmaxf(blk_max[e >> 1], v);
                }
            }
            float alpha[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float m = blk_max[h];
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                const float m_new = fmaxf(row_max[h], m);
                alpha[h] = (m_new == -INFINITY) ? 1.0f : exp2f(row_max[h] - m_new);
                row_max[h] = m_new;
                row_sum[h] *= alpha[h];
            }
            unsigned pf[2][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float pv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float m = row_max[e >> 1];
                    pv[e] = (s[j][e] == -INFINITY) ? 0.0f : exp2f(s[j][e] - m);
                    row_sum[e >> 1] += pv[e];
                }
                pf[j / 2][(j % 2) * 2 + 0] = pack2(pv[0], pv[1]);
                pf[j / 2][(j % 2) * 2 + 1] = pack2(pv[2], pv[3]);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                o[j][0] *= alpha[0];
                o[j][1] *= alpha[0];
                o[j][2] *= alpha[1];
                o[j][3] *= alpha[1];
            }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
                for (int np = 0; np < 8; ++np) {
                    unsigned b[4];
                    ldmatrix_x4_trans(b, &sm.kv[buf][1][kk * 16 + ((lane / 8) % 2) * 8 + lane % 8][np * 16 + (lane / 16) * 8]);
                    mma_16816(o[2 * np], pf[kk], b[0], b[1]);
                    mma_16816(o[2 * np + 1], pf[kk], b[2], b[3]);
                }
            }
        }
    }

    // ---- normalise and store
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = row_sum[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        row_sum[h] = l > 0.0f ? 1.0f / l : 0.0f;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int ql = qw + g + h * 8;
        if (ql >= rows_here) continue;
        __half* dst = p.out + (base + q0 + ql) * p.ldo + head * kHeadWidth;
        const bool live = q0 + ql < valid;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float a = live ? o[j][2 * h] * row_sum[h] : 0.0f;
            const float b = live ? o[j][2 * h + 1] * row_sum[h] : 0.0f;
            *reinterpret_cast<unsigned*>(dst + j * 8 + 2 * t) = pack2(a, b);
        }
    }
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

extern "C" int pk100_local_relpos_attention(
    void* stream, const void* query, int ldq, const void* key, int ldk, const void* value, int ldv,
    const void* position, const void* bias_u, const void* bias_v, void* output, int ldo,
    int segments, int seg_stride, int valid_rows, const int* seg_valid) {
    const int rc = check_attn(query, key, value, position, bias_u, bias_v, output, ldq, ldk, ldv,
                              ldo, segments, seg_stride);
    if (rc != PK100_OK) return rc;
    if (segments == 0) return PK100_OK;
    static bool configured = false;
    if (!configured) {
        const cudaError_t err = cudaFuncSetAttribute(local_attention_mma_kernel,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     static_cast<int>(sizeof(AttnSmem)));
        if (err != cudaSuccess) return static_cast<int>(err);
        configured = true;
    }
    AttnParams p{static_cast<const __half*>(query), ldq, static_cast<const __half*>(key), ldk,
                 static_cast<const __half*>(value), ldv, static_cast<const __half*>(position),
                 static_cast<const __half*>(bias_u), static_cast<const __half*>(bias_v),
                 static_cast<__half*>(output), ldo, segments, seg_stride, valid_rows, seg_valid};
    dim3 grid((seg_stride + kQTile - 1) / kQTile, kHeads, segments);
    local_attention_mma_kernel<<<grid, 128, sizeof(AttnSmem), static_cast<cudaStream_t>(stream)>>>(p);
    return pk100_launch_status();
}

extern "C" int pk100_pack_position_heads(void* stream, const void* input, void* output) {
    if (!input || !output) return PK100_ERR_NULL;
    const int total = kPositionRowsPadded * kHeads * kHeadWidth;
    pack_position_heads_kernel<<<(total + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(input), static_cast<__half*>(output));
    return pk100_launch_status();
}
