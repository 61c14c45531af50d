// Local relative-position multi-head attention (window +-128) on the 5th-generation tensor cores.
//
//   score[q,k] = ((Q_q + u_h) . K_k + (Q_q + v_h) . P_h[128 - q + k]) / sqrt(128)
//   keys k in [max(0, q-128), min(valid-1, q+128)] of the query's own utterance, fp32 softmax,
//   ctx = sum_k p . V_k  (definition: local_attention_simple_kernel; reference:
//   kernels/sm89/encoder.cu:1338-1461, tensor-core form :1500-2035).
//
// One CTA = 128 consecutive queries of one head of one utterance; their keys lie in a window of
// 384 rows.  The three contractions run as tcgen05.mma kind::f16 (M = 128) with fp32 accumulators in
// tensor memory:
//     QP = Q . P_h^T   (N = 128 + 128 + 16: the 257 position rows)   TMEM columns [0, 272)
//     S  = Q . K^T     (three key blocks of N = 128)                 [384, 512), [0, 128), [128, 256)
//     O  = Pr . V      (Pr = softmax probabilities, fp16, K = keys)  [256, 384)
// Operands arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) into three 32 KB slots
// that hold blocks of P_h, then K, then V in turn, each load issued as soon as its slot is free.  Q, P
// and K are K-major operands; V is used as it lies in memory (rows = keys = the K dimension of
// Pr . V, features contiguous), i.e. as an MN-major B operand: instruction-descriptor bit 16, and a
// shared-memory descriptor whose leading-dimension offset is the distance between the two 64-feature
// atoms and whose stride is the 1024 bytes between 8-key groups.  The u / v biases are added in fp32
// outside the MMAs (u . K_k and v . P_j are per-column constants).  QP is drained to shared memory as fp16 so that the relative shift is a plain
// gather (key kk of query ql reads column kk - ql).  The softmax is two passes over the S accumulators
// (row maximum, then exponentials) by sixteen warps, four per TMEM lane quadrant; the probabilities go
// back through swizzled shared memory as the A operand of the last contraction.
// Every wait is a bounded mbarrier wait; when one expires the kernel raises the status word and all
// roles leave through the common teardown (tensor memory freed).
#include <cuda.h>
#include <cuda_fp16.h>
#include <float.h>
#include <stdint.h>

#include <type_traits>

#include "pk100_internal.h"
#include "ptx_sm100.cuh"

namespace pk100 {

namespace att5 {

constexpr int kHeads = 8;
constexpr int kDim = 128;                 // head width
constexpr int kTile = 128;                // queries per CTA
constexpr int kReach = 128;               // keys on each side
constexpr int kWindow = kTile + 2 * kReach;          // 384 keys seen by a tile
constexpr int kPosRows = 272;             // position rows per head (257 used)
constexpr float kSoftmaxScale = 0.08838834764831845f;
constexpr int kParts = 4;                 // softmax warps per TMEM lane quadrant: 32 columns of a block each
constexpr int kSoftmaxWarps = 4 * kParts;
constexpr int kSoftmaxThreads = 32 * kSoftmaxWarps;
constexpr int kThreads = kSoftmaxThreads + 64;       // + TMA producer warp + MMA warp

constexpr int kAtomBytes = 128 * 128;     // [128 rows x 64 halves], 128-byte swizzle
constexpr int kSlotBytes = 2 * kAtomBytes;           // one 128-row operand block: features 0-63 | 64-127
constexpr int kTailBytes = 2 * 16 * 128;  // position rows 256..271
constexpr int kQpPitch = 274;             // halves per QP row: 137 words, odd, so that the 32 rows of a
                                          // warp fall into 32 different banks

// barrier indices
enum : int {
    B_IN = 0, B_QP_DONE, B_BIAS_DONE, B_QP_DRAINED,
    B_K_IN,                    // 3
    B_UK_DONE = B_K_IN + 3,    // 3
    B_S_DONE = B_UK_DONE + 3,  // 3
    B_V_IN = B_S_DONE + 3,     // 3
    B_P_READY = B_V_IN + 3,    // 3
    B_PV_DONE = B_P_READY + 3, // 3
    B_MAX = B_PV_DONE + 3,     // 4 (one per lane quadrant)
    B_SUM = B_MAX + 4,         // 4
    B_COUNT = B_SUM + 4
};

// Operand staging: three 32 KB slots take, in turn, the position rows (slots 0, 1 and the 4 KB tail),
// the key blocks (K0 -> slot 2 at once, K1 / K2 -> slots 0 / 1 when the position rows are done with)
// and the value blocks (V_b -> the slot K_b had, when S_b and its bias term are done).
struct Smem {
    alignas(1024) uint8_t q[kSlotBytes];              // Q tile, later the probability block
    alignas(1024) uint8_t slot[3][kSlotBytes];
    alignas(1024) uint8_t tail[kTailBytes];
    alignas(16) __half qp[kTile * kQpPitch + 8];
    float vp[288];
    float uk[kWindow];
    alignas(16) float bias_u[kDim];
    alignas(16) float bias_v[kDim];
    float rowmax[kParts][kTile];
    float rowsum[kParts][kTile];
    uint64_t bar[B_COUNT];
    uint32_t tmem_base;
    int abort;
};

struct Params {
    const __half* bias_u;     // [8, 128]
    const __half* bias_v;
    __half* out; int ldo;
    int segments, seg_stride, valid_rows;
    const int* seg_valid;
    int* status;
};

// byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a [rows x 64 halves] swizzled atom
__device__ __forceinline__ int swz(int row, int chunk) {
    return (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4);
}

// dot product of 32 fp32 bias values (in registers) with 32 consecutive halves (chunks first ..
// first + 3) of row `row` of a swizzled operand atom; two independent chains
__device__ __forceinline__ float bias_dot32(const uint8_t* atom, int row, int first, const float (&bias)[32]) {
    float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint4 raw = *reinterpret_cast<const uint4*>(atom + swz(row, first + c));
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 x = __half22float2(h[i]);
            acc0 = fmaf(bias[8 * c + 2 * i], x.x, acc0);
            acc1 = fmaf(bias[8 * c + 2 * i + 1], x.y, acc1);
        }
    }
    return acc0 + acc1;
}

// One copy of the polling loop for the whole kernel: the code of a CTA runs once, front to back,
// so its time is largely instruction fetch; every loop below is kept rolled for the same reason.
__device__ __noinline__ bool att_wait(uint64_t* bar, volatile int* abort_flag) {
    return mbar_wait_bounded(bar, 0u, abort_flag);
}
#define ATT_WAIT(index)                                                         \
    if (!att_wait(&sm.bar[index], abort_flag)) break

__global__ void __launch_bounds__(kThreads, 1)
local_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                               const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_p16,
                               const __grid_constant__ CUtensorMap map_v, const Params p) {
    extern __shared__ uint8_t att5_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(att5_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int head = blockIdx.y, seg = blockIdx.z;
    const int q0 = blockIdx.x * kTile;
    int valid = p.seg_valid != nullptr ? p.seg_valid[seg] : p.valid_rows;
    valid = min(valid, p.seg_stride);
    const int base = seg * p.seg_stride;
    const int rows_here = min(kTile, p.seg_stride - q0);

    // (the segment lengths, biases and position rows are constant over the kernel chain)
    grid_dependents_launch();
    if (q0 >= valid) {                       // the whole tile is padding: zero-fill and leave
        grid_dependency_wait();
        for (int c = tid; c < rows_here * 16; c += kThreads)
            *reinterpret_cast<uint4*>(p.out + static_cast<size_t>(base + q0 + c / 16) * p.ldo + head * kDim + (c % 16) * 8) =
                make_uint4(0, 0, 0, 0);
        return;
    }

    volatile int* abort_flag = &sm.abort;
    if (tid == 0) {
        sm.abort = 0;
        for (int i = 0; i < B_COUNT; ++i) {
            int count = 1;                                             // TMA arrive / tcgen05.commit
            if (i == B_BIAS_DONE || i == B_QP_DRAINED || (i >= B_UK_DONE && i < B_UK_DONE + 3) ||
                (i >= B_P_READY && i < B_P_READY + 3))
                count = kSoftmaxWarps;
            if (i >= B_MAX) count = kParts;
            mbar_init(&sm.bar[i], count);
        }
        fence_barrier_init();
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_p);
        prefetch_tensormap(&map_p16);
        prefetch_tensormap(&map_v);
    }
    if (tid < kDim) {
        sm.bias_u[tid] = __half2float(p.bias_u[head * kDim + tid]);
        sm.bias_v[tid] = __half2float(p.bias_v[head * kDim + tid]);
    }
    if (warp == kSoftmaxWarps + 1) {
        tmem_alloc(&sm.tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;
    grid_dependency_wait();                  // Q, K and V come from the kernel before
    const int key_first = q0 - kReach;       // window index kk <-> key key_first + kk
    // slot of key block b, and of value block b after it
    auto slot_of = [](int b) { return b == 0 ? 2 : b - 1; };
    // TMEM columns of the score block b and of the context
    auto score_col = [](int b) { return b == 0 ? 384u : (b == 1 ? 0u : 128u); };
    constexpr uint32_t kCtxCol = 256u;

    if (warp == kSoftmaxWarps) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            do {
                mbar_arrive_expect_tx(&sm.bar[B_IN], 3 * kSlotBytes + kTailBytes);
                for (int a = 0; a < 2; ++a) {
                    tma_load_2d(sm.q + a * kAtomBytes, &map_q, &sm.bar[B_IN], head * kDim + a * 64, base + q0);
                    for (int b = 0; b < 2; ++b)
                        tma_load_2d(sm.slot[b] + a * kAtomBytes, &map_p, &sm.bar[B_IN], a * 64, head * kPosRows + b * 128);
                    tma_load_2d(sm.tail + a * (kTailBytes / 2), &map_p16, &sm.bar[B_IN], a * 64, head * kPosRows + 256);
                }
                auto load_keys = [&](int b) {
                    mbar_arrive_expect_tx(&sm.bar[B_K_IN + b], kSlotBytes);
                    for (int a = 0; a < 2; ++a)
                        tma_load_2d(sm.slot[slot_of(b)] + a * kAtomBytes, &map_k, &sm.bar[B_K_IN + b],
                                    head * kDim + a * 64, base + key_first + b * 128);
                };
                load_keys(0);                       // slot 2 is free from the start
                // the other key blocks: once the position rows have been multiplied
                ATT_WAIT(B_QP_DONE);
                ATT_WAIT(B_BIAS_DONE);
                load_keys(1);
                load_keys(2);
                // values follow their key block into its slot
                bool ok = true;
                for (int b = 0; b < 3 && ok; ++b) {
                    ok = att_wait(&sm.bar[B_S_DONE + b], abort_flag) &&
                         att_wait(&sm.bar[B_UK_DONE + b], abort_flag);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&sm.bar[B_V_IN + b], kSlotBytes);
                    // rows = keys, 64 features per atom: the MN-major form of the B operand of Pr.V
                    for (int a = 0; a < 2; ++a)
                        tma_load_2d(sm.slot[slot_of(b)] + a * kAtomBytes, &map_v, &sm.bar[B_V_IN + b],
                                    head * kDim + a * 64, base + key_first + b * 128);
                }
            } while (false);
        }
    } else if (warp == kSoftmaxWarps + 1) {
        // ------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            do {
                constexpr uint32_t idesc128 = make_instr_desc<KIND_F16>(128, 128);
                constexpr uint32_t idesc16 = make_instr_desc<KIND_F16>(128, 16);
                const uint32_t q_addr = smem_u32(sm.q);
                ATT_WAIT(B_IN);
                tc_fence_after_sync();
                for (int ks = 0; ks < 8; ++ks) {           // 16 features per MMA
                    const int a = ks / 4, j = ks % 4;
                    const uint64_t da = make_smem_desc<128>(q_addr + a * kAtomBytes) + 2u * j;
                    for (int b = 0; b < 2; ++b)
                        tc_mma<KIND_F16>(tmem + 128u * b, da,
                                         make_smem_desc<128>(smem_u32(sm.slot[b]) + a * kAtomBytes) + 2u * j, idesc128, ks > 0);
                    tc_mma<KIND_F16>(tmem + 256u, da,
                                     make_smem_desc<128>(smem_u32(sm.tail) + a * (kTailBytes / 2)) + 2u * j, idesc16, ks > 0);
                }
                tc_commit(&sm.bar[B_QP_DONE]);
                bool ok = true;
                for (int b = 0; b < 3 && ok; ++b) {
                    if (b == 1) ok = att_wait(&sm.bar[B_QP_DRAINED], abort_flag);   // columns [0, 272) are free
                    if (ok) ok = att_wait(&sm.bar[B_K_IN + b], abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t k_addr = smem_u32(sm.slot[slot_of(b)]);
                    for (int ks = 0; ks < 8; ++ks) {
                        const int a = ks / 4, j = ks % 4;
                        tc_mma<KIND_F16>(tmem + score_col(b), make_smem_desc<128>(q_addr + a * kAtomBytes) + 2u * j,
                                         make_smem_desc<128>(k_addr + a * kAtomBytes) + 2u * j, idesc128, ks > 0);
                    }
                    tc_commit(&sm.bar[B_S_DONE + b]);
                }
                if (!ok) break;
                for (int b = 0; b < 3 && ok; ++b) {
                    ok = att_wait(&sm.bar[B_V_IN + b], abort_flag) &&
                         att_wait(&sm.bar[B_P_READY + b], abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t v_addr = smem_u32(sm.slot[slot_of(b)]);
                    for (int ks = 0; ks < 8; ++ks) {       // 16 keys per MMA
                        const int a = ks / 4, j = ks % 4;
                        // B = V[keys, features] as it lies in memory: MN-major (features contiguous),
                        // 8-key groups 1024 bytes apart, the second 64 features 16 KB on; 16 keys = 2048 bytes
                        constexpr uint32_t idesc_v = idesc128 | (1u << 16);
                        const uint64_t dv = static_cast<uint64_t>(((v_addr + ks * 2048u) & 0x3FFFFu) >> 4) |
                                            (static_cast<uint64_t>(kAtomBytes >> 4) << 16) | (64ull << 32) |
                                            (1ull << 46) | (2ull << 61);
                        tc_mma<KIND_F16>(tmem + kCtxCol, make_smem_desc<128>(q_addr + a * kAtomBytes) + 2u * j,
                                         dv, idesc_v, (b > 0 || ks > 0) ? 1u : 0u);
                    }
                    tc_commit(&sm.bar[B_PV_DONE + b]);
                }
            } while (false);
        }
    } else {
        // ------------------------------------------ bias terms, QP drain, softmax, output
        const int quad = warp % 4, part = warp / 4;
        const int ql = quad * 32 + lane;                       // query row inside the tile = TMEM lane
        const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quad * 32) << 16);
        constexpr float kLog2e = 1.4426950408889634f;
        const float scale2 = kSoftmaxScale * kLog2e;
        const bool q_live = q0 + ql < valid;
        do {
            // v . P_j for the 272 position rows (per-column constant of QP): four threads per row,
            // 32 features each, from the staged operand tiles
            ATT_WAIT(B_IN);
            const int qt = tid % 4;                                // this thread's features: 32 * qt ..
            float bias[32];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 t = *reinterpret_cast<const float4*>(&sm.bias_v[32 * qt + 4 * i]);
                bias[4 * i] = t.x; bias[4 * i + 1] = t.y; bias[4 * i + 2] = t.z; bias[4 * i + 3] = t.w;
            }
#pragma unroll 1
            for (int item = tid; item < 4 * kPosRows; item += kSoftmaxThreads) {
                const int row = item / 4;
                const uint8_t* atom = row < 256 ? sm.slot[row / 128] + (qt / 2) * kAtomBytes
                                                : sm.tail + (qt / 2) * (kTailBytes / 2);
                float acc = bias_dot32(atom, row < 256 ? row % 128 : row - 256, 4 * (qt % 2), bias);
                acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                acc += __shfl_xor_sync(0xffffffffu, acc, 2);
                if (qt == 0) sm.vp[row] = acc;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.bar[B_BIAS_DONE]);
            ATT_WAIT(B_BIAS_DONE);
            // QP: tensor memory -> fp16 rows in shared memory, bias term added.  Row ql is stored shifted
            // right by (ql & 1) halves, so that the run of position columns a key piece needs (kk0 - ql ...)
            // starts on a 32-bit word for every thread.  Part p drains columns [64p, 64p + 64), the last
            // part the 16 columns beyond as well.
            ATT_WAIT(B_QP_DONE);
            tc_fence_after_sync();
            {
                uint32_t* row = reinterpret_cast<uint32_t*>(&sm.qp[ql * kQpPitch]);
                const bool odd = (ql & 1) != 0;
                // 32 columns per step (part 3: a last step of 16 columns, the load still 32 wide: the columns
                // beyond 272 hold stale accumulators that are never stored)
                const int steps = part == kParts - 1 ? 3 : 2;
#pragma unroll 1
                for (int st = 0; st < steps; ++st) {
                    const int c0 = 64 * part + 32 * st;
                    const int words = st == 2 ? 8 : 16;
                    uint32_t r[32], w[16];
                    tmem_ld_32x32(lane_addr + static_cast<uint32_t>(c0), r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float4 t = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        if (4 * i < 2 * words) t = *reinterpret_cast<const float4*>(&sm.vp[c0 + 4 * i]);
                        const __half2 h0 = __floats2half2_rn(__uint_as_float(r[4 * i + 0]) + t.x, __uint_as_float(r[4 * i + 1]) + t.y);
                        const __half2 h1 = __floats2half2_rn(__uint_as_float(r[4 * i + 2]) + t.z, __uint_as_float(r[4 * i + 3]) + t.w);
                        w[2 * i + 0] = *reinterpret_cast<const uint32_t*>(&h0);
                        w[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&h1);
                    }
                    // an odd row's words hold (column 2m - 1, column 2m): shifted by one half, the two
                    // words shared with the neighbouring chunks are written as halves
                    uint32_t* dst = row + c0 / 2;
                    if (!odd) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (i < words) dst[i] = w[i];
                    } else {
                        reinterpret_cast<__half*>(dst)[1] = __ushort_as_half(static_cast<unsigned short>(w[0] & 0xFFFFu));
#pragma unroll
                        for (int i = 1; i < 16; ++i)
                            if (i < words) dst[i] = __byte_perm(w[i - 1], w[i], 0x5432);
                        const uint32_t last = words == 16 ? w[15] : w[7];
                        reinterpret_cast<__half*>(dst + words)[0] = __ushort_as_half(static_cast<unsigned short>(last >> 16));
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.bar[B_QP_DRAINED]);
            // u . K_kk for the keys of each block, as soon as the block has landed: four threads per key
            {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 t = *reinterpret_cast<const float4*>(&sm.bias_u[32 * qt + 4 * i]);
                    bias[4 * i] = t.x; bias[4 * i + 1] = t.y; bias[4 * i + 2] = t.z; bias[4 * i + 3] = t.w;
                }
                bool ok = true;
#pragma unroll 1
                for (int b = 0; b < 3 && ok; ++b) {
                    ok = att_wait(&sm.bar[B_K_IN + b], abort_flag);
                    if (!ok) break;
                    const int row = tid / 4;
                    float acc = bias_dot32(sm.slot[slot_of(b)] + (qt / 2) * kAtomBytes, row, 4 * (qt % 2), bias);
                    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
                    if (qt == 0) sm.uk[b * 128 + row] = acc;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm.bar[B_UK_DONE + b]);
                }
                for (int b = 0; b < 3 && ok; ++b) ok = att_wait(&sm.bar[B_UK_DONE + b], abort_flag);
                if (!ok) break;
            }
            ATT_WAIT(B_QP_DRAINED);
            {
                bool ok = true;
                for (int b = 0; b < 3 && ok; ++b) ok = att_wait(&sm.bar[B_S_DONE + b], abort_flag);
                if (!ok) break;
            }
            tc_fence_after_sync();

            // keys this query sees, in window coordinates: [lo, hi] (empty for a padding row)
            const int lo = max(ql, -key_first);
            const int hi = q_live ? min(ql + 2 * kReach, valid - 1 - key_first) : -1;
            // the same for the whole warp: pieces outside [w_lo, w_hi] are skipped
            const int w_lo = max(quad * 32, -key_first), w_hi = min(quad * 32 + 31 + 2 * kReach, valid - 1 - key_first);
            const unsigned span = static_cast<unsigned>(hi - lo);          // hi < lo: nothing passes
            // A piece = 16 consecutive columns of this thread's scores; this warp owns two pieces (32
            // columns) of every block.  Pass 0 finds the row maximum, pass 1 writes the probabilities,
            // block by block, into the A operand of the last contraction (one rolled loop for both).
            float mx = -INFINITY, sum = 0.0f;
            bool ok = true;
#pragma unroll 1
            for (int pass = 0; pass < 2 && ok; ++pass) {
#pragma unroll 1
                for (int b = 0; b < 3 && ok; ++b) {
                    uint32_t w[16];
                    const int kk0 = b * 128 + part * 32;
                    float s[32];
                    const bool live = !(kk0 + 31 < w_lo || kk0 > w_hi);
                    if (live) {
                        uint32_t r[32];
                        tmem_ld_32x32(lane_addr + score_col(b) + static_cast<uint32_t>(kk0 % 128), r);
                        // position scores of columns kk0 - ql .. + 31: stored from half (ql & 1) on, so the
                        // run starts at a word of the row (kk0 is even)
                        const __half2* qp2 = reinterpret_cast<const __half2*>(&sm.qp[ql * kQpPitch + kk0 - ql + (ql & 1)]);
                        const float4* uk4 = reinterpret_cast<const float4*>(&sm.uk[kk0]);
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const float4 u = uk4[c];
                            const float2 a = __half22float2(qp2[2 * c]), bb = __half22float2(qp2[2 * c + 1]);
                            s[4 * c + 0] = a.x + u.x; s[4 * c + 1] = a.y + u.y; s[4 * c + 2] = bb.x + u.z; s[4 * c + 3] = bb.y + u.w;
                        }
                        tmem_ld_wait();
                        const int off = kk0 - lo;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const bool in = hi >= lo && static_cast<unsigned>(off + i) <= span;
                            s[i] = in ? (__uint_as_float(r[i]) + s[i]) * scale2 : -INFINITY;
                        }
                    }
                    if (pass == 0) {
                        if (live) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, s[i]);
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            float p0 = 0.0f, p1 = 0.0f;                     // ex2(-inf) = 0
                            if (live) {
                                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(s[2 * e] - mx));
                                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(s[2 * e + 1] - mx));
                            }
                            sum += p0 + p1;
                            const __half2 h = __floats2half2_rn(p0, p1);
                            w[e] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                    }
                    if (pass == 1) {
                        if (b > 0) ok = att_wait(&sm.bar[B_PV_DONE + b - 1], abort_flag);   // the buffer is free
                        if (ok) {
                            uint8_t* atom = sm.q + (part / 2) * kAtomBytes;   // keys 64 * (part / 2) .. + 63 of the block
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                *reinterpret_cast<uint4*>(atom + swz(ql, 4 * (part % 2) + e)) =
                                    make_uint4(w[4 * e], w[4 * e + 1], w[4 * e + 2], w[4 * e + 3]);
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&sm.bar[B_P_READY + b]);
                        }
                    }
                }
                if (pass == 0) {
                    sm.rowmax[part][ql] = mx;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm.bar[B_MAX + quad]);
                    ok = att_wait(&sm.bar[B_MAX + quad], abort_flag);
                    mx = fmaxf(fmaxf(sm.rowmax[0][ql], sm.rowmax[1][ql]), fmaxf(sm.rowmax[2][ql], sm.rowmax[3][ql]));
                    if (mx == -INFINITY) mx = 0.0f;            // a query without keys: every probability is 0
                }
            }
            if (!ok) break;
            sm.rowsum[part][ql] = sum;
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.bar[B_SUM + quad]);
            ATT_WAIT(B_SUM + quad);
            sum = (sm.rowsum[0][ql] + sm.rowsum[1][ql]) + (sm.rowsum[2][ql] + sm.rowsum[3][ql]);
            const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
            ATT_WAIT(B_PV_DONE + 2);
            tc_fence_after_sync();
            // context: this warp writes features [32 * part, +32) of its 32 queries
            {
                uint32_t r[32];
                tmem_ld_32x32(lane_addr + kCtxCol + static_cast<uint32_t>(part * 32), r);
                tmem_ld_wait();
                if (ql < rows_here) {
                    uint32_t w[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const __half2 h = __floats2half2_rn(__uint_as_float(r[2 * i]) * inv, __uint_as_float(r[2 * i + 1]) * inv);
                        w[i] = q_live ? *reinterpret_cast<const uint32_t*>(&h) : 0u;
                    }
                    uint4* dst = reinterpret_cast<uint4*>(p.out + static_cast<size_t>(base + q0 + ql) * p.ldo + head * kDim + part * 32);
#pragma unroll
                    for (int i = 0; i < 4; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
                }
            }
        } while (false);
    }

    // ------------------------------------------------------------------- teardown
    if (*abort_flag != 0) {
        // give copies / MMAs still in flight time to land before shared and tensor memory are released
        const uint64_t start = global_timer_ns();
        while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
        if (tid == 0 && p.status != nullptr) atomicExch(p.status, 1);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kSoftmaxWarps + 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace att5
}  // namespace pk100

using namespace pk100;

extern "C" int pk100_local_relpos_attention_tcgen05(
    void* stream_v, const void* query, int ldq, const void* key, int ldk, const void* value, int ldv,
    const void* position, const void* bias_u, const void* bias_v, void* output, int ldo, int segments,
    int seg_stride, int valid_rows, const int* seg_valid, int* status) {
    using namespace att5;
    if (!query || !key || !value || !position || !bias_u || !bias_v || !output) return PK100_ERR_NULL;
    if (segments < 0 || seg_stride <= 0) return PK100_ERR_SHAPE;
    if (seg_stride % kTile != 0) return PK100_ERR_SHAPE;          // whole 128-query tiles
    if (ldq < 1024 || ldk < 1024 || ldv < 1024 || ldo < 1024 || (ldq | ldk | ldv | ldo) % 8 != 0) return PK100_ERR_SHAPE;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(query) | reinterpret_cast<uintptr_t>(key) |
                           reinterpret_cast<uintptr_t>(value) | reinterpret_cast<uintptr_t>(position) |
                           reinterpret_cast<uintptr_t>(output);
    if (bits & 15u) return PK100_ERR_ALIGN;
    if (segments == 0) return PK100_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const unsigned long long rows = static_cast<unsigned long long>(segments) * seg_stride;

    CUtensorMap map_q, map_k, map_p, map_p16, map_v;
    int rc = pk100_tensor_map_2d(&map_q, query, 2, rows, 1024, ldq, kTile, 128);
    if (rc == PK100_OK) rc = pk100_tensor_map_2d(&map_k, key, 2, rows, 1024, ldk, 128, 128);
    if (rc == PK100_OK) rc = pk100_tensor_map_2d(&map_p, position, 2, kHeads * kPosRows, kDim, kDim, 128, 128);
    if (rc == PK100_OK) rc = pk100_tensor_map_2d(&map_p16, position, 2, kHeads * kPosRows, kDim, kDim, 16, 128);
    if (rc == PK100_OK) rc = pk100_tensor_map_2d(&map_v, value, 2, rows, 1024, ldv, 128, 128);
    if (rc != PK100_OK) return rc;

    constexpr int smem_bytes = static_cast<int>(sizeof(Smem)) + 1024;
    static bool configured = false;
    if (!configured) {
        const cudaError_t err = cudaFuncSetAttribute(local_attention_tcgen05_kernel,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (err != cudaSuccess) return static_cast<int>(err);
        configured = true;
    }
    Params p{static_cast<const __half*>(bias_u), static_cast<const __half*>(bias_v), static_cast<__half*>(output), ldo,
             segments, seg_stride, valid_rows, seg_valid, status};
    dim3 grid(seg_stride / kTile, kHeads, segments);
    pk100_launch_chained(local_attention_tcgen05_kernel, grid, dim3(kThreads), smem_bytes, stream, map_q, map_k, map_p, map_p16, map_v, p);
    return pk100_launch_status();
}
