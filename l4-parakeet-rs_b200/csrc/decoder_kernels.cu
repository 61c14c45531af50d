// TDT greedy decode for a batch of up to 8 utterances that advance in lockstep rounds
// (a round = LSTM -> prediction projection for the utterances that just emitted a token, then
// joint + argmax for all live ones).  Three kernels share one contract and one set of decision
// rules:
//   tdt_cluster_kernel   one 16-CTA thread-block cluster; vectors are exchanged through
//                        distributed shared memory (st.async + mbarrier complete_tx), layer 0's
//                        recurrent weights live in tensor memory, the joint rows in shared
//                        memory, the rest streams from L2.  The kernel of the hot path.
//   tdt_exchange_kernel  one CTA per SM, all weights resident in shared memory, exchanges
//                        through tagged 64-bit global-memory slots (no cluster needed).
//   tdt_greedy_kernel    one persistent cooperative kernel with the reference's structure: per
//                        round [LSTM layer 0 | barrier | LSTM layer 1 | barrier | prediction
//                        projection | barrier], then joint + argmax | barrier.  A cross-check.
// The cluster and the barrier kernel also have the numerics of the reference's long-request
// kernel (INT8 codes of the recurrent weights and of the hidden state, kernels/sm89/
// decoder.cu:452-784).  Every wait (grid barrier, mbarrier, slot poll) is bounded: when one
// expires the kernel records it in the status word and every CTA leaves.
//
// Decision rules follow kernels/sm89/decoder.cu:35-46 (order-preserving key,
// ties to the lower token id), :416-422 (first strict maximum duration) and
// :431-445 (frame advance, at most 10 symbols per frame, blank keeps the state).
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <limits.h>
#include <float.h>
#include <stdint.h>

#include <atomic>
#include <type_traits>

#include "pk100_internal.h"
#include "ptx_sm100.cuh"

namespace pk100 {

constexpr int kHidden = 640;
constexpr int kGates = 4 * kHidden;
constexpr int kTokenOutputs = 1025;
constexpr int kBlank = 1024;
constexpr int kDurations = 5;
constexpr int kJointRows = kTokenOutputs + kDurations;
constexpr int kMaxSymbols = 10;
constexpr int kMaxUtt = PK100_DECODER_MAX_UTTERANCES;
constexpr int kDecThreads = 512;
constexpr int kDecWarps = kDecThreads / 32;

// Workspace layout (floats), per utterance u:
//   state[u][bank 0/1][h l0 | h l1 | c l0 | c l1]   2 * 4 * 640
//   pred[u][640]
// then per utterance 3 decision slots (u64) and 3 x 5 duration logits, then the
// barrier words.  Sized by pk100_tdt_workspace_bytes().
constexpr int kStatePerUtt = 2 * 4 * kHidden;
struct DecLayout {
    size_t state, pred, decisions, durations, barrier, total;
};
__host__ __device__ inline DecLayout dec_layout(int utts) {
    DecLayout l;
    size_t off = 0;
    l.state = off; off += static_cast<size_t>(utts) * kStatePerUtt * 4;
    l.pred = off; off += static_cast<size_t>(utts) * kHidden * 4;
    off = (off + 15) / 16 * 16;
    l.decisions = off; off += static_cast<size_t>(utts) * 3 * 8;
    l.durations = off; off += static_cast<size_t>(utts) * 3 * kDurations * 4;
    off = (off + 255) / 256 * 256;
    l.barrier = off; off += 256;
    l.total = off;
    return l;
}

struct DecParams {
    const __half* enc_proj;      // [utts * seg_stride, 640]
    int seg_stride;
    const int* frames;           // [utts] frames to decode per utterance (device)
    int utts, layers;
    const __half* embedding;     // [1025, 640]
    const __half* w_ih[2];       // [2560, 640]
    const __half* w_hh[2];
    const float* b_ih[2];        // [2560]
    const float* b_hh[2];
    const __half* w_pred;        // [640, 640]
    const float* b_pred;
    const __half* w_joint;       // [1030, 640]
    const float* b_joint;
    uint8_t* workspace;
    int32_t* tokens;             // [utts, max_tokens]
    int32_t* durations_out;      // [utts, max_tokens] or nullptr
    int32_t* counts;             // [utts]
    int max_tokens;
    int* status;
    // Long-request numerics (the reference's kernel for 1024 frames or more): max |w| of
    // w_hh[0], w_hh[1], w_ih[1] as three floats in device memory; nullptr = fp16 weights.
    const float* cache_absmax;
    // Long-request numerics: fp32 [1025, 2560] table embedding . w_ih[0]^T, entries rounded to fp16
    // (src/cuda/decoder.rs:355-383), built by a tensor-core GEMM like the reference's.
    const float* input_table;
    // Only utterances with frames_lo <= frames[u] < frames_hi take part (cluster and barrier
    // kernels); the others are left alone, their counts unwritten.
    int frames_lo, frames_hi;
};
__device__ __forceinline__ bool in_window(const DecParams& p, int u) {
    const int f = p.frames[u];
    return f >= p.frames_lo && f < p.frames_hi;
}

// INT8 cache of the long-request kernel (kernels/sm89/decoder.cu:96-98, :552-553, :568-572):
// codes = rne(w / scale) clamped to +-127 with scale = max|w| / 127 per tensor; the hidden state
// that multiplies them is rne(h * 127).  Codes and their 640-term dot products are integers
// below 2^24, so fp16 storage and fp32 (or tensor-core) accumulation reproduce the integer
// arithmetic exactly in any summation order.
//
// The reference builds its decoder unit with --use_fast_math (build.rs:78-83, :100-102), which
// replaces x / y by __fdividef, expf by __expf and tanhf by __tanhf.  The 8-bit rounding of h turns
// the error of those approximations (tanh: about 2^-11 relative) into different codes, so the
// long-request numerics are reproduced with the same intrinsics, spelled out here because this
// library is built without that flag.
__device__ __forceinline__ int quantize_i8(float v) { return max(-127, min(127, __float2int_rn(v))); }
__device__ __forceinline__ float cache_scale(const float* absmax, int i) {
    const float m = absmax[i];
    return m > 0.0f ? __fdividef(m, 127.0f) : 1.0f;
}
__device__ __forceinline__ float cache_mul(float scale) { return __fdividef(scale, 127.0f); }
__device__ __forceinline__ __half cache_code(__half w, float scale) {
    return __int2half_rn(quantize_i8(__fdividef(__half2float(w), scale)));
}
__device__ __forceinline__ float ref_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float ref_tanh(float x) { return __tanhf(x); }
// lstm_cell of decoder.cu:148-163 under those substitutions; returns h
__device__ __forceinline__ float ref_lstm_cell(const float (&gate)[4], float& cstate) {
    const float ig = ref_sigmoid(gate[0]), fg = ref_sigmoid(gate[1]);
    const float gg = ref_tanh(gate[2]), og = ref_sigmoid(gate[3]);
    // The reference's compiled form of `forget * c + input * g` fuses the input-gate product onto
    // the ROUNDED forget-gate product; found by running its kernel beside this one: the other two
    // forms part from its tokens after a few hundred steps (the 8-bit rounding of h amplifies one ulp).
    const float cell = fmaf(ig, gg, __fmul_rn(fg, cstate));
    cstate = cell;
    return __fmul_rn(og, ref_tanh(cell));
}

// max |w| over a tensor; `out` holds the bits of a non-negative float (ordered like unsigned), zeroed before
__global__ void tdt_absmax_kernel(const __half* __restrict__ w, int n, unsigned* out) {
    float m = 0.0f;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        m = fmaxf(m, fabsf(__half2float(w[i])));
#pragma unroll
    for (int off = 16; off > 0; off /= 2) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if (threadIdx.x % 32 == 0) atomicMax(out, __float_as_uint(m));
}

__device__ __forceinline__ bool better(float s, int id, float os, int oid) {
    return s > os || (s == os && id < oid);
}

__device__ __forceinline__ unsigned long long decision_key(float score, int id) {
    if (score == 0.0f) score = 0.0f;     // canonicalise -0
    const unsigned bits = __float_as_uint(score);
    const unsigned ordered = (bits & 0x80000000u) ? ~bits : (bits ^ 0x80000000u);
    return (static_cast<unsigned long long>(ordered) << 32) | (0xffffffffu - static_cast<unsigned>(id));
}

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int off = 16; off > 0; off /= 2) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Bounded grid barrier: counter + generation word in global memory.
struct GridBarrier {
    unsigned* count;
    volatile unsigned* generation;
    volatile int* abort;
    unsigned expected;
    unsigned local_gen;

    __device__ bool sync() {
        __shared__ int s_ok;
        __syncthreads();
        if (threadIdx.x == 0) {
            int ok = 1;
            __threadfence();
            const unsigned target = local_gen + 1;
            if (atomicAdd(count, 1u) == expected - 1) {
                *count = 0;
                __threadfence();
                *generation = target;
            } else {
                const unsigned long long start = clock64();
                unsigned polls = 0;
                while (*generation != target) {
                    if ((++polls & 255u) == 0u) {
                        // ~2e9 cycles is about one second: far beyond any legal wait
                        if (*abort != 0 || clock64() - start > 2000000000ull) {
                            *abort = 1;
                            ok = 0;
                            break;
                        }
                    }
                }
            }
            __threadfence();
            s_ok = ok;
        }
        __syncthreads();
        local_gen += 1;
        return s_ok != 0;
    }
};

__device__ __forceinline__ float dot640(const __half* w_smem, const float* x_smem, int lane) {
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < kHidden / 64; ++i) {
        const int idx = 2 * lane + 64 * i;
        const float2 w = __half22float2(*reinterpret_cast<const __half2*>(w_smem + idx));
        const float2 x = *reinterpret_cast<const float2*>(x_smem + idx);
        acc = fmaf(w.x, x.x, acc);
        acc = fmaf(w.y, x.y, acc);
    }
    return acc;
}

// The same dot products in the summation order of the reference's long-request kernel
// (decoder.cu:672-684, :697-713): the bias starts the fma chain of lane 0; a prediction row is
// spread over the 32 lanes (elements 2l + 64w), a joint row over a half-warp (elements 2l + 32s).
// Every lane returns the sum.
__device__ __forceinline__ float dot640_ref_warp(const __half* w_smem, const float* x_smem, int lane, float bias) {
    float acc = lane == 0 ? bias : 0.0f;
#pragma unroll
    for (int i = 0; i < kHidden / 64; ++i) {
        const int idx = 2 * lane + 64 * i;
        const float2 w = __half22float2(*reinterpret_cast<const __half2*>(w_smem + idx));
        const float2 x = *reinterpret_cast<const float2*>(x_smem + idx);
        acc = fmaf(w.x, x.x, acc);
        acc = fmaf(w.y, x.y, acc);
    }
#pragma unroll
    for (int off = 16; off > 0; off /= 2) acc += __shfl_down_sync(0xffffffffu, acc, off);
    return __shfl_sync(0xffffffffu, acc, 0);
}
__device__ __forceinline__ float dot640_ref_half_warp(const __half* w_smem, const float* x_smem, int lane, float bias) {
    const int hl = lane % 16;               // both halves of the warp compute the same row
    float acc = hl == 0 ? bias : 0.0f;
#pragma unroll
    for (int i = 0; i < kHidden / 32; ++i) {
        const int idx = 2 * hl + 32 * i;
        const float2 w = __half22float2(*reinterpret_cast<const __half2*>(w_smem + idx));
        const float2 x = *reinterpret_cast<const float2*>(x_smem + idx);
        acc = fmaf(w.x, x.x, acc);
        acc = fmaf(w.y, x.y, acc);
    }
#pragma unroll
    for (int off = 8; off > 0; off /= 2) acc += __shfl_down_sync(0xffffffffu, acc, off, 16);
    return __shfl_sync(0xffffffffu, acc, 0);
}

__global__ void __launch_bounds__(kDecThreads, 1) tdt_greedy_kernel(const DecParams p) {
    extern __shared__ __align__(16) uint8_t dsmem[];
    const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
    const int G = gridDim.x, cta = blockIdx.x;
    const int units = (kHidden + G - 1) / G;          // hidden units / pred rows per CTA
    const int jrows = (kJointRows + G - 1) / G;       // joint rows per CTA
    const DecLayout lay = dec_layout(p.utts);

    // ---- shared memory carve-up
    __half* s_lstm = reinterpret_cast<__half*>(dsmem);                         // [layers][units][8][640]
    __half* s_pred = s_lstm + static_cast<size_t>(p.layers) * units * 8 * kHidden;   // [units][640]
    __half* s_joint = s_pred + static_cast<size_t>(units) * kHidden;           // [jrows][640]
    float* s_vec = reinterpret_cast<float*>(s_joint + static_cast<size_t>(jrows) * kHidden);  // [utts][1280]
    __shared__ unsigned long long s_best[kMaxUtt];
    __shared__ int s_frame[kMaxUtt], s_symbols[kMaxUtt], s_last[kMaxUtt], s_count[kMaxUtt];
    __shared__ uint8_t s_emitted[kMaxUtt], s_valid[kMaxUtt], s_alt[kMaxUtt], s_done[kMaxUtt];

    // ---- load this CTA's weight slices (once); long-request numerics: INT8 codes of the
    // recurrent weights and of layer 1's input weights, held as fp16 integers
    const bool cache = p.cache_absmax != nullptr;
    float cscale[3] = {1.0f, 1.0f, 1.0f};       // w_hh[0], w_hh[1], w_ih[1]
    if (cache)
        for (int i = 0; i < (p.layers == 2 ? 3 : 1); ++i) cscale[i] = cache_scale(p.cache_absmax, i);
    for (int l = 0; l < p.layers; ++l) {
        for (int i = 0; i < units; ++i) {
            const int unit = cta + G * i;
            for (int r = 0; r < 8; ++r) {
                __half* dst = s_lstm + ((static_cast<size_t>(l) * units + i) * 8 + r) * kHidden;
                const __half* src = (r < 4 ? p.w_ih[l] : p.w_hh[l]) +
                                    (static_cast<size_t>(r & 3) * kHidden + unit) * kHidden;
                const int coded = !cache ? -1 : (r >= 4 ? l : (l == 1 ? 2 : -1));
                for (int c = tid; c < kHidden; c += kDecThreads) {
                    __half v = unit < kHidden ? src[c] : __float2half(0.0f);
                    if (coded >= 0) v = cache_code(v, cscale[coded]);
                    dst[c] = v;
                }
            }
        }
    }
    for (int i = 0; i < units; ++i) {
        const int row = cta + G * i;
        for (int c = tid; c < kHidden; c += kDecThreads)
            s_pred[i * kHidden + c] = row < kHidden ? p.w_pred[static_cast<size_t>(row) * kHidden + c]
                                                    : __float2half(0.0f);
    }
    for (int i = 0; i < jrows; ++i) {
        const int row = cta + G * i;
        for (int c = tid; c < kHidden; c += kDecThreads)
            s_joint[i * kHidden + c] = row < kJointRows ? p.w_joint[static_cast<size_t>(row) * kHidden + c]
                                                        : __float2half(0.0f);
    }

    float* g_state = reinterpret_cast<float*>(p.workspace + lay.state);
    float* g_pred = reinterpret_cast<float*>(p.workspace + lay.pred);
    unsigned long long* g_dec = reinterpret_cast<unsigned long long*>(p.workspace + lay.decisions);
    float* g_dur = reinterpret_cast<float*>(p.workspace + lay.durations);
    unsigned* g_bar = reinterpret_cast<unsigned*>(p.workspace + lay.barrier);

    GridBarrier bar{g_bar, g_bar + 1, reinterpret_cast<volatile int*>(g_bar + 2),
                    static_cast<unsigned>(G), 0u};
    // the launcher zeroes the workspace (state, barrier words) before the kernel starts
    if (tid < p.utts) {
        s_frame[tid] = 0; s_symbols[tid] = 0; s_last[tid] = kBlank; s_count[tid] = 0;
        s_emitted[tid] = 0; s_valid[tid] = 0; s_alt[tid] = 0;
        s_done[tid] = p.frames[tid] <= 0 || !in_window(p, tid);
    }
    if (cta == 0 && tid < p.utts * 3) g_dec[tid] = decision_key(-FLT_MAX, kTokenOutputs);
    bool ok = bar.sync();

    int slot = 0;
    while (ok) {
        // ---- which utterances are still running / need a new prediction
        bool any_running = false, any_update = false;
        for (int u = 0; u < p.utts; ++u) {
            any_running |= !s_done[u];
            any_update |= !s_done[u] && !s_valid[u];
        }
        if (!any_running) break;

        if (any_update) {
            for (int l = 0; l < p.layers && ok; ++l) {
                // stage x (embedding or lower layer's candidate h) and committed h
                for (int u = 0; u < p.utts; ++u) {
                    if (s_done[u] || s_valid[u]) continue;
                    const float* st = g_state + static_cast<size_t>(u) * kStatePerUtt;
                    const float* committed = st + (s_alt[u] ? 4 * kHidden : 0);
                    const float* candidate = st + (s_alt[u] ? 0 : 4 * kHidden);
                    float* vec = s_vec + u * 2 * kHidden;
                    for (int c = tid; c < kHidden; c += kDecThreads) {
                        float x;
                        if (l == 0) {
                            x = s_emitted[u] ? __half2float(p.embedding[static_cast<size_t>(s_last[u]) * kHidden + c])
                                             : 0.0f;
                        } else {
                            x = __ldcg(candidate + (l - 1) * kHidden + c);
                            if (cache) x = static_cast<float>(quantize_i8(x * 127.0f));
                        }
                        vec[c] = x;
                        const float hv = __ldcg(committed + l * kHidden + c);
                        vec[kHidden + c] = cache ? static_cast<float>(quantize_i8(hv * 127.0f)) : hv;
                    }
                }
                __syncthreads();
                for (int task = warp; task < units * p.utts; task += kDecWarps) {
                    const int i = task / p.utts, u = task % p.utts;
                    const int unit = cta + G * i;
                    if (unit >= kHidden || s_done[u] || s_valid[u]) continue;
                    const __half* wrow = s_lstm + (static_cast<size_t>(l) * units + i) * 8 * kHidden;
                    const float* vec = s_vec + u * 2 * kHidden;
                    float gate[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        if (!cache) {
                            float acc = dot640(wrow + r * kHidden, vec, lane) +
                                        dot640(wrow + (4 + r) * kHidden, vec + kHidden, lane);
                            acc = warp_sum_f(acc);
                            gate[r] = acc + p.b_ih[l][r * kHidden + unit] + p.b_hh[l][r * kHidden + unit];
                        } else {
                            // decoder.cu:626-640 (layer 0: recurrent codes + bias + fp16 table entry),
                            // :655-663 (layer 1: recurrent + input codes, then bias)
                            // layer 0: the table entry of the last token (zero before the first one)
                            const float in = l == 0
                                ? (s_emitted[u] ? p.input_table[static_cast<size_t>(s_last[u]) * kGates + r * kHidden + unit] : 0.0f)
                                : warp_sum_f(dot640(wrow + r * kHidden, vec, lane));
                            // rounded product, never fused with the additions that follow (see the cluster kernel)
                            const float rec = __fmul_rn(warp_sum_f(dot640(wrow + (4 + r) * kHidden, vec + kHidden, lane)),
                                                        cache_mul(cscale[l]));
                            const float bias = p.b_ih[l][r * kHidden + unit] + p.b_hh[l][r * kHidden + unit];
                            gate[r] = l == 0 ? __fadd_rn(__fadd_rn(rec, bias), in)
                                             : __fadd_rn(fmaf(in, cache_mul(cscale[2]), rec), bias);
                        }
                    }
                    if (lane == 0) {
                        float* st = g_state + static_cast<size_t>(u) * kStatePerUtt;
                        const float* committed = st + (s_alt[u] ? 4 * kHidden : 0);
                        float* candidate = st + (s_alt[u] ? 0 : 4 * kHidden);
                        if (cache) {
                            float cell = __ldcg(committed + (2 + l) * kHidden + unit);
                            const float h = ref_lstm_cell(gate, cell);
                            __stcg(candidate + (2 + l) * kHidden + unit, cell);
                            __stcg(candidate + l * kHidden + unit, h);
                        } else {
                            const float ig = 1.0f / (1.0f + expf(-gate[0]));
                            const float fg = 1.0f / (1.0f + expf(-gate[1]));
                            const float gg = tanhf(gate[2]);
                            const float og = 1.0f / (1.0f + expf(-gate[3]));
                            const float cell = fg * __ldcg(committed + (2 + l) * kHidden + unit) + ig * gg;
                            __stcg(candidate + (2 + l) * kHidden + unit, cell);
                            __stcg(candidate + l * kHidden + unit, og * tanhf(cell));
                        }
                    }
                }
                ok = bar.sync();
            }
            if (!ok) break;
            // ---- prediction projection from the top layer's candidate h
            for (int u = 0; u < p.utts; ++u) {
                if (s_done[u] || s_valid[u]) continue;
                const float* st = g_state + static_cast<size_t>(u) * kStatePerUtt;
                const float* candidate = st + (s_alt[u] ? 0 : 4 * kHidden);
                for (int c = tid; c < kHidden; c += kDecThreads)
                    s_vec[u * 2 * kHidden + c] = __ldcg(candidate + (p.layers - 1) * kHidden + c);
            }
            __syncthreads();
            for (int task = warp; task < units * p.utts; task += kDecWarps) {
                const int i = task / p.utts, u = task % p.utts;
                const int row = cta + G * i;
                if (row >= kHidden || s_done[u] || s_valid[u]) continue;
                const float acc = cache
                    ? dot640_ref_warp(s_pred + i * kHidden, s_vec + u * 2 * kHidden, lane, p.b_pred[row])
                    : warp_sum_f(dot640(s_pred + i * kHidden, s_vec + u * 2 * kHidden, lane)) + p.b_pred[row];
                if (lane == 0) __stcg(g_pred + static_cast<size_t>(u) * kHidden + row, acc);
            }
            ok = bar.sync();
            if (!ok) break;
            if (tid < p.utts && !s_done[tid]) s_valid[tid] = 1;
            __syncthreads();
        }

        // ---- joint network + argmax
        const int next_slot = slot == 2 ? 0 : slot + 1;
        if (tid < p.utts) {
            s_best[tid] = decision_key(-FLT_MAX, kTokenOutputs);
            if (cta == 0) g_dec[tid * 3 + next_slot] = decision_key(-FLT_MAX, kTokenOutputs);
        }
        for (int u = 0; u < p.utts; ++u) {
            if (s_done[u]) continue;
            const __half* enc = p.enc_proj + (static_cast<size_t>(u) * p.seg_stride + s_frame[u]) * kHidden;
            const float* pred = g_pred + static_cast<size_t>(u) * kHidden;
            for (int c = tid; c < kHidden; c += kDecThreads)
                s_vec[u * 2 * kHidden + c] = fmaxf(__half2float(enc[c]) + __ldcg(pred + c), 0.0f);
        }
        __syncthreads();
        for (int task = warp; task < jrows * p.utts; task += kDecWarps) {
            const int i = task / p.utts, u = task % p.utts;
            const int row = cta + G * i;
            if (row >= kJointRows || s_done[u]) continue;
            float acc = cache
                ? dot640_ref_half_warp(s_joint + i * kHidden, s_vec + u * 2 * kHidden, lane, p.b_joint[row])
                : warp_sum_f(dot640(s_joint + i * kHidden, s_vec + u * 2 * kHidden, lane)) + p.b_joint[row];
            if (lane == 0) {
                if (row >= kTokenOutputs) {
                    __stcg(g_dur + (static_cast<size_t>(u) * 3 + slot) * kDurations + (row - kTokenOutputs), acc);
                } else if (acc == acc) {          // NaN never wins
                    atomicMax(&s_best[u], decision_key(acc, row));
                }
            }
        }
        __syncthreads();
        if (tid < p.utts && !s_done[tid]) atomicMax(g_dec + tid * 3 + slot, s_best[tid]);
        ok = bar.sync();
        if (!ok) break;

        // ---- every CTA applies the same decisions to its replica of the control state
        if (tid < p.utts && !s_done[tid]) {
            const int u = tid;
            const unsigned long long key = __ldcg(g_dec + u * 3 + slot);
            int token = static_cast<int>(0xffffffffu - static_cast<unsigned>(key));
            // every token score of the round was NaN (no key beat the initial one): a blank, and
            // the call reports it (status bit 4); 1025 is no row of the embedding table
            if (token > kBlank) { token = kBlank; if (cta == 0 && p.status != nullptr) atomicOr(p.status, 4); }
            const float* dl = g_dur + (static_cast<size_t>(u) * 3 + slot) * kDurations;
            int duration = 0;
            float best = __ldcg(dl);
            for (int i = 1; i < kDurations; ++i) {
                const float v = __ldcg(dl + i);
                if (v > best) { best = v; duration = i; }
            }
            if (token != kBlank) {
                if (cta == 0 && s_count[u] < p.max_tokens) {
                    p.tokens[static_cast<size_t>(u) * p.max_tokens + s_count[u]] = token;
                    if (p.durations_out != nullptr)
                        p.durations_out[static_cast<size_t>(u) * p.max_tokens + s_count[u]] = duration;
                }
                s_count[u] += 1;
                s_last[u] = token;
                s_emitted[u] = 1;
                s_valid[u] = 0;
                s_alt[u] ^= 1;
            }
            s_symbols[u] += 1;
            s_frame[u] += duration;
            if (duration != 0 || s_symbols[u] == kMaxSymbols) {
                if (duration == 0) s_frame[u] += 1;
                s_symbols[u] = 0;
            }
            if (s_frame[u] >= min(p.frames[u], p.seg_stride)) s_done[u] = 1;   // never past the utterance's block
        }
        __syncthreads();
        slot = next_slot;
    }

    if (cta == 0 && tid < p.utts && in_window(p, tid)) p.counts[tid] = min(s_count[tid], p.max_tokens);
    if (!ok && cta == 0 && tid == 0 && p.status != nullptr) atomicExch(p.status, 2);
}

}  // namespace pk100

namespace pk100 {

// ===========================================================================
// Exchange-based decoder (the hot-path kernel).
//
// Same slicing of the work across one CTA per SM (every weight slice resident in shared
// memory; each of the 20 warps owns one gate row of one hidden unit and computes it for
// all utterances at once), but there is no grid barrier: producers publish every value together with a tag
// ({fp32 value, u32 tag} in one 64-bit store) and consumers poll the data itself until
// the tag matches the version they need.  Tags are the per-utterance LSTM version for
// hidden states / prediction vectors and the round number for the joint decisions, so
// a slot can never be confused with its previous content, and nobody can run two
// versions ahead of anybody else because every decision needs a key from every CTA.
// Every poll is bounded; when one expires the kernel raises a global abort flag,
// records status 2 and all CTAs leave.
constexpr int kXThreads = 640;
constexpr int kXWarps = kXThreads / 32;
constexpr int kXMaxGrid = 256;
constexpr unsigned kEpochMask = 0x1FFFFFu;

struct XchLayout { size_t xh, xp, xk, xd, abort, total; };
__host__ __device__ inline XchLayout xch_layout(int utts) {
    XchLayout l;
    size_t off = 0;
    l.xh = off; off += static_cast<size_t>(2) * 2 * utts * kHidden * 8;
    l.xp = off; off += static_cast<size_t>(2) * utts * kHidden * 8;
    l.xk = off; off += static_cast<size_t>(2) * utts * kXMaxGrid * 8;
    l.xd = off; off += static_cast<size_t>(2) * utts * 8 * 8;
    l.abort = off; off += 256;
    l.total = off;
    return l;
}

__device__ __forceinline__ void xch_store(unsigned long long* slot, float value, unsigned tag) {
    const unsigned long long packed = (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(value);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(slot), "l"(packed) : "memory");
}
__device__ __forceinline__ unsigned long long xch_load(const unsigned long long* slot) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(slot) : "memory");
    return v;
}

// Poll one tagged slot until its tag equals `tag`.  Returns false (and raises the global
// abort flag) when the budget runs out or another thread already gave up.
__device__ __forceinline__ bool xch_wait(const unsigned long long* slot, unsigned tag, float* value,
                                         volatile int* abort_flag) {
    unsigned long long v = xch_load(slot);
    if (static_cast<unsigned>(v >> 32) != tag) {
        const long long start = clock64();
        unsigned polls = 0;
        do {
            v = xch_load(slot);
            if ((++polls & 127u) == 0u) {
                if (*abort_flag != 0 || clock64() - start > 2000000000ll) {   // ~1 s
                    *abort_flag = 1;
                    return false;
                }
            }
        } while (static_cast<unsigned>(v >> 32) != tag);
    }
    *value = __uint_as_float(static_cast<unsigned>(v));
    return true;
}


// Column `c` of up to 8 utterances at once: all loads are issued before any tag is
// checked, so a phase costs one memory round trip when the data is already there.
// slot(u) = base + u * stride; want[u] == 0 means "skip utterance u".
__device__ __forceinline__ bool xch_wait8(const unsigned long long* base, size_t stride, const unsigned (&want)[8],
                                          const size_t (&offset)[8], float (&value)[8], volatile int* abort_flag) {
    unsigned long long v[8];
    unsigned pending = 0;
#pragma unroll
    for (int u = 0; u < 8; ++u)
        if (want[u] != 0u) {
            pending |= 1u << u;
            v[u] = xch_load(base + u * stride + offset[u]);
        }
    long long start = 0;
    unsigned polls = 0;
    while (true) {
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if ((pending >> u) & 1u) {
                if (static_cast<unsigned>(v[u] >> 32) == want[u]) {
                    pending &= ~(1u << u);
                    value[u] = __uint_as_float(static_cast<unsigned>(v[u]));
                }
            }
        if (pending == 0u) return true;
        if (polls == 0u) start = clock64();
        if ((++polls & 63u) == 0u && (*abort_flag != 0 || clock64() - start > 2000000000ll)) {   // ~1 s
            *abort_flag = 1;
            return false;
        }
        // reload every entry that is still missing, all loads in flight together
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if ((pending >> u) & 1u) v[u] = xch_load(base + u * stride + offset[u]);
    }
}

// Sum 8 per-lane partials across the warp with 9 shuffles.  On return every lane holds
// the total of utterance  u = 4*bit4(lane) + 2*bit3(lane) + bit2(lane).
__device__ __forceinline__ float reduce8(const float (&v)[8], int lane) {
    float a[4], b[2], c;
    const bool hi16 = lane & 16, hi8 = lane & 8, hi4 = lane & 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float send = hi16 ? v[j] : v[j + 4];
        const float recv = __shfl_xor_sync(0xffffffffu, send, 16);
        a[j] = (hi16 ? v[j + 4] : v[j]) + recv;
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const float send = hi8 ? a[j] : a[j + 2];
        const float recv = __shfl_xor_sync(0xffffffffu, send, 8);
        b[j] = (hi8 ? a[j + 2] : a[j]) + recv;
    }
    {
        const float send = hi4 ? b[0] : b[1];
        const float recv = __shfl_xor_sync(0xffffffffu, send, 4);
        c = (hi4 ? b[1] : b[0]) + recv;
    }
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    return c;
}

__device__ __forceinline__ void load_row_slices(const __half* row, int lane, __half2 (&w)[10]) {
#pragma unroll
    for (int m = 0; m < 10; ++m) w[m] = *reinterpret_cast<const __half2*>(row + 2 * lane + 64 * m);
}

// partial dot of this lane's 20 weights with x[u][...] for 8 utterances
__device__ __forceinline__ void dot8(const __half2 (&w)[10], const float* x, int lane, float (&acc)[8]) {
#pragma unroll
    for (int m = 0; m < 10; ++m) {
        const float2 wf = __half22float2(w[m]);
        const int idx = 2 * lane + 64 * m;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float2 xv = *reinterpret_cast<const float2*>(x + u * kHidden + idx);
            acc[u] = fmaf(wf.x, xv.x, acc[u]);
            acc[u] = fmaf(wf.y, xv.y, acc[u]);
        }
    }
}

// Activations are kept as fp16 (hi, lo) pairs: x = hi + lo to ~2^-22, so the tiny GEMMs of
// a round run on tensor cores (mma.sync m16n8k16, fp32 accumulate) without losing the fp32
// state: rows 0-7 of an A tile hold the hi parts of utterances 0-7, rows 8-15 the lo parts,
// and the two halves of each accumulator column are added after the MMA.
constexpr int kAct = kHidden + 8;            // padded pitch (halves) of activation / weight rows
constexpr int kLstmK = 2 * kHidden;          // [input | recurrent]
constexpr int kLstmPitch = kLstmK + 8;
constexpr int kLstmRows = 20;                // 5 hidden units x 4 gates per CTA

struct XSmem {
    __half wl[2][kLstmRows][kLstmPitch];  // [layer][unit slot * 4 + gate][w_ih row | w_hh row]
    __half wp[8][kAct];                   // this CTA's prediction-projection rows
    __half wj[8][kAct];                   // this CTA's joint rows
    __half ax[16][kAct];                  // LSTM input / joint input (hi rows 0-7, lo rows 8-15)
    __half ah[2][16][kAct];               // committed hidden state per layer, all 640 units
    float part[kXWarps][8][24];           // per-warp partial sums of the K-split
    float pred[kMaxUtt][kHidden];         // cached prediction vectors
    float gate[kMaxUtt][8][4];            // [utt][unit slot][gate]
    float cstate[2][2][8][kMaxUtt];       // [layer][version parity][unit slot][utt]
    float bias[2][8][4];                  // b_ih + b_hh per owned unit and gate
    float pred_bias[8];
    float joint_bias[8];
    unsigned long long best[kMaxUtt];
    unsigned long long rowkey[kMaxUtt][8];   // this CTA's joint rows: one key per (utterance, row slot)
    float dur[kMaxUtt][8];
    int frame[kMaxUtt], symbols[kMaxUtt], last[kMaxUtt], count[kMaxUtt], ver[kMaxUtt], pred_ver[kMaxUtt];
    int total_frames[kMaxUtt];
    alignas(8) unsigned char emitted[kMaxUtt];
    alignas(8) unsigned char valid[kMaxUtt];
    alignas(8) unsigned char done[kMaxUtt];      // read as one 64-bit word: entries >= utts are 1
    alignas(8) unsigned char need[kMaxUtt];      // !done && !valid, refreshed at the end of every round
    int ok;
};

__device__ __forceinline__ void split_store(__half (*buf)[kAct], int u, int col, float v) {
    const __half hi = __float2half_rn(v);
    buf[u][col] = hi;
    buf[u + 8][col] = __float2half_rn(v - __half2float(hi));
}

__device__ __forceinline__ void dec_ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void dec_ldmatrix_x2(unsigned (&r)[2], const void* smem) {
    const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
                 : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void dec_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

#ifdef PK100_DEC_PROFILE
#define PK_STAMP(i) do { if (tid == 0) { const long long now__ = clock64(); prof[i] += now__ - last_stamp; last_stamp = now__; } } while (0)
#else
#define PK_STAMP(i) do { } while (0)
#endif

__global__ void __launch_bounds__(kXThreads, 1) tdt_exchange_kernel(const DecParams p) {
#ifdef PK100_DEC_PROFILE
    long long prof[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    long long last_stamp = clock64();
#endif
    extern __shared__ __align__(16) uint8_t xs_raw[];
    XSmem& sm = *reinterpret_cast<XSmem*>(xs_raw);
    const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
    const int g = lane / 4, t = lane % 4;
    const int G = gridDim.x, cta = blockIdx.x;
    const int units = (kHidden + G - 1) / G;            // <= 5 (checked on the host)
    const int jrows = (kJointRows + G - 1) / G;         // <= 8
    const XchLayout lay = xch_layout(p.utts);
    unsigned long long* xh = reinterpret_cast<unsigned long long*>(p.workspace + lay.xh);
    unsigned long long* xp = reinterpret_cast<unsigned long long*>(p.workspace + lay.xp);
    unsigned long long* xk = reinterpret_cast<unsigned long long*>(p.workspace + lay.xk);
    unsigned long long* xd = reinterpret_cast<unsigned long long*>(p.workspace + lay.xd);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(p.workspace + lay.abort);
    const int U = p.utts;

    // ---- this CTA's weight slices -> shared memory (once)
    for (int i = tid; i < 2 * kLstmRows * kLstmPitch; i += kXThreads) {
        const int c = i % kLstmPitch, n = (i / kLstmPitch) % kLstmRows, l = i / (kLstmRows * kLstmPitch);
        const int slot = n / 4, gt = n % 4;
        const int unit = cta + G * slot;
        __half v = __float2half(0.0f);
        if (l < p.layers && slot < units && unit < kHidden && c < kLstmK) {
            const __half* src = c < kHidden ? p.w_ih[l] : p.w_hh[l];
            v = src[(static_cast<size_t>(gt) * kHidden + unit) * kHidden + (c % kHidden)];
        }
        sm.wl[l][n][c] = v;
    }
    for (int i = tid; i < 8 * kAct; i += kXThreads) {
        const int slot = i / kAct, c = i % kAct;
        const int row = cta + G * slot;
        sm.wp[slot][c] = (slot < units && row < kHidden && c < kHidden)
            ? p.w_pred[static_cast<size_t>(row) * kHidden + c] : __float2half(0.0f);
        sm.wj[slot][c] = (slot < jrows && row < kJointRows && c < kHidden)
            ? p.w_joint[static_cast<size_t>(row) * kHidden + c] : __float2half(0.0f);
    }
    for (int i = tid; i < 16 * kAct; i += kXThreads) {
        (&sm.ax[0][0])[i] = __float2half(0.0f);
        (&sm.ah[0][0][0])[i] = __float2half(0.0f);
        (&sm.ah[1][0][0])[i] = __float2half(0.0f);
    }
    for (int i = tid; i < kMaxUtt * kHidden; i += kXThreads) (&sm.pred[0][0])[i] = 0.0f;
    for (int i = tid; i < 2 * 2 * 8 * kMaxUtt; i += kXThreads) (&sm.cstate[0][0][0][0])[i] = 0.0f;
    if (tid < 2 * 8 * 4) {
        const int l = tid / 32, slot = (tid / 4) % 8, gt = tid % 4;
        const int unit = cta + G * slot;
        sm.bias[l][slot][gt] = (l < p.layers && slot < units && unit < kHidden)
            ? p.b_ih[l][gt * kHidden + unit] + p.b_hh[l][gt * kHidden + unit] : 0.0f;
    }
    if (tid < 8) {
        const int row = cta + G * tid;
        sm.pred_bias[tid] = (tid < units && row < kHidden) ? p.b_pred[row] : 0.0f;
        sm.joint_bias[tid] = (tid < jrows && row < kJointRows) ? p.b_joint[row] : 0.0f;
    }
    if (tid < kMaxUtt) {
        sm.frame[tid] = 0; sm.symbols[tid] = 0; sm.last[tid] = kBlank; sm.count[tid] = 0;
        sm.ver[tid] = 0; sm.pred_ver[tid] = 0; sm.emitted[tid] = 0; sm.valid[tid] = 0;
        sm.total_frames[tid] = tid < U ? min(p.frames[tid], p.seg_stride) : 0;   // never past the utterance's block
        sm.done[tid] = tid >= U || p.frames[tid] <= 0;
        sm.need[tid] = !(tid >= U || p.frames[tid] <= 0);
    }
    if (tid == 0) sm.ok = 1;
    __syncthreads();

    // One K-split GEMM: out[u][n] partials of A(16 x 16*ksteps) . B(n x K)^T for this warp's
    // k-steps, hi/lo rows folded, written to sm.part[warp][u][n].  NT = number of 8-row tiles.
    auto small_gemm = [&](const __half (*a)[kAct], int a_col0, const __half* b, int b_pitch, int b_rows,
                          int b_col0, int ksteps, auto nt_tag) {
        constexpr int NT = decltype(nt_tag)::value;
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[j][e] = 0.0f;
        for (int ks = 0; ks < ksteps; ++ks) {
            unsigned af[4];
            dec_ldmatrix_x4(af, &a[lane % 16][a_col0 + ks * 16 + (lane / 16) * 8]);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                // B tile j: rows j*8 .. j*8+7 (clamped into the stored rows; surplus columns unused)
                int row = j * 8 + lane % 8;
                row = row < b_rows ? row : b_rows - 1;
                unsigned bf[2];
                dec_ldmatrix_x2(bf, b + static_cast<size_t>(row) * b_pitch + b_col0 + ks * 16 + ((lane / 8) % 2) * 8);
                dec_mma(acc[j], af, bf[0], bf[1]);
            }
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            sm.part[warp][g][j * 8 + 2 * t] = acc[j][0] + acc[j][2];
            sm.part[warp][g][j * 8 + 2 * t + 1] = acc[j][1] + acc[j][3];
        }
    };
    auto sum_parts = [&](int u, int n, int warps) {
        float v = 0.0f;
        for (int w = 0; w < warps; ++w) v += sm.part[w][u][n];
        return v;
    };

    unsigned round = 0;
    while (true) {
        const unsigned long long done8 = *reinterpret_cast<const unsigned long long*>(sm.done);
        const unsigned long long need8 = *reinterpret_cast<const unsigned long long*>(sm.need);
        if (done8 == 0x0101010101010101ull || sm.ok == 0) break;
        const bool any_need = need8 != 0ull;
        PK_STAMP(0);

        if (any_need) {
            for (int l = 0; l < p.layers; ++l) {
                if (sm.ok == 0) break;
                // input of layer l (one thread per column: kXThreads == kHidden).  Layer 0 reads
                // the embedding row that the decision warp staged in sm.ax when the token was
                // chosen; upper layers take the lower layer's fresh hidden state from the exchange
                if (l > 0) {
                    unsigned want[8];
                    size_t off[8];
                    float val[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        want[u] = (u < U && sm.need[u]) ? static_cast<unsigned>(sm.ver[u] + 1) : 0u;
                        off[u] = (static_cast<size_t>(l - 1) * 2 + (want[u] & 1)) * U * kHidden + tid;
                    }
                    if (!xch_wait8(xh, kHidden, want, off, val, abort_flag)) sm.ok = 0;
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (want[u] != 0u) {
                            split_store(sm.ax, u, tid, val[u]);
                            split_store(sm.ah[l - 1], u, tid, val[u]);   // lower layer's next committed state
                        }
                    __syncthreads();
                }
                PK_STAMP(1);
                if (sm.ok == 0) break;
                // gates[u][20 rows] = [x | h] . [w_ih | w_hh]^T, K = 1280 split over the 20 warps
                if (warp < 10) small_gemm(sm.ax, warp * 64, &sm.wl[l][0][0], kLstmPitch, kLstmRows, warp * 64, 4,
                                          std::integral_constant<int, 3>{});
                else small_gemm(sm.ah[l], (warp - 10) * 64, &sm.wl[l][0][0], kLstmPitch, kLstmRows,
                                kHidden + (warp - 10) * 64, 4, std::integral_constant<int, 3>{});
                __syncthreads();
                if (tid < 8 * kLstmRows) {
                    const int u = tid / kLstmRows, n = tid % kLstmRows;
                    sm.gate[u][n / 4][n % 4] = sum_parts(u, n, kXWarps) + sm.bias[l][n / 4][n % 4];
                }
                __syncthreads();
                if (tid < units * U) {
                    const int slot = tid / U, u = tid % U;
                    const int unit = cta + G * slot;
                    if (unit < kHidden && sm.need[u]) {
                        const unsigned tag = static_cast<unsigned>(sm.ver[u] + 1);
                        const float ig = 1.0f / (1.0f + expf(-sm.gate[u][slot][0]));
                        const float fg = 1.0f / (1.0f + expf(-sm.gate[u][slot][1]));
                        const float gg = tanhf(sm.gate[u][slot][2]);
                        const float og = 1.0f / (1.0f + expf(-sm.gate[u][slot][3]));
                        const float cell = fg * sm.cstate[l][(tag & 1) ^ 1][slot][u] + ig * gg;
                        sm.cstate[l][tag & 1][slot][u] = cell;
                        xch_store(xh + ((static_cast<size_t>(l) * 2 + (tag & 1)) * U + u) * kHidden + unit,
                                  og * tanhf(cell), tag);
                    }
                }
                __syncthreads();
                PK_STAMP(2);
            }
            if (sm.ok == 0) break;
            // ---- top layer's fresh hidden state -> committed copy + prediction projection
            {
                const int top = p.layers - 1;
                unsigned want[8];
                size_t off[8];
                float val[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    want[u] = (u < U && sm.need[u]) ? static_cast<unsigned>(sm.ver[u] + 1) : 0u;
                    off[u] = (static_cast<size_t>(top) * 2 + (want[u] & 1)) * U * kHidden + tid;
                }
                if (!xch_wait8(xh, kHidden, want, off, val, abort_flag)) sm.ok = 0;
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (want[u] != 0u) split_store(sm.ah[top], u, tid, val[u]);
            }
            __syncthreads();
            PK_STAMP(3);
            if (sm.ok == 0) break;
            // pred[u][row] = h_top . w_pred^T, K = 640 split over the 20 warps (2 k-steps each)
            small_gemm(sm.ah[p.layers - 1], warp * 32, &sm.wp[0][0], kAct, 8, warp * 32, 2,
                       std::integral_constant<int, 1>{});
            __syncthreads();
            if (tid < 8 * 8) {
                const int u = tid / 8, slot = tid % 8;
                const int row = cta + G * slot;
                if (u < U && sm.need[u] && slot < units && row < kHidden) {
                    const unsigned tag = static_cast<unsigned>(sm.ver[u] + 1);
                    xch_store(xp + (static_cast<size_t>(tag & 1) * U + u) * kHidden + row,
                              sum_parts(u, slot, kXWarps) + sm.pred_bias[slot], tag);
                }
            }
            PK_STAMP(4);
        }

        // ---- joint: refresh cached prediction vectors whose version changed, build relu(enc + pred)
        {
            unsigned want[8];
            size_t off[8];
            float val[8];
            __half e[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool live = u < U && !sm.done[u];
                // sm.ver is bumped in the state update below; a prediction computed in this
                // round carries version ver + 1
                const int ver_now = sm.ver[u] + (sm.need[u] ? 1 : 0);
                want[u] = (live && sm.pred_ver[u] != ver_now) ? static_cast<unsigned>(ver_now) : 0u;
                off[u] = static_cast<size_t>(want[u] & 1) * U * kHidden + tid;
                if (live)
                    e[u] = __ldg(p.enc_proj + (static_cast<size_t>(u) * p.seg_stride + sm.frame[u]) * kHidden + tid);
            }
            if (!xch_wait8(xp, kHidden, want, off, val, abort_flag)) sm.ok = 0;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (u >= U || sm.done[u]) continue;
                if (want[u] != 0u) sm.pred[u][tid] = val[u];
                split_store(sm.ax, u, tid, fmaxf(__half2float(e[u]) + sm.pred[u][tid], 0.0f));
            }
        }
        __syncthreads();
        PK_STAMP(5);
        if (sm.ok == 0) break;
        if (tid < U) sm.pred_ver[tid] = sm.ver[tid] + (sm.need[tid] ? 1 : 0);
        const unsigned epoch = (round + 1) & kEpochMask;
        small_gemm(sm.ax, warp * 32, &sm.wj[0][0], kAct, 8, warp * 32, 2, std::integral_constant<int, 1>{});
        __syncthreads();
        if (tid < 8 * 8) {
            const int u = tid / 8, slot = tid % 8;
            const int row = cta + G * slot;
            unsigned long long key = 0ull;
            if (u < U && !sm.done[u] && slot < jrows && row < kJointRows) {
                const float total = sum_parts(u, slot, kXWarps) + sm.joint_bias[slot];
                if (row >= kTokenOutputs) {
                    xch_store(xd + (static_cast<size_t>(round & 1) * U + u) * 8 + (row - kTokenOutputs), total, round + 1);
                } else if (total == total) {          // NaN never wins
                    float sc = total;
                    if (sc == 0.0f) sc = 0.0f;
                    const unsigned bits = __float_as_uint(sc);
                    const unsigned ordered = (bits & 0x80000000u) ? ~bits : (bits ^ 0x80000000u);
                    key = (static_cast<unsigned long long>(ordered) << 32) |
                          (static_cast<unsigned long long>(2047 - row) << 21) | epoch;
                }
            }
            sm.rowkey[u][slot] = key;
        }
        __syncthreads();
        PK_STAMP(6);
        if (tid < U && !sm.done[tid]) {
            unsigned long long best = 0ull;
#pragma unroll
            for (int w = 0; w < 8; ++w) best = sm.rowkey[tid][w] > best ? sm.rowkey[tid][w] : best;
            // a CTA whose rows all produced NaN still publishes a (losing) key for this round
            if (best == 0ull) best = (static_cast<unsigned long long>(2047 - kTokenOutputs) << 21) | epoch;
            asm volatile("st.relaxed.gpu.global.u64 [%0], %1;"
                         ::"l"(xk + (static_cast<size_t>(round & 1) * U + tid) * kXMaxGrid + cta), "l"(best) : "memory");
        }

        // ---- decision: warp u reduces the keys of all CTAs for utterance u (loads in flight
        // together, shuffle reduction) and fetches the five duration logits
        if (warp < U && !sm.done[warp]) {
            const int u = warp;
            const unsigned long long* row = xk + (static_cast<size_t>(round & 1) * U + u) * kXMaxGrid;
            unsigned long long v[8];
            bool good = true;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = lane + 32 * j;
                v[j] = c < G ? xch_load(row + c) : 0ull;
            }
            unsigned long long dv = 0ull;
            const unsigned long long* dslot = xd + (static_cast<size_t>(round & 1) * U + u) * 8 + lane;
            if (lane < kDurations) dv = xch_load(dslot);
            unsigned long long best = 0ull;
            {
                unsigned pending = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (lane + 32 * j < G) pending |= 1u << j;
                bool dur_pending = lane < kDurations;
                long long start = 0;
                unsigned polls = 0;
                while (true) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (((pending >> j) & 1u) && (static_cast<unsigned>(v[j]) & kEpochMask) == epoch) {
                            pending &= ~(1u << j);
                            best = v[j] > best ? v[j] : best;
                        }
                    if (dur_pending && static_cast<unsigned>(dv >> 32) == round + 1) dur_pending = false;
                    if (pending == 0u && !dur_pending) break;
                    if (polls == 0u) start = clock64();
                    if ((++polls & 63u) == 0u && (*abort_flag != 0 || clock64() - start > 2000000000ll)) {
                        *abort_flag = 1;
                        good = false;
                        break;
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if ((pending >> j) & 1u) v[j] = xch_load(row + lane + 32 * j);
                    if (dur_pending) dv = xch_load(dslot);
                }
            }
#pragma unroll
            for (int off = 16; off > 0; off /= 2) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, off);
                best = other > best ? other : best;
            }
            if (!__all_sync(0xffffffffu, good)) sm.ok = 0;
            int token = 2047 - static_cast<int>((best >> 21) & 0x7FFull);
            // every token score of the round was NaN (only losing keys were published): a blank,
            // reported as status bit 4; 1025 is no row of the embedding table
            if (token > kBlank) {
                token = kBlank;
                if (cta == 0 && lane == 0 && good && p.status != nullptr) atomicOr(p.status, 4);
            }
            // first strict maximum of the five duration logits (lanes 0..4 hold one each)
            const float my_dur = __uint_as_float(static_cast<unsigned>(dv));
            int duration = 0;
            float best_dur = __shfl_sync(0xffffffffu, my_dur, 0);
#pragma unroll
            for (int i = 1; i < kDurations; ++i) {
                const float v = __shfl_sync(0xffffffffu, my_dur, i);
                if (v > best_dur) { best_dur = v; duration = i; }
            }
            // the token's embedding row is the next LSTM input: fetch it now (fp16 exactly)
            if (token != kBlank) {
                const __half* emb = p.embedding + static_cast<size_t>(token) * kHidden;
                for (int c = lane * 8; c < kHidden; c += 256) {
                    *reinterpret_cast<uint4*>(&sm.ax[u][c]) = __ldg(reinterpret_cast<const uint4*>(emb + c));
                    *reinterpret_cast<uint4*>(&sm.ax[u + 8][c]) = make_uint4(0, 0, 0, 0);
                }
            }
            if (lane == 0) {
                if (sm.need[u]) { sm.ver[u] += 1; sm.valid[u] = 1; }   // this round's prediction is now current
                if (token != kBlank) {
                    if (cta == 0 && sm.count[u] < p.max_tokens) {
                        p.tokens[static_cast<size_t>(u) * p.max_tokens + sm.count[u]] = token;
                        if (p.durations_out != nullptr)
                            p.durations_out[static_cast<size_t>(u) * p.max_tokens + sm.count[u]] = duration;
                    }
                    sm.count[u] += 1;
                    sm.last[u] = token;
                    sm.emitted[u] = 1;
                    sm.valid[u] = 0;
                }
                int frame = sm.frame[u] + duration;
                int symbols = sm.symbols[u] + 1;
                if (duration != 0 || symbols == kMaxSymbols) {
                    if (duration == 0) frame += 1;
                    symbols = 0;
                }
                sm.frame[u] = frame;
                sm.symbols[u] = symbols;
                const bool done = frame >= sm.total_frames[u];
                sm.done[u] = done;
                sm.need[u] = !done && !sm.valid[u];
            }
        }
        __syncthreads();
        PK_STAMP(8);
        round += 1;
    }
    __syncthreads();
#ifdef PK100_DEC_PROFILE
    if (cta == 0 && tid == 0)
        for (int i = 0; i < 10; ++i) reinterpret_cast<volatile long long*>(p.workspace + lay.abort)[2 + i] = prof[i];
#endif
    if (cta == 0 && tid < U) p.counts[tid] = min(sm.count[tid], p.max_tokens);
    // number of lockstep rounds of this decode, for diagnostics (second word of the flag area)
    if (cta == 0 && tid == 0) reinterpret_cast<volatile int*>(p.workspace + lay.abort)[2] = static_cast<int>(round);
    if (sm.ok == 0 && tid == 0 && p.status != nullptr) atomicExch(p.status, 2);
}


// ---------------------------------------------------------------------------
// Cluster decoder.
//
// One thread-block cluster of 16 CTAs decodes the batch.  The phases of a round hand their
// vectors to the peers through distributed shared memory: every CTA pushes its slice into all
// 16 CTAs with st.async, which also credits the bytes to an mbarrier of the receiving CTA, and
// each CTA waits (bounded) on its own mbarrier only.  An exchange costs one SM-to-SM hop
// instead of the 2-3 us of global-memory slots polled by 148 CTAs.  The price: 16 CTAs
// cannot hold the 8 MB of fp16 weights in shared memory, so
//   - the joint rows (needed every round) stay resident,
//   - the recurrent LSTM weights of layer 0 sit in tensor memory (unused otherwise: the MMAs
//     here are mma.sync), written once per call and read back per k-step pair,
//   - the prediction projection (and a second LSTM layer) is streamed from L2 on the rounds
//     that follow a non-blank token, from a copy in "fragment order": the 16 bytes a lane
//     needs for two k-steps of mma.m16n8k16 are contiguous, so a warp pulls 512 contiguous
//     bytes per load straight into registers, several loads deep,
//   - the input half of the LSTM, W_ih . embedding[token], is a table [1025, 2560] computed
//     once per call by one GEMM; a round gathers 4 x 40 floats of the token's row per CTA.
// Every CTA runs the same control flow on replicated utterance state.
constexpr int kCl = 16;                          // CTAs per cluster
constexpr int kClUnits = kHidden / kCl;          // 40 hidden units / prediction rows per CTA
constexpr int kClJoint = 65;                     // joint rows per CTA (16 x 65 >= 1030)
constexpr int kClThreads = 640;
constexpr int kClWarps = kClThreads / 32;
constexpr int kPartFloats = 6400;                // K-split partial sums of any of the three GEMMs

// A [rows x K] weight slice split over the 20 warps as KG k-groups x NG row-groups; a warp
// walks KP pairs of k-steps (32 columns each) over up to NT row tiles of 8 (TILES in total).
template <int KG_, int NG_, int KP_, int NT_, int TILES_>
struct FragShape {
    static constexpr int KG = KG_, NG = NG_, KP = KP_, NT = NT_, kTiles = TILES_;
    static constexpr int kRows = kTiles * 8;
    // row pitch of the partial sums: = 8 (mod 32) floats, so the 8-byte stores of a half-warp
    // (4 utterances x 4 column pairs) fall into 16 different bank pairs
    static constexpr int kPitch = kRows + ((8 - kRows % 32) + 32) % 32;
    static constexpr int kCols = KG * KP * 32;
    static constexpr int kPerCta = KG * KP * kTiles * 32;   // uint4 per CTA
    static_assert(KG * NG == kClWarps, "one (k-group, row-group) per warp");
    static_assert(NG * NT >= kTiles && (NG - 1) * NT < kTiles, "row groups cover the tiles");
    static_assert(KG * 8 * kPitch <= kPartFloats, "partials fit");
    static_assert(kCols % kHidden == 0, "K = 640, or 1280 for [input | recurrent]");
};
using LstmShape = FragShape<4, 5, 5, 4, 20>;   // 160 gate rows x 640 (recurrent weights)
using PredShape = FragShape<20, 1, 1, 5, 5>;   // 40 rows x 640
using JointShape = FragShape<10, 2, 2, 5, 9>;  // 72 rows (65 used) x 640
using Lstm1Shape = FragShape<4, 5, 10, 4, 20>; // second LSTM layer: 160 gate rows x 1280 ([h of layer 0 | own h])
// Measured alternatives that were not kept: four k-groups for the prediction and joint GEMMs (fewer
// partial sums to add, but longer dependent MMA chains: 8.7 instead of 8.0 us per round), and layer 0's
// recurrent GEMM moved into the wait for the keys (it overlaps little: the keys arrive within a few
// hundred cycles, and the token's table row is then waited for at the top of the next round).

struct ClLayout { size_t base, lstm, pred, joint, xtab, lstm1, cache, total; };
__host__ __device__ inline ClLayout cl_layout(int utts) {
    ClLayout l;
    const size_t a = dec_layout(utts).total, b = xch_layout(utts).total;
    l.base = ((a > b ? a : b) + 255) / 256 * 256;
    size_t off = l.base;
    l.lstm = off; off += static_cast<size_t>(kCl) * LstmShape::kPerCta * 16;
    l.pred = off; off += static_cast<size_t>(kCl) * PredShape::kPerCta * 16;
    l.joint = off; off += static_cast<size_t>(kCl) * JointShape::kPerCta * 16;
    l.xtab = off; off += static_cast<size_t>(kTokenOutputs) * kGates * 4;
    l.lstm1 = off; off += static_cast<size_t>(kCl) * Lstm1Shape::kPerCta * 16;
    l.cache = off; off += 256;        // max |w| of the three tensors of the INT8 cache
    l.total = off;
    return l;
}

enum : int { CLPACK_LSTM = 0, CLPACK_PRED = 1, CLPACK_JOINT = 2, CLPACK_LSTM_IH_HH = 3 };

// dst[cta][kg][kp][tile][lane] = the B fragments (b0, b1) of k-steps 2*kp and 2*kp+1 of row tile
// `tile`: lane (g = lane / 4, t = lane % 4) holds W[row g][k0 + 2t, +1, +8, +9] per k-step.
// With `absmax` (long-request numerics) the values stored are the INT8 codes of the tensor,
// scale index `scale_first` for w and `scale_second` for w_second.
template <typename Shape, int Mode>
__global__ void tdt_pack_kernel(uint4* dst, const __half* w, const __half* w_second, const float* absmax,
                                int scale_first, int scale_second) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= kCl * Shape::kPerCta) return;
    int rest = idx;
    const int lane = rest % 32; rest /= 32;
    const int tile = rest % Shape::kTiles; rest /= Shape::kTiles;
    const int kp = rest % Shape::KP; rest /= Shape::KP;
    const int kg = rest % Shape::KG; rest /= Shape::KG;
    const int r = rest;
    const int g = lane / 4, t = lane % 4;
    const int n = tile * 8 + g;
    const int k0 = (kg * Shape::KP + kp) * 32;
    int row = -1;
    if (Mode == CLPACK_LSTM || Mode == CLPACK_LSTM_IH_HH) row = (n % 4) * kHidden + r * kClUnits + n / 4;   // gate-major rows
    else if (Mode == CLPACK_PRED) row = r * kClUnits + n;
    else if (n < kClJoint && r * kClJoint + n < kJointRows) row = r * kClJoint + n;
    auto pair = [&](int k) -> unsigned {
        if (row < 0) return 0u;
        // CLPACK_LSTM_IH_HH: columns 0..639 from w (input weights), 640..1279 from w_second (recurrent)
        const bool second = Mode == CLPACK_LSTM_IH_HH && k >= kHidden;
        const __half* src = second ? w_second + static_cast<size_t>(row) * kHidden + (k - kHidden)
                                   : w + static_cast<size_t>(row) * kHidden + k;
        __half v0 = src[0], v1 = src[1];
        if (absmax != nullptr) {
            const float scale = cache_scale(absmax, second ? scale_second : scale_first);
            v0 = cache_code(v0, scale);
            v1 = cache_code(v1, scale);
        }
        return static_cast<unsigned>(__half_as_ushort(v0)) | (static_cast<unsigned>(__half_as_ushort(v1)) << 16);
    };
    dst[idx] = make_uint4(pair(k0 + 2 * t), pair(k0 + 2 * t + 8), pair(k0 + 16 + 2 * t), pair(k0 + 16 + 2 * t + 8));
}

constexpr int kEncChunks = kHidden / 8;          // 16-byte chunks of one projected encoder row

// Two LSTM layers: second committed state, its receive buffer, cell state, bias, barrier.
template <int Layers> struct CSecondLayer {};
template <> struct CSecondLayer<2> {
    __half ah1[16][kAct];
    __half hx1[16][kAct];
    float cstate1[kMaxUtt][kClUnits];
    float lstm_bias1[kClUnits][4];
    uint64_t hbar1;
};

// With one layer the joint rows stay resident; with two they are streamed like the other
// weights (the second layer's state needs the room).
template <int Layers>
struct CSmemT {
    uint4 wj[Layers == 1 ? JointShape::kPerCta : 1];   // this CTA's joint rows in fragment order (resident)
    __half ax[16][kAct];                  // joint input (hi rows 0-7, lo rows 8-15)
    __half ah[16][kAct];                  // committed hidden state, all 640 units
    __half hx[16][kAct];                  // fresh hidden state, written by all CTAs of the cluster
    float pred[kMaxUtt][kHidden];         // prediction vectors, written by all CTAs of the cluster
    float part[kPartFloats];              // [k-group][utterance][row] partial sums
    __half enc[kMaxUtt][kHidden];         // projected encoder row of each utterance's current frame
    float xg[kMaxUtt][kClUnits * 4];      // W_ih . embedding[last token] for this CTA's gate rows
    float cstate[kMaxUtt][kClUnits];
    alignas(16) __half stage_h[16][kClUnits];     // this CTA's slice of h (hi / lo) on its way out
    alignas(16) __half stage_q[kMaxUtt][kClUnits];  // long-request numerics: its INT8 codes rne(h * 127)
    float cache_mul[3];                           // scale / 127 of w_hh[0], w_hh[1], w_ih[1]
    uint32_t tmem_base;                           // tensor memory holding layer 0's recurrent weights
    alignas(16) float stage_p[kMaxUtt][kClUnits]; // this CTA's slice of the prediction vector
    float lstm_bias[kClUnits][4];
    float pred_bias[kClUnits];
    float joint_bias[JointShape::kRows];
    unsigned long long keys[2][kCl][kMaxUtt];   // [round parity][source CTA][utterance], written by peers
    float dur[2][kMaxUtt][8];                   // [round parity][utterance][duration], written by the owner
    uint64_t hbar, pbar, kbar[2];               // exchange mbarriers (count 1 + transaction bytes)
    int frame[kMaxUtt], symbols[kMaxUtt], count[kMaxUtt], total_frames[kMaxUtt];
    alignas(8) unsigned char valid[kMaxUtt];
    alignas(8) unsigned char done[kMaxUtt];      // read as one 64-bit word: entries >= utts are 1
    alignas(8) unsigned char need[kMaxUtt];      // !done && !valid
    int abort;
    CSecondLayer<Layers> second;
#ifdef PK100_DEC_PROFILE
    long long prof[16], last_stamp;       // per-phase cycle totals of thread 0
#endif
};
using CSmem = CSmemT<1>;
static_assert(sizeof(CSmemT<2>) <= 227 * 1024 && sizeof(CSmem) <= 227 * 1024, "cluster decoder state fits one CTA's shared memory");

// Remote store that credits its bytes to an mbarrier of the destination CTA.  `addr` and `bar`
// are shared::cluster addresses of the same CTA.
__device__ __forceinline__ void st_async_v4(uint32_t addr, uint4 v, uint32_t bar) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "r"(bar) : "memory");
}
__device__ __forceinline__ void st_async_b64(uint32_t addr, unsigned long long v, uint32_t bar) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.b64 [%0], %1, [%2];"
                 ::"r"(addr), "l"(v), "r"(bar) : "memory");
}
__device__ __forceinline__ void st_async_b32(uint32_t addr, unsigned v, uint32_t bar) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                 ::"r"(addr), "r"(v), "r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float fast_tanh(float x) { return 2.0f * fast_sigmoid(2.0f * x) - 1.0f; }

// part[kg][u][row] = A(16 x 640, hi / lo rows) . W^T for this warp's k-group and row group.
// The weight fragments run through a register ring `Depth` k-step pairs ahead of the MMAs;
// frag_prefetch issues the loads of the first `Stages` pairs (weights do not depend on the
// activations, so this can be done before the activations have arrived), frag_compute the rest.
template <typename Shape, int Depth>
struct FragRing { uint4 buf[Depth + 1][Shape::NT]; };

template <typename Shape, bool Global>
__device__ __forceinline__ uint4 frag_fetch(const uint4* w, int warp, int lane, int kp, int j) {
    const int kg = warp / Shape::NG, ng = warp % Shape::NG;
    const uint4* ptr = w + static_cast<size_t>(kg * Shape::KP + kp) * Shape::kTiles * 32 + (ng * Shape::NT + j) * 32 + lane;
    return Global ? __ldg(ptr) : *ptr;
}
template <typename Shape>
__device__ __forceinline__ bool frag_live(int warp, int j) {
    return Shape::NG * Shape::NT == Shape::kTiles || (warp % Shape::NG) * Shape::NT + j < Shape::kTiles;
}

template <typename Shape, bool Global, int Depth, int First, int Stages>
__device__ __forceinline__ void frag_prefetch(const uint4* w, FragRing<Shape, Depth>& ring, int warp, int lane) {
#pragma unroll
    for (int s = First; s < First + Stages && s < Shape::KP && s < Depth; ++s)
#pragma unroll
        for (int j = 0; j < Shape::NT; ++j)
            if (frag_live<Shape>(warp, j)) ring.buf[s][j] = frag_fetch<Shape, Global>(w, warp, lane, s, j);
}

// `Loaded` = prologue stages already issued by frag_prefetch.  `HiOnly`: A has 8 rows (one per
// utterance, no low-order rows), as for the integer codes of the long-request numerics.
template <typename Shape, bool Global, int Depth, int Loaded, bool HiOnly = false>
__device__ __forceinline__ void frag_compute(const uint4* w, const __half* a, float* part,
                                             FragRing<Shape, Depth>& ring, int warp, int lane) {
    constexpr int KP = Shape::KP, NT = Shape::NT;
    const int kg = warp / Shape::NG, ng = warp % Shape::NG;
    const int g = lane / 4, t = lane % 4;
    frag_prefetch<Shape, Global, Depth, Loaded, Depth - Loaded>(w, ring, warp, lane);
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.0f;
    const __half* arow = HiOnly ? a + (lane % 8) * kAct + ((lane / 8) % 2) * 8 + kg * KP * 32
                                : a + (lane % 16) * kAct + (lane / 16) * 8 + kg * KP * 32;
#pragma unroll
    for (int kp = 0; kp < KP; ++kp) {
        if (kp + Depth < KP) {
#pragma unroll
            for (int j = 0; j < NT; ++j)
                if (frag_live<Shape>(warp, j))
                    ring.buf[(kp + Depth) % (Depth + 1)][j] = frag_fetch<Shape, Global>(w, warp, lane, kp + Depth, j);
        }
        unsigned a0[4], a1[4];
        if constexpr (HiOnly) {
            unsigned lo[2], hi[2];       // rows 0-7: columns k .. k+7 and k+8 .. k+15
            dec_ldmatrix_x2(lo, arow + kp * 32);
            dec_ldmatrix_x2(hi, arow + kp * 32 + 16);
            a0[0] = lo[0]; a0[1] = 0u; a0[2] = lo[1]; a0[3] = 0u;
            a1[0] = hi[0]; a1[1] = 0u; a1[2] = hi[1]; a1[3] = 0u;
        } else {
            dec_ldmatrix_x4(a0, arow + kp * 32);
            dec_ldmatrix_x4(a1, arow + kp * 32 + 16);
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            if (!frag_live<Shape>(warp, j)) continue;
            const uint4 b = ring.buf[kp % (Depth + 1)][j];
            dec_mma(acc[j], a0, b.x, b.y);
            dec_mma(acc[j], a1, b.z, b.w);
        }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        if (!frag_live<Shape>(warp, j)) continue;
        float* dst = part + (kg * 8 + g) * Shape::kPitch + (ng * NT + j) * 8 + 2 * t;
        // hi row + lo row of utterance g
        *reinterpret_cast<float2*>(dst) = HiOnly ? make_float2(acc[j][0], acc[j][1])
                                                 : make_float2(acc[j][0] + acc[j][2], acc[j][1] + acc[j][3]);
    }
}

// Layer 0's recurrent weights live in TENSOR MEMORY for the whole call: the 205 KB slice of a CTA
// (160 gate rows x 640, fragment order) does not fit beside the joint rows in shared memory, but
// the 256 KB of TMEM are otherwise unused by this kernel (its MMAs are register-operand
// mma.sync).  A warp can reach the 32 lanes of its quadrant (warp % 4); the five warps of a quadrant
// take 80 columns each: lane L, columns 16 * kp + 4 * j .. + 3 = the uint4 that lane L feeds to the
// MMAs of k-step pair kp and row tile j.  One tcgen05.ld.32x32b.x16 per k-step pair replaces four
// 512-byte loads from L2, which bounded this GEMM at the SM's L2 port (about 70 bytes per cycle).
constexpr uint32_t kTmemColumns = 512;
static_assert(LstmShape::NT == 4 && LstmShape::NG * LstmShape::NT == LstmShape::kTiles, "16 columns per k-step pair");
static_assert((kClWarps / 4) * LstmShape::KP * 16 <= kTmemColumns && kClWarps % 4 == 0, "recurrent slice fits TMEM");

__device__ __forceinline__ uint32_t lstm_tmem_addr(uint32_t base, int warp) {
    return base + (static_cast<uint32_t>((warp % 4) * 32) << 16) + static_cast<uint32_t>((warp / 4) * LstmShape::KP * 16);
}

// set-up: this warp's fragments, global (fragment-ordered copy) -> TMEM
__device__ __forceinline__ void lstm_tmem_fill(const uint4* w, uint32_t taddr, int warp, int lane) {
#pragma unroll
    for (int kp = 0; kp < LstmShape::KP; ++kp) {
        uint32_t r[16];
#pragma unroll
        for (int j = 0; j < LstmShape::NT; ++j) {
            const uint4 v = frag_fetch<LstmShape, true>(w, warp, lane, kp, j);
            r[4 * j] = v.x; r[4 * j + 1] = v.y; r[4 * j + 2] = v.z; r[4 * j + 3] = v.w;
        }
        tmem_st_32x16(taddr + kp * 16, r);
    }
    tmem_st_wait();
}

// part[kg][u][row] = A . W_hh^T with the weights read from TMEM; the load of k-step pair kp + 1 is
// in flight while the MMAs of pair kp issue
template <bool HiOnly>
__device__ __forceinline__ void lstm_compute_tmem(uint32_t taddr, const __half* a, float* part, int warp, int lane) {
    using Shape = LstmShape;
    constexpr int KP = Shape::KP, NT = Shape::NT;
    const int kg = warp / Shape::NG, ng = warp % Shape::NG;
    const int g = lane / 4, t = lane % 4;
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.0f;
    const __half* arow = HiOnly ? a + (lane % 8) * kAct + ((lane / 8) % 2) * 8 + kg * KP * 32
                                : a + (lane % 16) * kAct + (lane / 16) * 8 + kg * KP * 32;
    uint32_t wbuf[2][16];
    tmem_ld_32x16(taddr, wbuf[0]);
    tmem_ld_wait();
#pragma unroll
    for (int kp = 0; kp < KP; ++kp) {
        if (kp + 1 < KP) tmem_ld_32x16(taddr + (kp + 1) * 16, wbuf[(kp + 1) % 2]);
        unsigned a0[4], a1[4];
        if constexpr (HiOnly) {
            unsigned lo[2], hi[2];
            dec_ldmatrix_x2(lo, arow + kp * 32);
            dec_ldmatrix_x2(hi, arow + kp * 32 + 16);
            a0[0] = lo[0]; a0[1] = 0u; a0[2] = lo[1]; a0[3] = 0u;
            a1[0] = hi[0]; a1[1] = 0u; a1[2] = hi[1]; a1[3] = 0u;
        } else {
            dec_ldmatrix_x4(a0, arow + kp * 32);
            dec_ldmatrix_x4(a1, arow + kp * 32 + 16);
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const uint32_t* b = &wbuf[kp % 2][4 * j];
            dec_mma(acc[j], a0, b[0], b[1]);
            dec_mma(acc[j], a1, b[2], b[3]);
        }
        if (kp + 1 < KP) tmem_ld_wait();
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        float* dst = part + (kg * 8 + g) * Shape::kPitch + (ng * NT + j) * 8 + 2 * t;
        *reinterpret_cast<float2*>(dst) = HiOnly ? make_float2(acc[j][0], acc[j][1])
                                                 : make_float2(acc[j][0] + acc[j][2], acc[j][1] + acc[j][3]);
    }
}

#ifdef PK100_DEC_PROFILE
#define CL_STAMP(i) do { if (tid == 0) { const long long now__ = clock64(); sm.prof[i] += now__ - sm.last_stamp; sm.last_stamp = now__; } } while (0)
#else
#define CL_STAMP(i) do { } while (0)
#endif

// `Cache` = long-request numerics: recurrent weights (and layer 1's input weights) arrive as INT8
// codes in the packed copies, `xtab` is rounded to fp16, and every hidden state also travels as
// codes: rows 0-7 of ah / ah1 hold the committed codes (the A operand of the recurrent GEMMs),
// rows 8-15 receive the fresh codes from the cluster.
template <int Layers, bool Cache>
__global__ void __launch_bounds__(kClThreads, 1)
tdt_cluster_kernel(const DecParams p, const uint4* packed_lstm, const uint4* packed_pred,
                   const uint4* packed_joint, const float* xtab, const uint4* packed_lstm1) {
    extern __shared__ __align__(16) uint8_t cs_raw[];
    CSmemT<Layers>& sm = *reinterpret_cast<CSmemT<Layers>*>(cs_raw);
#ifdef PK100_DEC_PROFILE
    if (threadIdx.x == 0) {
        for (int i = 0; i < 16; ++i) sm.prof[i] = 0;
        sm.last_stamp = clock64();
    }
#endif
    const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
    const int r = static_cast<int>(cluster_ctarank());
    const int U = p.utts;
    volatile int* abort_flag = &sm.abort;

    // ---- set-up: resident joint slice, biases, cleared state, first encoder rows
    const uint4* wjoint = packed_joint + static_cast<size_t>(r) * JointShape::kPerCta;
    if constexpr (Layers == 1) {
        // (the long-request numerics read the joint rows from the caller's matrix instead)
        if constexpr (!Cache)
            for (int i = tid; i < JointShape::kPerCta; i += kClThreads) sm.wj[i] = __ldg(wjoint + i);
    } else {
        for (int i = tid; i < 16 * kAct; i += kClThreads) {
            (&sm.second.ah1[0][0])[i] = __float2half(0.0f);
            (&sm.second.hx1[0][0])[i] = __float2half(0.0f);
        }
        for (int i = tid; i < kMaxUtt * kClUnits; i += kClThreads) (&sm.second.cstate1[0][0])[i] = 0.0f;
        if (tid < kClUnits * 4) {
            const int slot = tid / 4, gt = tid % 4;
            const int row = gt * kHidden + r * kClUnits + slot;
            sm.second.lstm_bias1[slot][gt] = p.b_ih[1][row] + p.b_hh[1][row];
        }
        if (tid == 0) mbar_init(&sm.second.hbar1, 1);
    }
    for (int i = tid; i < 16 * kAct; i += kClThreads) {
        (&sm.ax[0][0])[i] = __float2half(0.0f);
        (&sm.ah[0][0])[i] = __float2half(0.0f);
        (&sm.hx[0][0])[i] = __float2half(0.0f);
    }
    for (int i = tid; i < kMaxUtt * kHidden; i += kClThreads) {
        (&sm.pred[0][0])[i] = 0.0f;
        (&sm.enc[0][0])[i] = __float2half(0.0f);
    }
    for (int i = tid; i < kMaxUtt * kClUnits * 4; i += kClThreads) (&sm.xg[0][0])[i] = 0.0f;   // no token yet: zero input
    for (int i = tid; i < kMaxUtt * kClUnits; i += kClThreads) (&sm.cstate[0][0])[i] = 0.0f;
    if (tid < kClUnits * 4) {
        const int slot = tid / 4, gt = tid % 4;
        const int row = gt * kHidden + r * kClUnits + slot;
        sm.lstm_bias[slot][gt] = p.b_ih[0][row] + p.b_hh[0][row];
    }
    if (tid < kClUnits) sm.pred_bias[tid] = p.b_pred[r * kClUnits + tid];
    if (tid < 3) sm.cache_mul[tid] = (Cache && (tid == 0 || Layers == 2)) ? cache_mul(cache_scale(p.cache_absmax, tid)) : 0.0f;
    if (tid < JointShape::kRows) {
        const int row = r * kClJoint + tid;
        sm.joint_bias[tid] = (tid < kClJoint && row < kJointRows) ? p.b_joint[row] : 0.0f;
    }
    if (tid < kMaxUtt) {
        sm.frame[tid] = 0; sm.symbols[tid] = 0; sm.count[tid] = 0; sm.valid[tid] = 0;
        sm.total_frames[tid] = tid < U ? min(p.frames[tid], p.seg_stride) : 0;   // never past the utterance's block
        const bool done = tid >= U || p.frames[tid] <= 0 || !in_window(p, tid);
        sm.done[tid] = done;
        sm.need[tid] = !done;
    }
    for (int i = tid; i < 2 * kCl * kMaxUtt; i += kClThreads) (&sm.keys[0][0][0])[i] = 0ull;
    for (int i = tid; i < 2 * kMaxUtt * 8; i += kClThreads) (&sm.dur[0][0][0])[i] = 0.0f;
    if (tid == 0) {
        mbar_init(&sm.hbar, 1);
        mbar_init(&sm.pbar, 1);
        mbar_init(&sm.kbar[0], 1);
        mbar_init(&sm.kbar[1], 1);
        sm.abort = 0;
        fence_barrier_init();
    }
    if (warp == 1) {                 // one warp owns the tensor-memory allocation (all of it; one CTA per SM)
        tmem_alloc(&sm.tmem_base, kTmemColumns);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp < U && !sm.done[warp]) {
        const __half* src = p.enc_proj + static_cast<size_t>(warp) * p.seg_stride * kHidden;
        for (int c = lane; c < kEncChunks; c += 32) cp_async_16(&sm.enc[warp][c * 8], src + c * 8);
    }
    __syncthreads();
    cluster_sync_all();      // every CTA's shared memory and mbarriers are ready before a peer writes

    const uint4* wl = packed_lstm + static_cast<size_t>(r) * LstmShape::kPerCta;
    const uint4* wp = packed_pred + static_cast<size_t>(r) * PredShape::kPerCta;
    // sender role of this thread: peer CTA and two of the 80 16-byte items of a slice
    const uint32_t peer = static_cast<uint32_t>(tid / kClUnits);
    const int item0 = tid % kClUnits;
    uint32_t hphase = 0, pphase = 0, kphase[2] = {0, 0};
    [[maybe_unused]] uint32_t h1phase = 0;
    [[maybe_unused]] const uint4* wl1 = packed_lstm1 + static_cast<size_t>(r) * Lstm1Shape::kPerCta;
    // layer 0's recurrent weights: once from the fragment-ordered copy into tensor memory
    const uint32_t lstm_taddr = lstm_tmem_addr(sm.tmem_base, warp);
    lstm_tmem_fill(wl, lstm_taddr, warp, lane);

    // LSTM cell of one (utterance, unit) from its four gate sums; stages h for the exchange
    auto cell_update = [&](const float (&gsum)[4], float& cstate, int u, int slot) {
        float h;
        if constexpr (Cache) {
            // the reference's approximations: h is rounded to 8 bits next, and a code that flips moves a gate
            h = ref_lstm_cell(gsum, cstate);
            sm.stage_q[u][slot] = __int2half_rn(quantize_i8(h * 127.0f));
            // the prediction projection of this mode reads the fp32 state (decoder.cu:672-681), so the
            // slice travels as fp32: stage_h viewed as float[8][40], the same bytes as a hi / lo pair
            reinterpret_cast<float*>(&sm.stage_h[0][0])[u * kClUnits + slot] = h;
        } else {
            const float cell = fast_sigmoid(gsum[1]) * cstate + fast_sigmoid(gsum[0]) * fast_tanh(gsum[2]);
            cstate = cell;
            h = fast_sigmoid(gsum[3]) * fast_tanh(cell);
            const __half hi = __float2half_rn(h);
            sm.stage_h[u][slot] = hi;
            sm.stage_h[u + 8][slot] = __float2half_rn(h - __half2float(hi));
        }
    };
    // this CTA's staged slice of a hidden state -> `fresh` (hi / lo rows) of every CTA, and with
    // Cache its codes -> rows 8-15 of `committed`; all bytes are credited to `bar_local` there
    auto send_hidden = [&](__half (*fresh)[kAct], __half (*committed)[kAct], uint64_t* bar_local) {
        const uint32_t bar = map_to_cta(smem_u32(bar_local), peer);
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int item = item0 + it * kClUnits;
            if constexpr (Cache) {
                // 0..79: 8 utterances x 10 chunks of 4 floats into `fresh` viewed as float[8][640]
                const int u = item / 10, chunk = item % 10;
                if (u < U && sm.need[u]) {
                    const uint4 v = *reinterpret_cast<const uint4*>(
                        reinterpret_cast<const float*>(&sm.stage_h[0][0]) + u * kClUnits + chunk * 4);
                    float* dst = reinterpret_cast<float*>(&fresh[0][0]) + u * kHidden + r * kClUnits + chunk * 4;
                    st_async_v4(map_to_cta(smem_u32(dst), peer), v, bar);
                }
            } else {
                // 0..79: 16 rows x 5 chunks of 8 units
                const int row = item / 5, chunk = item % 5;
                const int u = row % 8;
                if (u < U && sm.need[u]) {
                    const uint4 v = *reinterpret_cast<const uint4*>(&sm.stage_h[row][chunk * 8]);
                    st_async_v4(map_to_cta(smem_u32(&fresh[row][r * kClUnits + chunk * 8]), peer), v, bar);
                }
            }
        }
        if constexpr (Cache) {
            const int u = item0 / 5, chunk = item0 % 5;
            if (u < U && sm.need[u]) {
                const uint4 v = *reinterpret_cast<const uint4*>(&sm.stage_q[u][chunk * 8]);
                st_async_v4(map_to_cta(smem_u32(&committed[8 + u][r * kClUnits + chunk * 8]), peer), v, bar);
            }
        }
    };
    // bytes one stepping utterance contributes to a hidden-state exchange
    constexpr uint32_t kHiddenTx = 2 * kHidden * 2 + (Cache ? kHidden * 2 : 0);
    // the threads from `first` on make the fresh state the committed one
    auto commit_hidden = [&](const __half (*fresh)[kAct], __half (*committed)[kAct], int first) {
        constexpr int kRows = Cache ? 8 : 16;
        for (int i = tid - first; i < kRows * kEncChunks; i += kClThreads - first) {
            const int row = i / kEncChunks, c = i % kEncChunks;
            const int u = row % 8;
            if (u < U && sm.need[u]) {
                const __half* src = Cache ? &committed[8 + row][c * 8] : &fresh[row][c * 8];
                *reinterpret_cast<uint4*>(&committed[row][c * 8]) = *reinterpret_cast<const uint4*>(src);
            }
        }
    };

    unsigned round = 0;
    while (true) {
        const unsigned long long done8 = *reinterpret_cast<const unsigned long long*>(sm.done);
        const unsigned long long need8 = *reinterpret_cast<const unsigned long long*>(sm.need);
        // a wait that gave up raised sm.abort; it is read here, after the CTA barrier that ends a
        // round, so every thread of the CTA takes the same branch
        if (done8 == 0x0101010101010101ull || sm.abort != 0) break;
        const int needs = __popcll(need8), lives = 8 - __popcll(done8);
        CL_STAMP(0);

        if (need8 != 0ull) {
            // ---- LSTM: gates of this CTA's 40 units = table row + h . w_hh^T + bias
            lstm_compute_tmem<Cache>(lstm_taddr, &sm.ah[0][0], sm.part, warp, lane);
            cp_async_wait_all();             // table rows / encoder rows requested at the last decision
            __syncthreads();
            CL_STAMP(1);
            if (tid < kMaxUtt * kClUnits) {
                const int slot = tid % kClUnits, u = tid / kClUnits;
                if (u < U && sm.need[u]) {
                    const float4 x = *reinterpret_cast<const float4*>(&sm.xg[u][slot * 4]);
                    float gsum[4];
                    if constexpr (Cache) {
                        // exact integer dot products; order of decoder.cu:636-637: (recurrent + bias) + table
                        float rec[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                        for (int kg = 0; kg < LstmShape::KG; ++kg) {
                            const float4 v = *reinterpret_cast<const float4*>(
                                &sm.part[(kg * 8 + u) * LstmShape::kPitch + slot * 4]);
                            rec[0] += v.x; rec[1] += v.y; rec[2] += v.z; rec[3] += v.w;
                        }
                        const float mul = sm.cache_mul[0];
                        const float xin[4] = {x.x, x.y, x.z, x.w};
                        // the scaled recurrent sum is rounded BEFORE the bias is added, as in the reference
                        // (decoder.cu:113, :626-640: products rounded per lane, then summed): a fused
                        // multiply-add here parts from the reference kernel's tokens after a few hundred steps
#pragma unroll
                        for (int g4 = 0; g4 < 4; ++g4)
                            gsum[g4] = __fadd_rn(__fadd_rn(__fmul_rn(rec[g4], mul), sm.lstm_bias[slot][g4]), xin[g4]);
                    } else {
                        gsum[0] = sm.lstm_bias[slot][0] + x.x; gsum[1] = sm.lstm_bias[slot][1] + x.y;
                        gsum[2] = sm.lstm_bias[slot][2] + x.z; gsum[3] = sm.lstm_bias[slot][3] + x.w;
#pragma unroll
                        for (int kg = 0; kg < LstmShape::KG; ++kg) {
                            const float4 v = *reinterpret_cast<const float4*>(
                                &sm.part[(kg * 8 + u) * LstmShape::kPitch + slot * 4]);
                            gsum[0] += v.x; gsum[1] += v.y; gsum[2] += v.z; gsum[3] += v.w;
                        }
                    }
                    cell_update(gsum, sm.cstate[u][slot], u, slot);
                }
            }
            if (tid == 0) mbar_arrive_expect_tx(&sm.hbar, static_cast<uint32_t>(needs) * kHiddenTx);
            __syncthreads();
            CL_STAMP(2);
            send_hidden(sm.hx, sm.ah, &sm.hbar);     // h slice -> every CTA's hx (and codes)
            // the prediction weights of this warp are requested while the hidden state travels
            [[maybe_unused]] FragRing<PredShape, 1> pred_ring;
            if constexpr (Layers == 1 && !Cache) frag_prefetch<PredShape, true, 1, 0, 1>(wp, pred_ring, warp, lane);
            mbar_wait_bounded(&sm.hbar, hphase, abort_flag);
            hphase ^= 1u;
            CL_STAMP(3);
            const __half (*top_fresh)[kAct] = sm.hx;      // fresh hidden state of the top layer
            __half (*top_committed)[kAct] = sm.ah;
            if constexpr (Layers == 2) {
                // ---- second LSTM layer: gates = [fresh h of layer 0 | own h] . [w_ih | w_hh]^T + bias
                {
                    FragRing<Lstm1Shape, 2> ring1;
                    const int kg = warp / Lstm1Shape::NG;
                    // k-groups 0, 1 read the 640 columns of hx (Cache: the fresh codes of layer 0 in
                    // rows 8-15 of ah), groups 2, 3 those of ah1
                    const __half* a = kg < 2 ? (Cache ? &sm.ah[8][0] : &sm.hx[0][0]) : &sm.second.ah1[0][0] - kHidden;
                    frag_compute<Lstm1Shape, true, 2, 0, Cache>(wl1, a, sm.part, ring1, warp, lane);
                }
                __syncthreads();
                if (tid < kMaxUtt * kClUnits) {
                    const int slot = tid % kClUnits, u = tid / kClUnits;
                    if (u < U && sm.need[u]) {
                        float gsum[4] = {sm.second.lstm_bias1[slot][0], sm.second.lstm_bias1[slot][1],
                                         sm.second.lstm_bias1[slot][2], sm.second.lstm_bias1[slot][3]};
                        if constexpr (Cache) {
                            // k-groups 0, 1: input codes (scale of w_ih[1]); 2, 3: recurrent codes;
                            // decoder.cu:655-663 adds the bias last
                            float in[4] = {0.0f, 0.0f, 0.0f, 0.0f}, rec[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                            for (int kg = 0; kg < Lstm1Shape::KG; ++kg) {
                                const float4 v = *reinterpret_cast<const float4*>(
                                    &sm.part[(kg * 8 + u) * Lstm1Shape::kPitch + slot * 4]);
                                float (&dst)[4] = kg < 2 ? in : rec;
                                dst[0] += v.x; dst[1] += v.y; dst[2] += v.z; dst[3] += v.w;
                            }
#pragma unroll
                            // rounded recurrent product first, the input product fused onto it (decoder.cu:113, :660)
                            for (int g4 = 0; g4 < 4; ++g4)
                                gsum[g4] = __fadd_rn(fmaf(in[g4], sm.cache_mul[2], __fmul_rn(rec[g4], sm.cache_mul[1])), gsum[g4]);
                        } else {
#pragma unroll
                            for (int kg = 0; kg < Lstm1Shape::KG; ++kg) {
                                const float4 v = *reinterpret_cast<const float4*>(
                                    &sm.part[(kg * 8 + u) * Lstm1Shape::kPitch + slot * 4]);
                                gsum[0] += v.x; gsum[1] += v.y; gsum[2] += v.z; gsum[3] += v.w;
                            }
                        }
                        cell_update(gsum, sm.second.cstate1[u][slot], u, slot);
                    }
                } else {
                    // meanwhile: commit the fresh state of layer 0
                    commit_hidden(sm.hx, sm.ah, kMaxUtt * kClUnits);
                }
                if (tid == 0) mbar_arrive_expect_tx(&sm.second.hbar1, static_cast<uint32_t>(needs) * kHiddenTx);
                __syncthreads();
                send_hidden(sm.second.hx1, sm.second.ah1, &sm.second.hbar1);
                if constexpr (!Cache) frag_prefetch<PredShape, true, 1, 0, 1>(wp, pred_ring, warp, lane);
                mbar_wait_bounded(&sm.second.hbar1, h1phase, abort_flag);
                h1phase ^= 1u;
                top_fresh = sm.second.hx1;
                top_committed = sm.second.ah1;
            }
            if constexpr (Cache) {
                // ---- prediction projection in fp32 on the fp32 state, in the reference's summation
                // order (decoder.cu:672-684): lane l takes elements 2l + 64w, w = 0..9, as one fma
                // chain that starts from the bias in lane 0, then the shuffle tree of warp_sum
                const float* hf = reinterpret_cast<const float*>(&top_fresh[0][0]);
#pragma unroll
                for (int it = 0; it < kClUnits / kClWarps; ++it) {
                    const int n = warp + it * kClWarps;
                    const uint32_t* wrow = reinterpret_cast<const uint32_t*>(
                        p.w_pred + static_cast<size_t>(r * kClUnits + n) * kHidden);
                    uint32_t words[10];
#pragma unroll
                    for (int w = 0; w < 10; ++w) words[w] = __ldg(wrow + lane + 32 * w);
                    // the utterances run side by side: eight independent chains, each in its own order
                    float sum[kMaxUtt];
#pragma unroll
                    for (int u = 0; u < kMaxUtt; ++u) sum[u] = lane == 0 ? sm.pred_bias[n] : 0.0f;
#pragma unroll
                    for (int w = 0; w < 10; ++w) {
                        const float2 wv = __half22float2(*reinterpret_cast<const __half2*>(&words[w]));
#pragma unroll
                        for (int u = 0; u < kMaxUtt; ++u) {
                            if (((need8 >> (8 * u)) & 1ull) == 0ull) continue;
                            const float2 hv = *reinterpret_cast<const float2*>(hf + u * kHidden + 2 * lane + 64 * w);
                            sum[u] = fmaf(wv.x, hv.x, sum[u]);
                            sum[u] = fmaf(wv.y, hv.y, sum[u]);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < kMaxUtt; ++u) {
                        if (((need8 >> (8 * u)) & 1ull) == 0ull) continue;
#pragma unroll
                        for (int off = 16; off > 0; off /= 2) sum[u] += __shfl_down_sync(0xffffffffu, sum[u], off);
                        if (lane == 0) sm.stage_p[u][n] = sum[u];
                    }
                }
                CL_STAMP(4);
                commit_hidden(top_fresh, top_committed, 0);
            } else {
            // ---- prediction projection of the new state (A operand: the fresh rows of the top layer)
            frag_compute<PredShape, true, 1, 1>(wp, &top_fresh[0][0], sm.part, pred_ring, warp, lane);
            __syncthreads();
            CL_STAMP(4);
            if (tid < kMaxUtt * kClUnits) {
                const int row = tid % kClUnits, u = tid / kClUnits;
                if (u < U && sm.need[u]) {
                    float v = sm.pred_bias[row];
#pragma unroll
                    for (int kg = 0; kg < PredShape::KG; ++kg) v += sm.part[(kg * 8 + u) * PredShape::kPitch + row];
                    sm.stage_p[u][row] = v;
                }
            } else {
                // meanwhile the other threads commit the fresh hidden state for the next LSTM step
                commit_hidden(top_fresh, top_committed, kMaxUtt * kClUnits);
            }
            }
            if (tid == 0) mbar_arrive_expect_tx(&sm.pbar, static_cast<uint32_t>(needs) * kHidden * 4);
            __syncthreads();
            CL_STAMP(5);
            {   // prediction slice (10 chunks of 4 floats per utterance) -> every CTA's pred
                const uint32_t bar = map_to_cta(smem_u32(&sm.pbar), peer);
#pragma unroll
                for (int it = 0; it < 2; ++it) {
                    const int item = item0 + it * kClUnits;         // 0..79
                    const int u = item / 10, chunk = item % 10;
                    if (u < U && sm.need[u]) {
                        const uint4 v = *reinterpret_cast<const uint4*>(&sm.stage_p[u][chunk * 4]);
                        st_async_v4(map_to_cta(smem_u32(&sm.pred[u][r * kClUnits + chunk * 4]), peer), v, bar);
                    }
                }
            }
            mbar_wait_bounded(&sm.pbar, pphase, abort_flag);
            pphase ^= 1u;
            CL_STAMP(6);
        } else {
            cp_async_wait_all();
            __syncthreads();
        }

        // ---- joint input relu(enc + pred), one thread per column
        {
            float v[kMaxUtt];
#pragma unroll
            for (int u = 0; u < kMaxUtt; ++u) {
                const bool live = ((done8 >> (8 * u)) & 1ull) == 0ull;
                v[u] = live ? fmaxf(__half2float(sm.enc[u][tid]) + sm.pred[u][tid], 0.0f) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < kMaxUtt; ++u) {
                if (((done8 >> (8 * u)) & 1ull) != 0ull) continue;
                if constexpr (Cache) reinterpret_cast<float*>(&sm.ax[0][0])[u * kHidden + tid] = v[u];   // ax as float[8][640]
                else split_store(sm.ax, u, tid, v[u]);
            }
        }
        __syncthreads();
        CL_STAMP(7);
        if constexpr (Cache) {
            // joint rows in fp32 in the reference's summation order (decoder.cu:697-713): one row per
            // half-warp, half-lane l takes elements 2l + 32s, s = 0..19, as one fma chain that starts from
            // the bias in half-lane 0, then the shuffle tree of half_warp_sum.  The score (bias included)
            // lands in the k-group-0 slot of `part`.  Rows come from the caller's [1030, 640] matrix.
            const float* xf = reinterpret_cast<const float*>(&sm.ax[0][0]);
            const int hw = tid / 16, hl = tid % 16;
#pragma unroll 1
            for (int it = 0; it < 2; ++it) {
                const int n = hw + it * (kClThreads / 16);
                const int row = r * kClJoint + n;
                const bool owned = n < kClJoint && row < kJointRows;
                const uint32_t* wrow = reinterpret_cast<const uint32_t*>(
                    p.w_joint + static_cast<size_t>(owned ? row : 0) * kHidden);
                uint32_t words[20];
#pragma unroll
                for (int st = 0; st < 20; ++st) words[st] = __ldg(wrow + hl + 16 * st);
                const float bias = owned ? sm.joint_bias[n] : 0.0f;
                float score[kMaxUtt];
#pragma unroll
                for (int u = 0; u < kMaxUtt; ++u) score[u] = hl == 0 ? bias : 0.0f;
#pragma unroll
                for (int st = 0; st < 20; ++st) {
                    const float2 wv = __half22float2(*reinterpret_cast<const __half2*>(&words[st]));
#pragma unroll
                    for (int u = 0; u < kMaxUtt; ++u) {
                        if (((done8 >> (8 * u)) & 1ull) != 0ull) continue;
                        const float2 xv = *reinterpret_cast<const float2*>(xf + u * kHidden + 2 * hl + 32 * st);
                        score[u] = fmaf(wv.x, xv.x, score[u]);
                        score[u] = fmaf(wv.y, xv.y, score[u]);
                    }
                }
#pragma unroll
                for (int u = 0; u < kMaxUtt; ++u) {
                    if (((done8 >> (8 * u)) & 1ull) != 0ull) continue;
#pragma unroll
                    for (int off = 8; off > 0; off /= 2) score[u] += __shfl_down_sync(0xffffffffu, score[u], off, 16);
                    if (hl == 0 && owned) sm.part[u * JointShape::kPitch + n] = score[u];
                }
            }
        } else {
            FragRing<JointShape, 1> joint_ring;
            if constexpr (Layers == 1) frag_compute<JointShape, false, 1, 0>(sm.wj, &sm.ax[0][0], sm.part, joint_ring, warp, lane);
            else frag_compute<JointShape, true, 1, 0>(wjoint, &sm.ax[0][0], sm.part, joint_ring, warp, lane);
        }
        __syncthreads();
        CL_STAMP(8);
        const int par = static_cast<int>(round & 1u);
        const uint32_t kbar_local = smem_u32(&sm.kbar[par]);
        if (tid == 0) mbar_arrive_expect_tx(&sm.kbar[par], static_cast<uint32_t>(lives) * (kCl * 8 + kDurations * 4));
        // warp u: this CTA's 65 rows of utterance u -> its best key, sent by the same warp (a version
        // with two warps per utterance, a merge through shared memory and a CTA barrier before the
        // send cost 0.3 us more per round)
        if (warp < kMaxUtt) {
            const int u = warp;
            unsigned long long best = 0ull;
            const bool live_u = u < U && !sm.done[u];
            // three passes for every lane (the third covers row 64), so the warp stays converged up
            // to the shuffle reduction
#pragma unroll
            for (int it = 0; it < 3; ++it) {
                const int n = lane + it * 32;
                const int row = r * kClJoint + n;
                if (live_u && n < kClJoint && row < kJointRows) {
                    float total;
                    if constexpr (Cache) {
                        total = sm.part[u * JointShape::kPitch + n];      // finished score of the fp32 joint
                    } else {
                        total = sm.joint_bias[n];
#pragma unroll
                        for (int kg = 0; kg < JointShape::KG; ++kg) total += sm.part[(kg * 8 + u) * JointShape::kPitch + n];
                    }
                    if (row >= kTokenOutputs) {
                        const uint32_t local = smem_u32(&sm.dur[par][u][row - kTokenOutputs]);
                        for (uint32_t d = 0; d < kCl; ++d)
                            st_async_b32(map_to_cta(local, d), __float_as_uint(total), map_to_cta(kbar_local, d));
                    } else if (total == total) {          // NaN never wins
                        float sc = total;
                        if (sc == 0.0f) sc = 0.0f;        // canonicalise -0
                        const unsigned bits = __float_as_uint(sc);
                        const unsigned ordered = (bits & 0x80000000u) ? ~bits : (bits ^ 0x80000000u);
                        const unsigned long long key = (static_cast<unsigned long long>(ordered) << 32) |
                                                       (static_cast<unsigned long long>(2047 - row) << 21) | 1ull;
                        best = key > best ? key : best;
                    }
                }
            }
            __syncwarp();
#pragma unroll
            for (int off = 16; off > 0; off /= 2) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, off);
                best = other > best ? other : best;
            }
            // ---- this CTA's best row of utterance u -> every CTA of the cluster
            if (live_u && lane < kCl) {
                // a CTA whose rows all produced NaN still publishes a (losing) key
                if (best == 0ull) best = (static_cast<unsigned long long>(2047 - kTokenOutputs) << 21) | 1ull;
                st_async_b64(map_to_cta(smem_u32(&sm.keys[par][r][u]), static_cast<uint32_t>(lane)), best,
                             map_to_cta(kbar_local, static_cast<uint32_t>(lane)));
            }
        }
        CL_STAMP(9);
        mbar_wait_bounded(&sm.kbar[par], kphase[par], abort_flag);
        kphase[par] ^= 1u;
        CL_STAMP(10);

        // ---- decision (replicated in every CTA): warp u decides utterance u
        if (warp < U && !sm.done[warp]) {
            const int u = warp;
            unsigned long long best = lane < kCl ? sm.keys[par][lane][u] : 0ull;
#pragma unroll
            for (int off = 16; off > 0; off /= 2) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, off);
                best = other > best ? other : best;
            }
            int token = 2047 - static_cast<int>((best >> 21) & 0x7FFull);
            // keys not delivered (a wait gave up), or every token score of the round was NaN: a
            // blank; the second case is reported as status bit 4
            if (token > kBlank) {
                token = kBlank;
                if (r == 0 && lane == 0 && sm.abort == 0 && p.status != nullptr) atomicOr(p.status, 4);
            }
            // first strict maximum of the five duration logits
            int duration = 0;
            float best_dur = sm.dur[par][u][0];
#pragma unroll
            for (int i = 1; i < kDurations; ++i) {
                const float v = sm.dur[par][u][i];
                if (v > best_dur) { best_dur = v; duration = i; }
            }
            int frame = sm.frame[u] + duration;
            int symbols = sm.symbols[u] + 1;
            if (duration != 0 || symbols == kMaxSymbols) {
                if (duration == 0) frame += 1;
                symbols = 0;
            }
            const bool done = frame >= sm.total_frames[u];
            // requests for the next round, in flight while the state is updated: the token's
            // table row (this CTA's 4 x 40 gate inputs) and the encoder row of the new frame
            if (token != kBlank) {
                const float* row = xtab + static_cast<size_t>(token) * kGates + r * kClUnits;
                for (int n = lane; n < kClUnits * 4; n += 32) cp_async_4(&sm.xg[u][n], row + (n % 4) * kHidden + n / 4);
            }
            if (!done && frame != sm.frame[u]) {
                const __half* src = p.enc_proj + (static_cast<size_t>(u) * p.seg_stride + frame) * kHidden;
                for (int c = lane; c < kEncChunks; c += 32) cp_async_16(&sm.enc[u][c * 8], src + c * 8);
            }
            __syncwarp();
            if (lane == 0) {
                if (sm.need[u]) sm.valid[u] = 1;        // this round's prediction is now current
                if (token != kBlank) {
                    if (r == 0 && sm.count[u] < p.max_tokens) {
                        p.tokens[static_cast<size_t>(u) * p.max_tokens + sm.count[u]] = token;
                        if (p.durations_out != nullptr)
                            p.durations_out[static_cast<size_t>(u) * p.max_tokens + sm.count[u]] = duration;
                    }
                    sm.count[u] += 1;
                    sm.valid[u] = 0;
                }
                sm.frame[u] = frame;
                sm.symbols[u] = symbols;
                sm.done[u] = done;
                sm.need[u] = !done && !sm.valid[u];
            }
        }
        __syncthreads();
        CL_STAMP(11);
        round += 1;
    }
    cp_async_wait_all();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(sm.tmem_base, kTmemColumns);
    }
    cluster_sync_all();      // no CTA leaves while a peer may still address its shared memory
#ifdef PK100_DEC_PROFILE
    if (r == 0 && tid == 0)
        for (int i = 0; i < 16; ++i)
            reinterpret_cast<volatile long long*>(p.workspace + xch_layout(U).abort)[2 + i] = sm.prof[i];
#endif
    if (r == 0 && tid < U && in_window(p, tid)) p.counts[tid] = min(sm.count[tid], p.max_tokens);
    if (r == 0 && tid == 0) reinterpret_cast<volatile int*>(p.workspace + xch_layout(U).abort)[2] = static_cast<int>(round);
    if (sm.abort != 0 && tid == 0 && p.status != nullptr) atomicExch(p.status, 2);
}

}  // namespace pk100

using namespace pk100;

namespace {

size_t decoder_smem_bytes(int grid, int layers, int utts) {
    const int units = (kHidden + grid - 1) / grid;
    const int jrows = (kJointRows + grid - 1) / grid;
    return (static_cast<size_t>(layers) * units * 8 + units + jrows) * kHidden * sizeof(__half) +
           static_cast<size_t>(utts) * 2 * kHidden * sizeof(float);
}

int check_weights(const pk100_decoder_weights* w) {
    if (!w || !w->embedding || !w->w_pred || !w->b_pred || !w->w_joint || !w->b_joint) return PK100_ERR_NULL;
    if (w->layers < 1 || w->layers > 2) return PK100_ERR_SHAPE;
    for (int l = 0; l < w->layers; ++l)
        if (!w->w_ih[l] || !w->w_hh[l] || !w->b_ih[l] || !w->b_hh[l]) return PK100_ERR_NULL;
    return PK100_OK;
}

}  // namespace

extern "C" long long pk100_tdt_rounds_offset(int utterances) {
    if (utterances <= 0 || utterances > kMaxUtt) return -1;
    return static_cast<long long>(xch_layout(utterances).abort) + 8;
}

extern "C" long long pk100_tdt_workspace_bytes(int utterances) {
    if (utterances <= 0 || utterances > kMaxUtt) return 0;
    // barrier / exchange scratch, then the fragment-ordered weight copies of the cluster kernel
    return static_cast<long long>(cl_layout(utterances).total);
}

namespace {

// xtab[token][gate row] = embedding[token] . w_ih[0][gate row] (fp32, no bias) by one tensor-core
// GEMM; `round_fp16`: entries rounded to fp16 precision, as the reference's long-request kernel reads
// them from an fp16 table that its own tensor-core linear kernel wrote (src/cuda/decoder.rs:355-383)
__global__ void tdt_round_table_kernel(float* table, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) table[i] = __half2float(__float2half_rn(table[i]));
}

int build_input_table(void* stream_v, const pk100_decoder_weights* w, float* xtab, int* status, bool round_fp16) {
    pk100_gemm_args g{};
    g.kind = PK100_KIND_F16;
    g.epilogue = PK100_EPI_LINEAR;
    g.m = kTokenOutputs; g.n = kGates; g.k = kHidden;
    g.a = w->embedding; g.lda = kHidden;
    g.b = w->w_ih[0]; g.ldb = kHidden;
    g.row_scale = 1.0f;
    g.alpha = 1.0f;
    g.out = xtab; g.ld_out = kGates;
    g.out_type = PK100_OUT_F32;
    g.out_scale = 1.0f;
    g.status = status;
    const int grc = pk100_gemm(stream_v, &g);
    if (grc != PK100_OK) return grc;
    if (round_fp16) {
        const int n = kTokenOutputs * kGates;
        tdt_round_table_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream_v)>>>(xtab, n);
        pk100_count_launch();
        const cudaError_t err = cudaGetLastError();
        if (err != cudaSuccess) return static_cast<int>(err);
    }
    return PK100_OK;
}

// max |w| of w_hh[0], w_hh[1], w_ih[1] -> three floats at cl_layout().cache of the workspace
// (the per-tensor scales of the INT8 cache are derived inside every request, decoder.cu:517-555)
int launch_cache_absmax(cudaStream_t stream, const pk100_decoder_weights* w, uint8_t* ws, int utterances,
                        const float** out) {
    unsigned* slot = reinterpret_cast<unsigned*>(ws + cl_layout(utterances).cache);
    cudaError_t err = cudaMemsetAsync(slot, 0, 16, stream);
    if (err != cudaSuccess) return static_cast<int>(err);
    const int n = kGates * kHidden;
    tdt_absmax_kernel<<<160, 256, 0, stream>>>(static_cast<const __half*>(w->w_hh[0]), n, slot);
    pk100_count_launch();
    if (w->layers == 2) {
        tdt_absmax_kernel<<<160, 256, 0, stream>>>(static_cast<const __half*>(w->w_hh[1]), n, slot + 1);
        tdt_absmax_kernel<<<160, 256, 0, stream>>>(static_cast<const __half*>(w->w_ih[1]), n, slot + 2);
        pk100_count_launch();
        pk100_count_launch();
    }
    err = cudaGetLastError();
    if (err != cudaSuccess) return static_cast<int>(err);
    *out = reinterpret_cast<const float*>(slot);
    return PK100_OK;
}

int decode_barrier(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
                                int utterances, int seg_stride, const int* frames, void* workspace,
                                int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                                int* status, bool cache, int frames_lo = INT_MIN, int frames_hi = INT_MAX) {
    const int rc = check_weights(w);
    if (rc != PK100_OK) return rc;
    if (!enc_proj || !frames || !workspace || !tokens || !counts) return PK100_ERR_NULL;
    if (utterances == 0) return PK100_OK;
    if (utterances < 0 || seg_stride <= 0 || max_tokens <= 0) return PK100_ERR_SHAPE;
    if (utterances > kMaxUtt) return PK100_ERR_LIMIT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    int dev = 0, sms = 0, max_smem = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    const int grid = sms;
    const size_t smem = decoder_smem_bytes(grid, w->layers, utterances);
    if (smem + 1024 > static_cast<size_t>(max_smem)) return PK100_ERR_LIMIT;
    cudaError_t err = cudaFuncSetAttribute(tdt_greedy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
    if (err != cudaSuccess) return static_cast<int>(err);

    DecParams p{};
    p.enc_proj = static_cast<const __half*>(enc_proj);
    p.seg_stride = seg_stride;
    p.frames = frames;
    p.utts = utterances;
    p.layers = w->layers;
    p.embedding = static_cast<const __half*>(w->embedding);
    for (int l = 0; l < w->layers; ++l) {
        p.w_ih[l] = static_cast<const __half*>(w->w_ih[l]);
        p.w_hh[l] = static_cast<const __half*>(w->w_hh[l]);
        p.b_ih[l] = w->b_ih[l];
        p.b_hh[l] = w->b_hh[l];
    }
    p.w_pred = static_cast<const __half*>(w->w_pred);
    p.b_pred = w->b_pred;
    p.w_joint = static_cast<const __half*>(w->w_joint);
    p.b_joint = w->b_joint;
    p.workspace = static_cast<uint8_t*>(workspace);
    p.tokens = tokens;
    p.durations_out = durations;
    p.counts = counts;
    p.max_tokens = max_tokens;
    p.status = status;
    p.frames_lo = frames_lo;
    p.frames_hi = frames_hi;
    if (cache) {
        const int crc = launch_cache_absmax(stream, w, p.workspace, utterances, &p.cache_absmax);
        if (crc != PK100_OK) return crc;
        float* xtab = reinterpret_cast<float*>(p.workspace + cl_layout(utterances).xtab);
        const int trc = build_input_table(stream_v, w, xtab, status, true);
        if (trc != PK100_OK) return trc;
        p.input_table = xtab;
    }

    // state, decisions and the barrier words start from zero on every call
    err = cudaMemsetAsync(workspace, 0, dec_layout(utterances).total, stream);
    if (err != cudaSuccess) return static_cast<int>(err);
    void* args[] = {&p};
    // cooperative launch: the runtime refuses the launch unless every CTA is co-resident,
    // which the grid barrier needs
    err = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(tdt_greedy_kernel), dim3(grid),
                                      dim3(kDecThreads), args, smem, stream);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return static_cast<int>(err);
    }
    pk100_count_launch();
    return PK100_OK;
}

}  // namespace

extern "C" int pk100_tdt_decode_barrier(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
                                        int utterances, int seg_stride, const int* frames, void* workspace,
                                        int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                                        int* status) {
    return decode_barrier(stream_v, w, enc_proj, utterances, seg_stride, frames, workspace, tokens, durations,
                          counts, max_tokens, status, false);
}

extern "C" int pk100_tdt_decode_long_barrier(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
                                             int utterances, int seg_stride, const int* frames, void* workspace,
                                             int32_t* tokens, int32_t* durations, int32_t* counts,
                                             int max_tokens, int* status) {
    return decode_barrier(stream_v, w, enc_proj, utterances, seg_stride, frames, workspace, tokens, durations,
                          counts, max_tokens, status, true);
}

// ---------------------------------------------------------------------------
// Entry point for callers that cannot allocate device memory.
//
// Some embedders of this library run inside a host that owns the CUDA memory pool and
// forbids cudaMalloc from plug-in code (a serving process with a pre-sized arena, a
// real-time audio host, code running between the nodes of somebody else's stream
// capture).  For them the decoder's exchange scratch lives in the library image itself:
// a file-scope device array of fixed size, resident on every GPU that loads the library
// until the process exits.
constexpr size_t kStaticScratchBytes = 288 * 1024;   // covers xch_layout(8) = 279 808 bytes
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
// In host code `g_static_scratch` is only a handle for the runtime, not a device address:
// the address a kernel may dereference is looked up once per device.
// Entries are atomic: two host threads that make the first call on a device at once both look the
// address up and store the same value.  A cudaDeviceReset invalidates the cached address.
std::atomic<void*> g_static_scratch_ptr[64];

int static_scratch_address(void** out) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return static_cast<int>(err);
    if (dev < 0 || dev >= 64) return PK100_ERR_LIMIT;
    void* ptr = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        err = cudaGetSymbolAddress(&ptr, g_static_scratch);   // with device `dev` current
        if (err != cudaSuccess) {
            cudaGetLastError();
            return static_cast<int>(err);
        }
        g_static_scratch_ptr[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return PK100_OK;
}
}  // namespace

extern "C" int pk100_tdt_decode_exchange(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
                                         int utterances, int seg_stride, const int* frames, void* workspace,
                                         int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                                         int* status);

extern "C" int pk100_tdt_decode_static(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
                                       int utterances, int seg_stride, const int* frames, int32_t* tokens,
                                       int32_t* durations, int32_t* counts, int max_tokens, int* status) {
    if (utterances > kMaxUtt) return PK100_ERR_LIMIT;          // scratch is sized for 8 utterances
    if (utterances > 0 && xch_layout(utterances).total > kStaticScratchBytes) return PK100_ERR_LIMIT;
    void* scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != PK100_OK) return rc;
    // pk100_tdt_decode_exchange clears the part of the scratch it uses (stream-ordered memset of
    // existing memory) and launches the kernel: no allocation on this path
    return pk100_tdt_decode_exchange(stream_v, w, enc_proj, utterances, seg_stride, frames, scratch, tokens,
                                     durations, counts, max_tokens, status);
}

extern "C" int pk100_tdt_decode_exchange(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
                                         int utterances, int seg_stride, const int* frames, void* workspace,
                                         int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                                         int* status) {
    const int rc = check_weights(w);
    if (rc != PK100_OK) return rc;
    if (!enc_proj || !frames || !workspace || !tokens || !counts) return PK100_ERR_NULL;
    if (utterances == 0) return PK100_OK;
    if (utterances < 0 || seg_stride <= 0 || max_tokens <= 0) return PK100_ERR_SHAPE;
    if (utterances > kMaxUtt) return PK100_ERR_LIMIT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // 20 warps per CTA own (5 hidden units x 4 gates): the grid must cover 640 units with
    // at most 5 per CTA and 1030 joint rows with at most 8 per CTA
    if (sms < 129 || sms > kXMaxGrid) return pk100_tdt_decode_barrier(stream_v, w, enc_proj, utterances,
                                                                      seg_stride, frames, workspace, tokens,
                                                                      durations, counts, max_tokens, status);
    const int grid = sms;
    cudaError_t err = cudaFuncSetAttribute(tdt_exchange_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(sizeof(XSmem)));
    if (err != cudaSuccess) return static_cast<int>(err);
    DecParams p{};
    p.enc_proj = static_cast<const __half*>(enc_proj);
    p.seg_stride = seg_stride;
    p.frames = frames;
    p.utts = utterances;
    p.layers = w->layers;
    p.embedding = static_cast<const __half*>(w->embedding);
    for (int l = 0; l < w->layers; ++l) {
        p.w_ih[l] = static_cast<const __half*>(w->w_ih[l]);
        p.w_hh[l] = static_cast<const __half*>(w->w_hh[l]);
        p.b_ih[l] = w->b_ih[l];
        p.b_hh[l] = w->b_hh[l];
    }
    p.w_pred = static_cast<const __half*>(w->w_pred);
    p.b_pred = w->b_pred;
    p.w_joint = static_cast<const __half*>(w->w_joint);
    p.b_joint = w->b_joint;
    p.workspace = static_cast<uint8_t*>(workspace);
    p.tokens = tokens;
    p.durations_out = durations;
    p.counts = counts;
    p.max_tokens = max_tokens;
    p.status = status;
    p.frames_lo = INT_MIN;
    p.frames_hi = INT_MAX;
    // tags start at 1, so a cleared workspace holds no valid entry
    err = cudaMemsetAsync(workspace, 0, xch_layout(utterances).total, stream);
    if (err != cudaSuccess) return static_cast<int>(err);
    void* args[] = {&p};
    // cooperative launch = the runtime guarantees all CTAs are co-resident (they poll each other)
    err = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(tdt_exchange_kernel), dim3(grid),
                                      dim3(kXThreads), args, sizeof(XSmem), stream);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return static_cast<int>(err);
    }
    pk100_count_launch();
    return PK100_OK;
}

namespace {

// Can this device run a 16-CTA cluster of the cluster decoder?  Asked once per device and
// kernel variant (one or two LSTM layers).
template <int Layers, bool Cache>
bool cluster_decoder_available(int* capacity = nullptr) {
    static int cached[64] = {0};      // 0 = unknown, 1 = yes, 2 = no
    static int resident[64] = {0};    // clusters of this kernel the device holds at once
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (cached[dev] != 0) {
        if (capacity != nullptr) *capacity = resident[dev];
        return cached[dev] == 1;
    }
    bool ok = false;
    do {
        int max_smem = 0;
        cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (sizeof(CSmemT<Layers>) > static_cast<size_t>(max_smem)) break;
        if (cudaFuncSetAttribute(tdt_cluster_kernel<Layers, Cache>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(sizeof(CSmemT<Layers>))) != cudaSuccess) break;
        if (cudaFuncSetAttribute(tdt_cluster_kernel<Layers, Cache>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) !=
            cudaSuccess) break;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(kCl);
        cfg.blockDim = dim3(kClThreads);
        cfg.dynamicSmemBytes = sizeof(CSmemT<Layers>);
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = kCl;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, tdt_cluster_kernel<Layers, Cache>, &cfg) != cudaSuccess) break;
        ok = clusters >= 1;
        resident[dev] = clusters;
    } while (false);
    cudaGetLastError();
    cached[dev] = ok ? 1 : 2;
    if (capacity != nullptr) *capacity = resident[dev];
    return ok;
}

bool cluster_decoder_available_for(int layers, bool cache) {
    if (layers == 1) return cache ? cluster_decoder_available<1, true>() : cluster_decoder_available<1, false>();
    if (layers == 2) return cache ? cluster_decoder_available<2, true>() : cluster_decoder_available<2, false>();
    return false;
}

}  // namespace

extern "C" int pk100_tdt_cluster_capacity(int lstm_layers) {
    int clusters = 0;
    bool ok = false;
    if (lstm_layers == 1) ok = cluster_decoder_available<1, false>(&clusters);
    else if (lstm_layers == 2) ok = cluster_decoder_available<2, false>(&clusters);
    return ok ? clusters : 0;
}

namespace {

template <int Layers, bool Cache>
cudaError_t launch_cluster_kernel(cudaStream_t stream, const DecParams& p, const uint4* lstm, const uint4* pred,
                                  const uint4* joint, const float* xtab, const uint4* lstm1) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(kCl);
    cfg.blockDim = dim3(kClThreads);
    cfg.dynamicSmemBytes = sizeof(CSmemT<Layers>);
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = kCl;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, tdt_cluster_kernel<Layers, Cache>, p, lstm, pred, joint, xtab, lstm1);
}

}  // namespace

namespace {
int decode_cluster(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
                                        int utterances, int seg_stride, const int* frames, void* workspace,
                                        int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                                        int* status, bool cache, int frames_lo = INT_MIN, int frames_hi = INT_MAX) {
    const int rc = check_weights(w);
    if (rc != PK100_OK) return rc;
    if (!enc_proj || !frames || !workspace || !tokens || !counts) return PK100_ERR_NULL;
    if (utterances == 0) return PK100_OK;
    if (utterances < 0 || seg_stride <= 0 || max_tokens <= 0) return PK100_ERR_SHAPE;
    if (utterances > kMaxUtt) return PK100_ERR_LIMIT;
    if (!cluster_decoder_available_for(w->layers, cache)) return PK100_ERR_UNSUPPORTED;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const ClLayout lay = cl_layout(utterances);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    const float* absmax = nullptr;
    if (cache) {
        const int crc = launch_cache_absmax(stream, w, ws, utterances, &absmax);
        if (crc != PK100_OK) return crc;
    }
    uint4* packed_lstm = reinterpret_cast<uint4*>(ws + lay.lstm);
    uint4* packed_pred = reinterpret_cast<uint4*>(ws + lay.pred);
    uint4* packed_joint = reinterpret_cast<uint4*>(ws + lay.joint);
    uint4* packed_lstm1 = reinterpret_cast<uint4*>(ws + lay.lstm1);
    float* xtab = reinterpret_cast<float*>(ws + lay.xtab);
    const __half* w_hh = static_cast<const __half*>(w->w_hh[0]);
    const __half* w_pred = static_cast<const __half*>(w->w_pred);
    const __half* w_joint = static_cast<const __half*>(w->w_joint);
    // weights -> fragment order (they may change between calls, so this is done every call)
    tdt_pack_kernel<LstmShape, CLPACK_LSTM><<<(kCl * LstmShape::kPerCta + 255) / 256, 256, 0, stream>>>(
        packed_lstm, w_hh, nullptr, absmax, 0, 0);
    tdt_pack_kernel<PredShape, CLPACK_PRED><<<(kCl * PredShape::kPerCta + 255) / 256, 256, 0, stream>>>(
        packed_pred, w_pred, nullptr, nullptr, 0, 0);
    tdt_pack_kernel<JointShape, CLPACK_JOINT><<<(kCl * JointShape::kPerCta + 255) / 256, 256, 0, stream>>>(
        packed_joint, w_joint, nullptr, nullptr, 0, 0);
    pk100_count_launch();
    pk100_count_launch();
    pk100_count_launch();
    if (w->layers == 2) {
        tdt_pack_kernel<Lstm1Shape, CLPACK_LSTM_IH_HH><<<(kCl * Lstm1Shape::kPerCta + 255) / 256, 256, 0, stream>>>(
            packed_lstm1, static_cast<const __half*>(w->w_ih[1]), static_cast<const __half*>(w->w_hh[1]), absmax, 2, 1);
        pk100_count_launch();
    }
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return static_cast<int>(err);
    {
        const int trc = build_input_table(stream_v, w, xtab, status, cache);
        if (trc != PK100_OK) return trc;
    }

    DecParams p{};
    p.enc_proj = static_cast<const __half*>(enc_proj);
    p.seg_stride = seg_stride;
    p.frames = frames;
    p.utts = utterances;
    p.layers = w->layers;
    p.embedding = static_cast<const __half*>(w->embedding);
    for (int l = 0; l < w->layers; ++l) {
        p.w_ih[l] = static_cast<const __half*>(w->w_ih[l]);
        p.w_hh[l] = static_cast<const __half*>(w->w_hh[l]);
        p.b_ih[l] = w->b_ih[l];
        p.b_hh[l] = w->b_hh[l];
    }
    p.w_pred = w_pred;
    p.b_pred = w->b_pred;
    p.w_joint = w_joint;
    p.b_joint = w->b_joint;
    p.workspace = ws;
    p.tokens = tokens;
    p.durations_out = durations;
    p.counts = counts;
    p.max_tokens = max_tokens;
    p.status = status;
    p.cache_absmax = absmax;
    p.frames_lo = frames_lo;
    p.frames_hi = frames_hi;

    if (w->layers == 1)
        err = cache ? launch_cluster_kernel<1, true>(stream, p, packed_lstm, packed_pred, packed_joint, xtab, packed_lstm1)
                    : launch_cluster_kernel<1, false>(stream, p, packed_lstm, packed_pred, packed_joint, xtab, packed_lstm1);
    else
        err = cache ? launch_cluster_kernel<2, true>(stream, p, packed_lstm, packed_pred, packed_joint, xtab, packed_lstm1)
                    : launch_cluster_kernel<2, false>(stream, p, packed_lstm, packed_pred, packed_joint, xtab, packed_lstm1);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return static_cast<int>(err);
    }
    pk100_count_launch();
    return PK100_OK;
}
}  // namespace

extern "C" int pk100_tdt_decode_cluster(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
                                        int utterances, int seg_stride, const int* frames, void* workspace,
                                        int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                                        int* status) {
    return decode_cluster(stream_v, w, enc_proj, utterances, seg_stride, frames, workspace, tokens, durations,
                          counts, max_tokens, status, false);
}

extern "C" int pk100_tdt_decode_long_cluster(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
                                             int utterances, int seg_stride, const int* frames, void* workspace,
                                             int32_t* tokens, int32_t* durations, int32_t* counts,
                                             int max_tokens, int* status) {
    return decode_cluster(stream_v, w, enc_proj, utterances, seg_stride, frames, workspace, tokens, durations,
                          counts, max_tokens, status, true);
}

extern "C" int pk100_tdt_decode_long(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
                                     int utterances, int seg_stride, const int* frames, void* workspace,
                                     int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                                     int* status) {
    // the cluster kernel where a 16-CTA cluster can be hosted, else the grid-barrier kernel
    if (w != nullptr && utterances > 0 && utterances <= kMaxUtt && cluster_decoder_available_for(w->layers, true))
        return pk100_tdt_decode_long_cluster(stream_v, w, enc_proj, utterances, seg_stride, frames, workspace,
                                             tokens, durations, counts, max_tokens, status);
    return pk100_tdt_decode_long_barrier(stream_v, w, enc_proj, utterances, seg_stride, frames, workspace, tokens,
                                         durations, counts, max_tokens, status);
}

extern "C" int pk100_tdt_decode_auto(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
                                     int utterances, int seg_stride, const int* frames, void* workspace,
                                     int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                                     int* status) {
    // the reference's rule per request (src/cuda/decoder.rs:15, :88), here per utterance: two
    // launches on the same stream, each decoding its own utterances and skipping the others
    constexpr int kLongRequestFrames = 1024;
    const bool cluster = w != nullptr && utterances > 0 && utterances <= kMaxUtt &&
                         cluster_decoder_available_for(w->layers, false) && cluster_decoder_available_for(w->layers, true);
    auto run = cluster ? decode_cluster : decode_barrier;
    const int rc = run(stream_v, w, enc_proj, utterances, seg_stride, frames, workspace, tokens, durations, counts,
                       max_tokens, status, false, INT_MIN, kLongRequestFrames);
    if (rc != PK100_OK) return rc;
    return run(stream_v, w, enc_proj, utterances, seg_stride, frames, workspace, tokens, durations, counts,
               max_tokens, status, true, kLongRequestFrames, INT_MAX);
}

extern "C" int pk100_tdt_decode(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
                                int utterances, int seg_stride, const int* frames, void* workspace,
                                int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                                int* status) {
    // a device that can host a 16-CTA cluster: the cluster kernel; anything else: the 148-CTA
    // exchange kernel
    if (w != nullptr && utterances > 0 && utterances <= kMaxUtt && cluster_decoder_available_for(w->layers, false))
        return pk100_tdt_decode_cluster(stream_v, w, enc_proj, utterances, seg_stride, frames, workspace, tokens,
                                        durations, counts, max_tokens, status);
    return pk100_tdt_decode_exchange(stream_v, w, enc_proj, utterances, seg_stride, frames, workspace, tokens,
                                     durations, counts, max_tokens, status);
}
