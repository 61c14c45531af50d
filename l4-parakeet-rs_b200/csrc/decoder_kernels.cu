// TDT greedy decode for a batch of utterances, one persistent cooperative kernel.
//
// Every decoder weight (LSTM input/recurrent gates, prediction projection,
// joint head; ~15 MB fp16) is sliced across the CTAs once and stays resident in
// shared memory for the whole decode; the utterances of the batch advance in
// lockstep rounds so each round reads the weights once for all of them.
// Per round: [LSTM layer 0 | barrier | LSTM layer 1 | barrier | prediction
// projection | barrier] for the utterances that just emitted a token, then
// joint + argmax | barrier.  Grid barriers are bounded: when one expires the
// kernel records it in the status word and every CTA leaves.
//
// Decision rules follow kernels/sm89/decoder.cu:35-46 (order-preserving key,
// ties to the lower token id), :416-422 (first strict maximum duration) and
// :431-445 (frame advance, at most 10 symbols per frame, blank keeps the state).
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <float.h>
#include <stdint.h>

#include "pk100_internal.h"

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
};

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

    // ---- load this CTA's weight slices (once)
    for (int l = 0; l < p.layers; ++l) {
        for (int i = 0; i < units; ++i) {
            const int unit = cta + G * i;
            for (int r = 0; r < 8; ++r) {
                __half* dst = s_lstm + ((static_cast<size_t>(l) * units + i) * 8 + r) * kHidden;
                const __half* src = (r < 4 ? p.w_ih[l] : p.w_hh[l]) +
                                    (static_cast<size_t>(r & 3) * kHidden + unit) * kHidden;
                for (int c = tid; c < kHidden; c += kDecThreads)
                    dst[c] = unit < kHidden ? src[c] : __float2half(0.0f);
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
        s_done[tid] = p.frames[tid] <= 0;
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
                        }
                        vec[c] = x;
                        vec[kHidden + c] = __ldcg(committed + l * kHidden + c);
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
                        float acc = dot640(wrow + r * kHidden, vec, lane) +
                                    dot640(wrow + (4 + r) * kHidden, vec + kHidden, lane);
                        acc = warp_sum_f(acc);
                        gate[r] = acc + p.b_ih[l][r * kHidden + unit] + p.b_hh[l][r * kHidden + unit];
                    }
                    if (lane == 0) {
                        float* st = g_state + static_cast<size_t>(u) * kStatePerUtt;
                        const float* committed = st + (s_alt[u] ? 4 * kHidden : 0);
                        float* candidate = st + (s_alt[u] ? 0 : 4 * kHidden);
                        const float ig = 1.0f / (1.0f + expf(-gate[0]));
                        const float fg = 1.0f / (1.0f + expf(-gate[1]));
                        const float gg = tanhf(gate[2]);
                        const float og = 1.0f / (1.0f + expf(-gate[3]));
                        const float cell = fg * __ldcg(committed + (2 + l) * kHidden + unit) + ig * gg;
                        __stcg(candidate + (2 + l) * kHidden + unit, cell);
                        __stcg(candidate + l * kHidden + unit, og * tanhf(cell));
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
                float acc = warp_sum_f(dot640(s_pred + i * kHidden, s_vec + u * 2 * kHidden, lane));
                if (lane == 0) __stcg(g_pred + static_cast<size_t>(u) * kHidden + row, acc + p.b_pred[row]);
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
            float acc = warp_sum_f(dot640(s_joint + i * kHidden, s_vec + u * 2 * kHidden, lane));
            if (lane == 0) {
                acc += p.b_joint[row];
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
            const int token = static_cast<int>(0xffffffffu - static_cast<unsigned>(key));
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
            if (s_frame[u] >= p.frames[u]) s_done[u] = 1;
        }
        __syncthreads();
        slot = next_slot;
    }

    if (cta == 0 && tid < p.utts) p.counts[tid] = min(s_count[tid], p.max_tokens);
    if (!ok && cta == 0 && tid == 0 && p.status != nullptr) atomicExch(p.status, 2);
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

extern "C" long long pk100_tdt_workspace_bytes(int utterances) {
    if (utterances <= 0 || utterances > kMaxUtt) return 0;
    return static_cast<long long>(dec_layout(utterances).total);
}

extern "C" int pk100_tdt_decode(void* stream_v, const pk100_decoder_weights* w, const void* enc_proj,
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
