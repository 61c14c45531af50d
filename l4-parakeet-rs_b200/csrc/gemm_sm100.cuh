// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D[M,N] = epilogue( A[M,K] . B[N,K]^T )      A, B row-major ("K-major")
//
// One CTA per SM loops over 128 x BLOCK_N output tiles.
//   warp 0      TMA producer: global -> swizzled shared-memory stage ring
//   warp 1      tcgen05.mma issuer (one elected lane); owns the TMEM allocation
//   warps 2..9  epilogue: tcgen05.ld the fp32/s32 accumulator, apply scales /
//               bias / activation / residual / quantisation, store to global
// Accumulators are double-buffered in TMEM (2 x BLOCK_N columns) so the MMAs of
// tile i+1 overlap the epilogue of tile i.  All waits are bounded (ptx_sm100.cuh).
#pragma once

#include <cuda_fp8.h>

#include "ptx_sm100.cuh"

namespace pk100 {

enum : int { OUT_F16 = 0, OUT_F32 = 1, OUT_E4M3 = 2, OUT_S8 = 3 };
enum : int { ACT_NONE = 0, ACT_SILU = 1, ACT_RELU = 2 };
enum : int { EPI_LINEAR = 0, EPI_GLU = 1, EPI_SPARSE_OUT = 2 };
// B operand sources: TMA from a K-major matrix, or INT4 group-quantised weights
// dequantised to fp16 in shared memory by the producer warps.
enum : int { BSRC_TMA = 0, BSRC_W4G128 = 1 };

struct GemmParams {
    int m, n, k;                 // n counts B rows (GLU: value rows + gate rows)
    // epilogue inputs
    const float* row_scales;     // [m] per-row activation scales, or nullptr
    float row_scale;             // used when row_scales == nullptr
    const float* col_scales;     // [n] per-output-channel weight scales, or nullptr
    const float* bias;           // [n] or nullptr
    int act;
    const __half* residual;      // [m, ld_res] or nullptr; may alias `out`
    int ld_res;
    float alpha;                 // out = alpha * value (+ residual)
    int valid_rows;              // rows >= valid_rows are stored as zero
    // output
    void* out;
    int ld_out;                  // elements
    int out_type;
    float out_scale;             // multiplier applied before E4M3 / S8 encoding
    // tile sparsity, producer side (EPI_SPARSE_OUT)
    float tau;
    uint8_t* keep_out;           // [ceil(m/128), n/64]
    float* stats_out;            // [ceil(m/128), n/64] or nullptr
    // tile sparsity, consumer side
    const uint8_t* keep_in;      // [ceil(m/128), k/64] or nullptr
    // INT4 group-128 weights (BSRC_W4G128)
    const uint8_t* w4_codes;     // [n, k/2], low nibble = even k
    const __half* w4_scales;     // [k/128, n]
    int* status;                 // set non-zero when a bounded wait gave up
};

constexpr int kBlockM = 128;
constexpr int kEpilogueWarps = 8;
constexpr int kGemmThreads = 32 * (2 + kEpilogueWarps);

// BRows = B rows staged per CTA per stage, EpiCols = accumulator columns of the tile.
template <int BRows, int SwizzleBytes, int EpiCols = BRows>
struct GemmSmem {
    static constexpr int kStageA = kBlockM * SwizzleBytes;
    static constexpr int kStageB = BRows * SwizzleBytes;
    static constexpr int kStageBytes = kStageA + kStageB;
    static constexpr int kBudget = 196 * 1024;
    static constexpr int kStagesRaw = kBudget / kStageBytes;
    static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
    static constexpr int kTileBytes = kStages * kStageBytes;
    // tail: barriers + tmem pointer + abort flag + epilogue staging
    static constexpr int kTailBytes = 64 * 8 + 16 + 2 * EpiCols * 4 + 64 * 4;
    static constexpr int kTotal = kTileBytes + kTailBytes + 1024;  // + alignment slack
};

__device__ __forceinline__ float silu_f(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float round_f16(float v) { return __half2float(__float2half_rn(v)); }

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

__device__ __forceinline__ int quant_s8(float v) {
    return max(-127, min(127, __float2int_rn(v)));
}

__device__ __forceinline__ uint32_t pack_s8x4(float a, float b, float c, float d) {
    return (quant_s8(a) & 255) | ((quant_s8(b) & 255) << 8) | ((quant_s8(c) & 255) << 16) |
           ((quant_s8(d) & 255) << 24);
}

template <int Kind>
__device__ __forceinline__ float acc_to_float(uint32_t r) {
    if constexpr (Kind == KIND_I8) {
        return static_cast<float>(static_cast<int>(r));
    } else {
        return __uint_as_float(r);
    }
}

// Named barrier over the epilogue warps only.
template <int Warps>
__device__ __forceinline__ void epilogue_bar_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(32 * Warps) : "memory");
}

// Store 32 consecutive output columns of one row.
__device__ __forceinline__ void store_chunk(void* out_row, int out_type, float out_scale,
                                            const float (&v)[32]) {
    if (out_type == OUT_F16) {
        uint4* dst = reinterpret_cast<uint4*>(out_row);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            dst[i] = make_uint4(pack_half2(v[8 * i + 0], v[8 * i + 1]),
                                pack_half2(v[8 * i + 2], v[8 * i + 3]),
                                pack_half2(v[8 * i + 4], v[8 * i + 5]),
                                pack_half2(v[8 * i + 6], v[8 * i + 7]));
        }
    } else if (out_type == OUT_F32) {
        float4* dst = reinterpret_cast<float4*>(out_row);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
    } else if (out_type == OUT_E4M3) {
        uint4* dst = reinterpret_cast<uint4*>(out_row);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int b = 16 * i + 4 * j;
                w[j] = pack_e4m3x4(round_f16(v[b]) * out_scale, round_f16(v[b + 1]) * out_scale,
                                   round_f16(v[b + 2]) * out_scale, round_f16(v[b + 3]) * out_scale);
            }
            dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
        uint4* dst = reinterpret_cast<uint4*>(out_row);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int b = 16 * i + 4 * j;
                w[j] = pack_s8x4(round_f16(v[b]) * out_scale, round_f16(v[b + 1]) * out_scale,
                                 round_f16(v[b + 2]) * out_scale, round_f16(v[b + 3]) * out_scale);
            }
            dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

__device__ __forceinline__ size_t out_elem_bytes(int out_type) {
    return out_type == OUT_F16 ? 2 : (out_type == OUT_F32 ? 4 : 1);
}

// Bit i of the mask = "64-element K tile i of M tile `mt` holds a non-zero".
// Without a bitmap every tile is live.  K <= 4096 (64 tiles) is checked on the host.
__device__ __forceinline__ uint64_t load_live_mask(const uint8_t* keep_in, int mt, int k_tiles64) {
    if (keep_in == nullptr) return ~0ull;
    const uint8_t* row = keep_in + static_cast<size_t>(mt) * k_tiles64;
    uint64_t mask = 0;
    for (int i = 0; i < k_tiles64; ++i) mask |= static_cast<uint64_t>(row[i] != 0) << i;
    return mask;
}

// Is K block `kb` (SwizzleBytes wide, 8-bit elements) live?
template <int SwizzleBytes>
__device__ __forceinline__ bool k_block_live(uint64_t mask, int kb) {
    if constexpr (SwizzleBytes == 64) {
        return (mask >> kb) & 1ull;
    } else {
        return ((mask >> (2 * kb)) & 3ull) != 0;
    }
}

// CtaGroup = 2: the CTAs of a 2-CTA cluster share one 256 x BlockN tile (tcgen05 cta_group::2).
// Each CTA stages its own 128 rows of A and BlockN/2 rows of B, so a tile costs 2/3 of the
// operand traffic of two independent 128 x BlockN tiles; the even CTA issues the MMAs, each CTA
// runs the epilogue of its own 128 accumulator rows.
template <int Kind, int BlockN, int SwizzleBytes, int Epi, int BSrc, int CtaGroup = 1>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const GemmParams p) {
    static_assert(CtaGroup == 1 || (CtaGroup == 2 && BlockN == 256 && BSrc == BSRC_TMA), "pairs: 256 columns, TMA");
    constexpr int kBRows = BlockN / CtaGroup;               // B rows staged by this CTA
    using Smem = GemmSmem<kBRows, SwizzleBytes, BlockN>;
    constexpr int kStages = Smem::kStages;
    constexpr int kElemBytes = Kind == KIND_F16 ? 2 : 1;
    constexpr int kBlockK = SwizzleBytes / kElemBytes;       // elements per K block
    constexpr int kMmasPerBlock = SwizzleBytes / 32;         // 32 bytes of K per MMA
    constexpr uint32_t kTmemCols = 2 * BlockN;
    constexpr int kBHalf = BlockN / 2;                       // rows per B load
    static_assert(BlockN == 64 || BlockN == 128 || BlockN == 256, "BlockN");
    static_assert(BSrc == BSRC_TMA || (Kind == KIND_F16 && SwizzleBytes == 128 && BlockN == 128 &&
                                       Epi == EPI_LINEAR), "w4: fp16 MMA, 128-column tiles, linear epilogue");
    // INT4 weights: 4 epilogue warps (one per TMEM lane quadrant) + 4 dequantisation warps;
    // otherwise 8 epilogue warps, two per quadrant, each half of the tile's columns.
    constexpr int kEpiWarps = BSrc == BSRC_W4G128 ? 4 : kEpilogueWarps;
    constexpr int kColSplit = kEpiWarps / 4;
    constexpr int kColsPerWarp = BlockN / kColSplit;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* tail = smem + Smem::kTileBytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
    uint64_t* empty_bar = full_bar + kStages;
    uint64_t* tmem_full_bar = empty_bar + kStages;
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;
    uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(tail + 64 * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 64 * 8 + 8);
    float* s_col_scale = reinterpret_cast<float*>(tail + 64 * 8 + 16);
    float* s_bias = s_col_scale + BlockN;
    float* s_reduce = s_bias + BlockN;                       // [kEpilogueWarps][4]

    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;

    const uint32_t rank = CtaGroup == 2 ? cluster_ctarank() : 0u;   // 0 = leader of the pair
    const int worker = static_cast<int>(blockIdx.x) / CtaGroup;      // pair (or CTA) index
    const int workers = static_cast<int>(gridDim.x) / CtaGroup;
    const int m_tiles = (p.m + kBlockM - 1) / kBlockM;                // 128-row tiles
    const int m_groups = (m_tiles + CtaGroup - 1) / CtaGroup;         // tiles of 128 * CtaGroup rows
    const int n_tiles = (p.n + BlockN - 1) / BlockN;
    const int num_tiles = m_groups * n_tiles;
    const int k_blocks = (p.k + kBlockK - 1) / kBlockK;
    const int k_tiles64 = p.k / 64;
    // live-K mask of a work item: union over the 128-row tiles it covers
    auto group_live_mask = [&](int mg) {
        uint64_t mask = load_live_mask(p.keep_in, mg * CtaGroup, k_tiles64);
        if (CtaGroup == 2 && p.keep_in != nullptr && mg * 2 + 1 < m_tiles)
            mask |= load_live_mask(p.keep_in, mg * 2 + 1, k_tiles64);
        return mask;
    };

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            // full: one arrive.expect_tx from the TMA lane (+ 4 producer warps for W4)
            mbar_init(full_bar + s, BSrc == BSRC_W4G128 ? 1 + 4 : 1);
            mbar_init(empty_bar + s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tmem_full_bar + b, 1);
            mbar_init(tmem_empty_bar + b, kEpiWarps * CtaGroup);
        }
        fence_barrier_init();
        prefetch_tensormap(&map_a);
        if constexpr (BSrc == BSRC_TMA) prefetch_tensormap(&map_b);
    }
    if (warp == 1) {
        if constexpr (CtaGroup == 2) {
            tmem_alloc_pair(tmem_ptr_smem, kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_ptr_smem, kTmemCols);
            tmem_relinquish();
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    // both CTAs' barriers exist before either one signals the other
    if constexpr (CtaGroup == 2) cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = worker; tile < num_tiles && ok; tile += workers) {
                const int mg = tile % m_groups;
                const int nt = tile / m_groups;
                const int m0 = (mg * CtaGroup + static_cast<int>(rank)) * kBlockM;
                const uint64_t live_mask = group_live_mask(mg);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (p.keep_in != nullptr && !k_block_live<SwizzleBytes>(live_mask, kb)) continue;
                    if (!mbar_wait_bounded(empty_bar + stage, phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * Smem::kStageBytes;
                    uint8_t* sb = sa + Smem::kStageA;
                    if constexpr (CtaGroup == 2) {
                        // the leader's barrier counts the bytes of both CTAs
                        if (rank == 0) mbar_arrive_expect_tx(full_bar + stage, 2 * Smem::kStageBytes);
                        const uint32_t bar = map_to_cta(smem_u32(full_bar + stage), 0);
                        int n_rows;
                        if constexpr (Epi == EPI_GLU) {
                            n_rows = rank == 0 ? nt * kBRows : p.n / 2 + nt * kBRows;   // values | gates
                        } else {
                            n_rows = nt * BlockN + static_cast<int>(rank) * kBRows;
                        }
                        tma_load_2d_pair(sa, &map_a, bar, kb * kBlockK, m0);
                        tma_load_2d_pair(sb, &map_b, bar, kb * kBlockK, n_rows);
                    } else if constexpr (BSrc == BSRC_TMA) {
                        mbar_arrive_expect_tx(full_bar + stage, Smem::kStageBytes);
                        tma_load_2d(sa, &map_a, full_bar + stage, kb * kBlockK, m0);
                        int n_first, n_second;
                        if constexpr (Epi == EPI_GLU) {
                            n_first = nt * kBHalf;
                            n_second = p.n / 2 + nt * kBHalf;
                        } else {
                            n_first = nt * BlockN;
                            n_second = n_first + kBHalf;
                        }
                        tma_load_2d(sb, &map_b, full_bar + stage, kb * kBlockK, n_first);
                        tma_load_2d(sb + kBHalf * SwizzleBytes, &map_b, full_bar + stage,
                                    kb * kBlockK, n_second);
                    } else {
                        mbar_arrive_expect_tx(full_bar + stage, Smem::kStageA);
                        tma_load_2d(sa, &map_a, full_bar + stage, kb * kBlockK, m0);
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_instr_desc<Kind>(kBlockM * CtaGroup, BlockN);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int tile = worker; tile < num_tiles && ok; tile += workers, ++local) {
                const int mg = tile % m_groups;
                const int buf = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                const uint64_t live_mask = group_live_mask(mg);
                if (!mbar_wait_bounded(tmem_empty_bar + buf, acc_phase ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * BlockN);
                uint32_t accumulate = 0;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (p.keep_in != nullptr && !k_block_live<SwizzleBytes>(live_mask, kb)) continue;
                    if (!mbar_wait_bounded(full_bar + stage, phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + stage * Smem::kStageBytes);
                    const uint32_t sb = sa + Smem::kStageA;
                    const uint64_t desc_a = make_smem_desc<SwizzleBytes>(sa);
                    const uint64_t desc_b = make_smem_desc<SwizzleBytes>(sb);
#pragma unroll
                    for (int j = 0; j < kMmasPerBlock; ++j) {
                        // advance 32 bytes along K inside the swizzle atom: +2 in 16-byte units
                        if constexpr (CtaGroup == 2)
                            tc_mma_pair<Kind>(tmem_d, desc_a + 2u * j, desc_b + 2u * j, idesc, accumulate);
                        else
                            tc_mma<Kind>(tmem_d, desc_a + 2u * j, desc_b + 2u * j, idesc, accumulate);
                        accumulate = 1;
                    }
                    // free the stage (in both CTAs of a pair) once the MMAs retire
                    if constexpr (CtaGroup == 2) {
                        tc_commit_pair(map_to_cta(smem_u32(empty_bar + stage), 0));
                        tc_commit_pair(map_to_cta(smem_u32(empty_bar + stage), 1));
                    } else {
                        tc_commit(empty_bar + stage);
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                if constexpr (CtaGroup == 2) {
                    if (accumulate != 0) {
                        tc_commit_pair(map_to_cta(smem_u32(tmem_full_bar + buf), 0));
                        tc_commit_pair(map_to_cta(smem_u32(tmem_full_bar + buf), 1));
                    } else {
                        mbar_arrive_cluster(map_to_cta(smem_u32(tmem_full_bar + buf), 0));
                        mbar_arrive_cluster(map_to_cta(smem_u32(tmem_full_bar + buf), 1));
                    }
                } else if (accumulate != 0) {
                    tc_commit(tmem_full_bar + buf);
                } else {
                    mbar_arrive(tmem_full_bar + buf);  // no live K block: accumulator unused
                }
            }
        }
    } else if (BSrc == BSRC_W4G128 && warp >= 2 + kEpiWarps) {
        // ------------------------------------- INT4 -> fp16 B-operand producer
        // Thread dq owns row dq of the 128-row B stage: 32 bytes of codes (64 K values) per K
        // block, one fp16 scale per 128 K.  W = f16(code * scale) is written straight into the
        // 128-byte-swizzled layout the MMA descriptor expects (16-byte chunk c of row r lives at
        // chunk c ^ (r & 7)), made visible to the async proxy, then the warp arrives on `full`.
        const int dq = static_cast<int>(threadIdx.x) - 32 * (2 + kEpiWarps);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = worker; tile < num_tiles && ok; tile += workers) {
            const int nt = tile / m_groups;
            const int n = nt * BlockN + dq;
            const bool row_ok = n < p.n;
            const uint8_t* codes = p.w4_codes + static_cast<size_t>(row_ok ? n : 0) * (p.k / 2);
            // software pipeline: the codes and scale of K block kb+1 are in flight while block kb
            // is converted, so the L2 latency is paid once per tile instead of once per block
            uint4 next_raw[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
            float next_scale = 0.0f;
            if (row_ok) {
                const uint4* src = reinterpret_cast<const uint4*>(codes);
                next_raw[0] = src[0];
                next_raw[1] = src[1];
                next_scale = __half2float(p.w4_scales[n]);
            }
            for (int kb = 0; kb < k_blocks; ++kb) {
                uint4 raw[2] = {next_raw[0], next_raw[1]};
                const float scale = next_scale;
                if (row_ok && kb + 1 < k_blocks) {
                    const uint4* src = reinterpret_cast<const uint4*>(codes + (kb + 1) * 32);
                    next_raw[0] = src[0];
                    next_raw[1] = src[1];
                    next_scale = __half2float(p.w4_scales[static_cast<size_t>((kb + 1) / 2) * p.n + n]);
                }
                const bool got = mbar_wait_bounded(empty_bar + stage, phase ^ 1u, abort_flag);
                if (!__all_sync(0xffffffffu, got)) {
                    ok = false;
                    break;
                }
                uint8_t* row_base = smem + stage * Smem::kStageBytes + Smem::kStageA + dq * 128;
                const uint32_t* words = reinterpret_cast<const uint32_t*>(raw);
                const __half2 scale2 = __float2half2_rn(scale);
#pragma unroll
                for (int c = 0; c < 8; ++c) {              // chunk c = K values 8c .. 8c+7 = one code word
                    // nibble n -> fp16 (1024 + (n ^ 8)) by OR-ing the biased nibble into the
                    // mantissa of 1024.0, minus 1032.0 = the signed code, exactly; HMUL2 by the
                    // fp16 group scale then rounds once, i.e. f16(code * scale).
                    const uint32_t wbits = words[c] ^ 0x88888888u;       // two's complement -> offset binary
                    uint32_t h[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // byte j holds codes (2j, 2j+1): low nibble -> low half, high nibble -> high half
                        const uint32_t byte = (wbits >> (8 * j)) & 0xFFu;
                        const uint32_t pair = ((byte & 0x0Fu) | ((byte & 0xF0u) << 12)) | 0x64006400u;
                        const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&pair),
                                                  __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408)));
                        const __half2 w = __hmul2(v, scale2);
                        h[j] = *reinterpret_cast<const uint32_t*>(&w);
                    }
                    *reinterpret_cast<uint4*>(row_base + ((c ^ (dq & 7)) * 16)) = make_uint4(h[0], h[1], h[2], h[3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(full_bar + stage);
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else {
        // ---------------------------------------------------------- epilogue
        const int ew = warp - 2;                 // 0..7
        const int quad = warp % 4;               // TMEM lane quadrant this warp may read
        const int half = ew / 4;                 // which part of the tile's columns
        const int et = static_cast<int>(threadIdx.x) - 64;   // 0 .. 32*kEpiWarps-1
        int local = 0;
        bool ok = true;
        for (int tile = worker; tile < num_tiles && ok; tile += workers, ++local) {
            const int mg = tile % m_groups;
            const int mt = mg * CtaGroup + static_cast<int>(rank);    // this CTA's 128-row tile
            const int nt = tile / m_groups;
            const int buf = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            const int row = mt * kBlockM + quad * 32 + lane;
            const int n0 = Epi == EPI_GLU ? nt * kBHalf : nt * BlockN;   // first output column
            // stage per-column scale / bias for this tile
            epilogue_bar_sync<kEpiWarps>();
            for (int c = et; c < BlockN; c += 32 * kEpiWarps) {
                int src;
                if constexpr (Epi == EPI_GLU) {
                    src = c < kBHalf ? nt * kBHalf + c : p.n / 2 + nt * kBHalf + (c - kBHalf);
                } else {
                    src = nt * BlockN + c;
                }
                const bool in = src < p.n;
                s_col_scale[c] = (p.col_scales != nullptr && in) ? p.col_scales[src] : 1.0f;
                s_bias[c] = (p.bias != nullptr && in) ? p.bias[src] : 0.0f;
            }
            epilogue_bar_sync<kEpiWarps>();

            bool live = true;
            if (p.keep_in != nullptr) {
                // MMAs were issued for this work item iff any K tile of any of its rows is live
                bool any = false;
                for (int t = mg * CtaGroup; t < mg * CtaGroup + CtaGroup && t < m_tiles; ++t) {
                    const uint8_t* krow = p.keep_in + static_cast<size_t>(t) * k_tiles64;
                    for (int i = lane; i < k_tiles64; i += 32) any |= krow[i] != 0;
                }
                live = __any_sync(0xffffffffu, any);
            }

            const bool got = mbar_wait_bounded(tmem_full_bar + buf, acc_phase, abort_flag);
            if (!__all_sync(0xffffffffu, got)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();

            const float rs = p.row_scales != nullptr ? (row < p.m ? p.row_scales[row] : 0.0f)
                                                     : p.row_scale;
            const uint32_t taddr_base = tmem_base + static_cast<uint32_t>(buf * BlockN) +
                                        (static_cast<uint32_t>(quad * 32) << 16);
            const size_t obytes = out_elem_bytes(p.out_type);

            if constexpr (Epi == EPI_LINEAR) {
                constexpr int kChunks = kColsPerWarp / 32;
#pragma unroll 1
                for (int c = 0; c < kChunks; ++c) {
                    const int col_local = half * kColsPerWarp + c * 32;
                    uint32_t r[32];
                    tmem_ld_32x32(taddr_base + col_local, r);
                    tmem_ld_wait();
                    const int col = n0 + col_local;
                    if (row < p.m && col < p.n) {
                        float v[32];
                        const bool zero_row = row >= p.valid_rows;
                        uint4 res_raw[4];
                        if (p.residual != nullptr) {
                            const uint4* rp = reinterpret_cast<const uint4*>(
                                p.residual + static_cast<size_t>(row) * p.ld_res + col);
#pragma unroll
                            for (int i = 0; i < 4; ++i) res_raw[i] = rp[i];
                        }
                        const __half* res_h = reinterpret_cast<const __half*>(res_raw);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            float x = live ? acc_to_float<Kind>(r[j]) : 0.0f;
                            x = x * rs * s_col_scale[col_local + j] + s_bias[col_local + j];
                            if (p.act == ACT_SILU) x = silu_f(x);
                            else if (p.act == ACT_RELU) x = fmaxf(x, 0.0f);
                            if (p.residual != nullptr) x = fmaf(p.alpha, x, __half2float(res_h[j]));
                            else x *= p.alpha;
                            v[j] = zero_row ? 0.0f : x;
                        }
                        uint8_t* out_row = reinterpret_cast<uint8_t*>(p.out) +
                            (static_cast<size_t>(row) * p.ld_out + col) * obytes;
                        store_chunk(out_row, p.out_type, p.out_scale, v);
                    }
                }
            } else if constexpr (Epi == EPI_GLU) {
                // columns [0, BlockN/2) hold values, [BlockN/2, BlockN) their gates
                constexpr int kChunks = BlockN / 4 / 32;
                static_assert(kChunks >= 1, "GLU needs BlockN >= 128");
#pragma unroll 1
                for (int c = 0; c < kChunks; ++c) {
                    const int col_local = half * (BlockN / 4) + c * 32;
                    uint32_t rv[32], rg[32];
                    tmem_ld_32x32(taddr_base + col_local, rv);
                    tmem_ld_32x32(taddr_base + kBHalf + col_local, rg);
                    tmem_ld_wait();
                    const int col = n0 + col_local;
                    if (row < p.m && col < p.n / 2) {
                        float v[32];
                        const bool zero_row = row >= p.valid_rows;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float value = round_f16(acc_to_float<Kind>(rv[j]) * rs *
                                                          s_col_scale[col_local + j]);
                            const float gate = round_f16(acc_to_float<Kind>(rg[j]) * rs *
                                                         s_col_scale[kBHalf + col_local + j]);
                            v[j] = zero_row ? 0.0f : __fdividef(value, 1.0f + __expf(-gate));
                        }
                        uint8_t* out_row = reinterpret_cast<uint8_t*>(p.out) +
                            (static_cast<size_t>(row) * p.ld_out + col) * obytes;
                        store_chunk(out_row, p.out_type, p.out_scale, v);
                    }
                }
            } else {
                // EPI_SPARSE_OUT: SiLU, per-(128 x 64) tile max|a| against tau, INT8 store.
                // Kept lean (about 8 instructions per element) because with K = 1024 the MMAs of
                // a tile take only ~4k cycles: SiLU(x) = x/2 * (1 + tanh(x/2)) costs one MUFU
                // (tanh.approx), the x32 of the INT8 encoding is folded into the same FMA, the
                // codes are produced in the first pass and held packed (32 registers).
                static_assert(Epi != EPI_SPARSE_OUT || BlockN == 256, "sparse-out uses BlockN 256");
                constexpr int kChunks = BlockN / 2 / 32;     // 4 chunks = two 64-wide tiles
                uint32_t q[kChunks][8];                       // INT8 codes, 4 per register
                float tile_max[2] = {0.0f, 0.0f};             // max |a * out_scale|
                const bool row_live = row < p.valid_rows && row < p.m;
                const float half_scale = 0.5f * p.out_scale;
#pragma unroll
                for (int c = 0; c < kChunks; ++c) {
                    const int col_local = half * (BlockN / 2) + c * 32;
                    uint32_t r[32];
                    tmem_ld_32x32(taddr_base + col_local, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        int code[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float x = acc_to_float<Kind>(r[j + e]) * (rs * s_col_scale[col_local + j + e]);
                            float th;
                            asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * x));
                            const float xs = x * half_scale;
                            float a = fmaf(xs, th, xs);          // SiLU(x) * out_scale
                            a = row_live ? a : 0.0f;
                            tile_max[c / 2] = fmaxf(tile_max[c / 2], fabsf(a));
                            // SiLU >= -0.279, so saturation at -128 is never reached: +-127 clamp holds
                            asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(code[e]) : "f"(a));
                        }
                        q[c][j / 4] = (code[0] & 255) | ((code[1] & 255) << 8) | ((code[2] & 255) << 16) |
                                      (static_cast<uint32_t>(code[3]) << 24);
                    }
                }
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    float mx = tile_max[t];
#pragma unroll
                    for (int off = 16; off > 0; off /= 2)
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
                    tile_max[t] = mx;
                }
                if (lane == 0) {
                    s_reduce[ew * 2 + 0] = tile_max[0];
                    s_reduce[ew * 2 + 1] = tile_max[1];
                }
                epilogue_bar_sync<kEpiWarps>();
                bool keep[2];
                const int n_tiles64 = p.n / 64;
                const float inv_out_scale = 1.0f / p.out_scale;
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    float mx = 0.0f;
#pragma unroll
                    for (int qd = 0; qd < 4; ++qd) mx = fmaxf(mx, s_reduce[(half * 4 + qd) * 2 + t]);
                    mx *= inv_out_scale;                        // statistic in activation units
                    keep[t] = mx >= p.tau;
                    const int tile64 = (n0 + half * (BlockN / 2)) / 64 + t;
                    if (quad == 0 && lane == 0 && tile64 < n_tiles64 && mt < m_tiles) {
                        p.keep_out[static_cast<size_t>(mt) * n_tiles64 + tile64] = keep[t] ? 1 : 0;
                        if (p.stats_out != nullptr)
                            p.stats_out[static_cast<size_t>(mt) * n_tiles64 + tile64] = mx;
                    }
                }
                if (row < p.m) {
#pragma unroll
                    for (int c = 0; c < kChunks; ++c) {
                        const int col = n0 + half * (BlockN / 2) + c * 32;
                        if (col >= p.n) continue;
                        uint4* dst = reinterpret_cast<uint4*>(
                            reinterpret_cast<uint8_t*>(p.out) + static_cast<size_t>(row) * p.ld_out + col);
                        const bool k = keep[c / 2];
                        dst[0] = k ? make_uint4(q[c][0], q[c][1], q[c][2], q[c][3]) : make_uint4(0, 0, 0, 0);
                        dst[1] = k ? make_uint4(q[c][4], q[c][5], q[c][6], q[c][7]) : make_uint4(0, 0, 0, 0);
                    }
                }
            }
            // release the accumulator buffer
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if constexpr (CtaGroup == 2) mbar_arrive_cluster(map_to_cta(smem_u32(tmem_empty_bar + buf), 0));
                else mbar_arrive(tmem_empty_bar + buf);
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    if (*abort_flag != 0) {
        // give copies / MMAs still in flight time to land before shared memory
        // and tensor memory are released
        const uint64_t start = global_timer_ns();
        while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
        if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, 1);
    }
    tc_fence_before_sync();
    __syncthreads();
    // a pair leaves together: the peer's shared and tensor memory stay valid until the
    // leader's last MMA and every remote arrive have landed
    if constexpr (CtaGroup == 2) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        if constexpr (CtaGroup == 2) tmem_dealloc_pair(tmem_base, kTmemCols);
        else tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace pk100
