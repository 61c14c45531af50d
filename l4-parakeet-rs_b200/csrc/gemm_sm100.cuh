// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D[M,N] = epilogue( A[M,K] . B[N,K]^T )      A, B row-major ("K-major")
//
// One CTA per SM loops over 128 x BLOCK_N output tiles.
//   warp 0      TMA producer: global -> swizzled shared-memory stage ring
//   warp 1      tcgen05.mma issuer (one elected lane); owns the TMEM allocation
//   warps 2..17 epilogue (16 warps, four per TMEM lane quadrant): tcgen05.ld the fp32/s32
//               accumulator, apply scales / bias / activation / residual / quantisation, store
//               through shared memory and a TMA store (or per thread)
// INT4 group-128 weights: 8 epilogue warps + 8 warps that dequantise the B stage into shared
// memory; a work item is 256 x 128 (two 128-row accumulators share every dequantised B stage).
// Accumulators are double-buffered in TMEM so the MMAs of tile i+1 overlap the epilogue of
// tile i.  All waits are bounded (ptx_sm100.cuh).
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
    // Bytes of one output row in a warp's 32-row slice when the slices leave through shared
    // memory and a TMA store (64 or 128); 0 = each thread stores its row piece directly.
    int store_row_bytes;
};

constexpr int kBlockM = 128;
// Warps per CTA: TMA producer + MMA issuer + epilogue warps (+ 8 dequantisation warps for INT4
// weights).  16 epilogue warps = 4 per TMEM lane quadrant, each a quarter of the tile's
// columns: the epilogue of a K = 1024 tile has to finish within the ~4k cycles its MMAs take.
// INT4 weights: kMTiles = 2 accumulators of 128 rows share each dequantised B stage (the
// conversion, not the MMA, bounds that kernel, so its cost is spread over twice the rows);
// 4 epilogue warps per accumulator, each all 128 columns of its 32 rows.
template <int BSrc>
struct GemmWarps {
    static constexpr int kMTiles = BSrc == BSRC_W4G128 ? 2 : 1;
    static constexpr int kEpilogue = BSrc == BSRC_W4G128 ? 8 : 16;
    static constexpr int kDequant = BSrc == BSRC_W4G128 ? 8 : 0;
    static constexpr int kThreads = 32 * (2 + kEpilogue + kDequant);
};

// Shared memory the epilogue warps stage their output slices in for the TMA store: 32 rows of
// up to 128 bytes per warp (64 bytes for the INT8 sparse-out tiles).  Only the 256-column TMA
// kernels use it.
template <int Epi, int BSrc, int BlockN>
constexpr int gemm_store_bytes() {
    if (BSrc != BSRC_TMA) return 0;
    // 128-column linear tiles: 32 columns per warp, 64-byte rows for fp16 output
    if (BlockN == 128 && Epi == EPI_LINEAR) return GemmWarps<BSrc>::kEpilogue * 32 * 64;
    if (BlockN != 256) return 0;
    return GemmWarps<BSrc>::kEpilogue * 32 * (Epi == EPI_SPARSE_OUT ? 64 : 128);
}

// BRows = B rows staged per CTA per stage, EpiCols = accumulator columns of the tile,
// StoreBytes = output staging for the TMA store.
template <int BRows, int SwizzleBytes, int EpiCols = BRows, int StoreBytes = 0, int ARows = kBlockM>
struct GemmSmem {
    static constexpr int kStageA = ARows * SwizzleBytes;
    static constexpr int kStageB = BRows * SwizzleBytes;
    static constexpr int kStageBytes = kStageA + kStageB;
    // tail: barriers + tmem pointer + abort flag + epilogue staging
    // (each epilogue warp keeps a private slice of column scales and biases: 32 bytes per column)
    // + the tile-skip schedule: one 64-bit live mask and one 16-bit rank per 128-row tile
    static constexpr int kSchedTiles = 512;
    static constexpr int kSchedOffset = 64 * 8 + 16 + 32 * EpiCols + 64 * 4;
    static constexpr int kTailBytes = kSchedOffset + kSchedTiles * (8 + 2);
    static constexpr int kStoreBytes = StoreBytes;
    // 227 KB per CTA, less the tail, the output staging and 1 KB of alignment slack; the
    // pipeline is not depth-sensitive (2 and 4 stages measured alike), so staging comes first
    static constexpr int kBudget = 227 * 1024 - 1024 - kTailBytes - kStoreBytes;
    static constexpr int kStagesRaw = kBudget / kStageBytes;
    static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
    static_assert(kStages >= 2, "at least a double-buffered operand pipeline");
    static constexpr int kTileBytes = kStages * kStageBytes;
    static constexpr int kTotal = kTileBytes + kStoreBytes + kTailBytes + 1024;
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

// Encode 16 consecutive output columns of one row (fp16: two 16-byte chunks, E4M3 / INT8: one).
__device__ __forceinline__ int pack_piece(int out_type, float out_scale, const float (&v)[16],
                                          uint4 (&w)[2]) {
    if (out_type == OUT_F16) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            w[i] = make_uint4(pack_half2(v[8 * i + 0], v[8 * i + 1]), pack_half2(v[8 * i + 2], v[8 * i + 3]),
                              pack_half2(v[8 * i + 4], v[8 * i + 5]), pack_half2(v[8 * i + 6], v[8 * i + 7]));
        }
        return 2;
    }
    uint32_t q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int b = 4 * j;
        const float a0 = round_f16(v[b]) * out_scale, a1 = round_f16(v[b + 1]) * out_scale;
        const float a2 = round_f16(v[b + 2]) * out_scale, a3 = round_f16(v[b + 3]) * out_scale;
        q[j] = out_type == OUT_E4M3 ? pack_e4m3x4(a0, a1, a2, a3) : pack_s8x4(a0, a1, a2, a3);
    }
    w[0] = make_uint4(q[0], q[1], q[2], q[3]);
    return 1;
}

// Store 16 consecutive output columns of one row straight to global memory.
__device__ __forceinline__ void store_piece(void* out_row, int out_type, float out_scale,
                                            const float (&v)[16]) {
    if (out_type == OUT_F32) {
        float4* dst = reinterpret_cast<float4*>(out_row);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
        return;
    }
    uint4 w[2];
    const int chunks = pack_piece(out_type, out_scale, v, w);
    uint4* dst = reinterpret_cast<uint4*>(out_row);
    dst[0] = w[0];
    if (chunks == 2) dst[1] = w[1];
}

// Put 16 consecutive output columns (piece `piece` of the warp's slice) into this lane's row
// of the staging slice.  16-byte chunks are XOR-swizzled with `swz`, the pattern of the TMA
// store's tensor map (64-byte rows: (row >> 1) & 3, 128-byte rows: row & 7).
__device__ __forceinline__ void stage_piece(uint8_t* stage_row, int piece, int swz, int out_type,
                                            float out_scale, const float (&v)[16]) {
    uint4 w[2];
    const int chunks = pack_piece(out_type, out_scale, v, w);
    if (chunks == 2) {
        *reinterpret_cast<uint4*>(stage_row + (((2 * piece) ^ swz) << 4)) = w[0];
        *reinterpret_cast<uint4*>(stage_row + (((2 * piece + 1) ^ swz) << 4)) = w[1];
    } else {
        *reinterpret_cast<uint4*>(stage_row + ((piece ^ swz) << 4)) = w[0];
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

// The same mask from 16-byte loads (`fetch`) compressed to bits (`mask`): one thread per 128-row
// tile fills the CTA's shared-memory copy of the bitmap with it when the kernel starts.
struct LiveMaskRow {
    uint4 w[4];          // up to 64 flag bytes
    bool vector;
    __device__ __forceinline__ void fetch(const uint8_t* keep_in, int mt, int k_tiles64) {
        vector = false;
        if (keep_in == nullptr) return;
        const uint8_t* row = keep_in + static_cast<size_t>(mt) * k_tiles64;
        if (k_tiles64 % 16 == 0 && (reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
            vector = true;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                w[i] = 16 * i < k_tiles64 ? __ldg(reinterpret_cast<const uint4*>(row) + i) : make_uint4(0, 0, 0, 0);
        }
    }
    // bit i of the result = byte i of a 4-byte word is non-zero
    static __device__ __forceinline__ uint32_t nonzero_bytes(uint32_t x) {
        const uint32_t t = (((x & 0x7f7f7f7fu) + 0x7f7f7f7fu) | x) & 0x80808080u;   // 0x80 per non-zero byte
        return ((t >> 7) * 0x00204081u >> 21) & 0xFu;                              // gather the four flags
    }
    __device__ __forceinline__ uint64_t mask(const uint8_t* keep_in, int mt, int k_tiles64) const {
        if (keep_in == nullptr) return ~0ull;
        if (!vector) return load_live_mask(keep_in, mt, k_tiles64);
        uint64_t m = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t words[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
                m |= static_cast<uint64_t>(nonzero_bytes(words[j])) << (16 * i + 4 * j);
        }
        return m;
    }
};

// Is K block `kb` (SwizzleBytes wide, 8-bit elements) live?
template <int SwizzleBytes>
__device__ __forceinline__ bool k_block_live(uint64_t mask, int kb) {
    if constexpr (SwizzleBytes == 64) {
        return (mask >> kb) & 1ull;
    } else {
        return ((mask >> (2 * kb)) & 3ull) != 0;
    }
}

// Number of live K blocks in a tile's mask.
template <int SwizzleBytes>
__device__ __forceinline__ int live_k_blocks(uint64_t mask) {
    if constexpr (SwizzleBytes == 64) {
        return __popcll(mask);
    } else {
        return __popcll((mask | (mask >> 1)) & 0x5555555555555555ull);
    }
}

// CtaGroup = 2: the CTAs of a 2-CTA cluster share one 256 x BlockN tile (tcgen05 cta_group::2).
// Each CTA stages its own 128 rows of A and BlockN/2 rows of B, so a tile costs 2/3 of the
// operand traffic of two independent 128 x BlockN tiles; the even CTA issues the MMAs, each CTA
// runs the epilogue of its own 128 accumulator rows.
template <int Kind, int BlockN, int SwizzleBytes, int Epi, int BSrc, int CtaGroup = 1>
__global__ void __launch_bounds__(GemmWarps<BSrc>::kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const __grid_constant__ CUtensorMap map_out,
            const GemmParams p) {
    static_assert(CtaGroup == 1 || (CtaGroup == 2 && BlockN == 256 && BSrc == BSRC_TMA), "pairs: 256 columns, TMA");
    constexpr int kBRows = BlockN / CtaGroup;               // B rows staged by this CTA
    constexpr int kMTiles = GemmWarps<BSrc>::kMTiles;       // 128-row accumulators per work item
    using Smem = GemmSmem<kBRows, SwizzleBytes, BlockN * kMTiles, gemm_store_bytes<Epi, BSrc, BlockN>(),
                          kBlockM * kMTiles>;
    constexpr int kStages = Smem::kStages;
    constexpr int kElemBytes = Kind == KIND_F16 ? 2 : 1;
    constexpr int kBlockK = SwizzleBytes / kElemBytes;       // elements per K block
    constexpr int kMmasPerBlock = SwizzleBytes / 32;         // 32 bytes of K per MMA
    constexpr uint32_t kTmemCols = 2 * kMTiles * BlockN;
    constexpr int kBHalf = BlockN / 2;                       // rows per B load
    static_assert(BlockN == 64 || BlockN == 128 || BlockN == 256, "BlockN");
    static_assert(BSrc == BSRC_TMA || (Kind == KIND_F16 && SwizzleBytes == 128 && BlockN == 128 &&
                                       Epi == EPI_LINEAR), "w4: fp16 MMA, 128-column tiles, linear epilogue");
    // 16 epilogue warps, four per TMEM lane quadrant, each a quarter of the tile's columns; INT4
    // weights: 8 epilogue warps, four per 128-row accumulator, + 8 dequantisation warps.
    constexpr int kEpiWarps = GemmWarps<BSrc>::kEpilogue;
    constexpr int kParts = kEpiWarps / 4 / kMTiles;          // column slices of one accumulator
    constexpr int kOutCols = Epi == EPI_GLU ? BlockN / 2 : BlockN;   // output columns of a tile
    constexpr int kColsPerWarp = kOutCols / kParts;
    static_assert(kColsPerWarp % 16 == 0, "each epilogue warp owns whole 16-column pieces");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* store_smem = smem + Smem::kTileBytes;            // 1 KB aligned: stage sizes are
    uint8_t* tail = store_smem + Smem::kStoreBytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
    uint64_t* empty_bar = full_bar + kStages;
    uint64_t* tmem_full_bar = empty_bar + kStages;
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;
    uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(tail + 64 * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 64 * 8 + 8);
    float* s_cols = reinterpret_cast<float*>(tail + 64 * 8 + 16);   // per-warp scale / bias slices
    float* s_reduce = s_cols + kEpiWarps * 2 * (BlockN / kParts);   // one float per epilogue warp
    uint64_t* s_live = reinterpret_cast<uint64_t*>(tail + Smem::kSchedOffset);   // live mask per 128-row tile
    uint16_t* s_order = reinterpret_cast<uint16_t*>(s_live + Smem::kSchedTiles);  // tiles, most live K blocks first

    const int warp = static_cast<int>(threadIdx.x) / 32;
    const int lane = static_cast<int>(threadIdx.x) % 32;

    const uint32_t rank = CtaGroup == 2 ? cluster_ctarank() : 0u;   // 0 = leader of the pair
    const int worker = static_cast<int>(blockIdx.x) / CtaGroup;      // pair (or CTA) index
    const int workers = static_cast<int>(gridDim.x) / CtaGroup;
    const int m_tiles = (p.m + kBlockM - 1) / kBlockM;                // 128-row tiles
    constexpr int kItemTiles = CtaGroup * kMTiles;                    // 128-row tiles per work item
    const int m_groups = (m_tiles + kItemTiles - 1) / kItemTiles;
    const int n_tiles = (p.n + BlockN - 1) / BlockN;
    const int num_tiles = m_groups * n_tiles;
    const int k_blocks = (p.k + kBlockK - 1) / kBlockK;
    const int k_tiles64 = p.k / 64;
    // Tile skip with one CTA per 128-row tile: the bitmap is read once into shared memory, and the
    // work items are dealt in order of their live K blocks (most first), forwards in even passes over
    // the CTAs and backwards in odd ones, so the CTA that drew the heaviest item of one pass draws the
    // lightest of the next (tiles differ several-fold in live blocks; dealt round-robin by index the
    // slowest CTA ran 1.45x the mean).
    const bool balanced = CtaGroup == 1 && kMTiles == 1 && p.keep_in != nullptr && m_tiles <= Smem::kSchedTiles;
    // live-K mask of a work item: union over the 128-row tiles it covers
    auto group_live_mask = [&](int mg) {
        if (balanced) return s_live[mg];
        uint64_t mask = load_live_mask(p.keep_in, mg * CtaGroup, k_tiles64);
        if (CtaGroup == 2 && p.keep_in != nullptr && mg * 2 + 1 < m_tiles)
            mask |= load_live_mask(p.keep_in, mg * 2 + 1, k_tiles64);
        return mask;
    };
    // i-th work item of this worker (false: none left)
    auto work_item = [&](int i, int& mg, int& nt) {
        if (balanced) {
            const int pos = i * workers + ((i & 1) ? workers - 1 - worker : worker);
            if (pos >= num_tiles) return false;
            mg = s_order[pos / n_tiles];
            nt = pos % n_tiles;
            return true;
        }
        const int tile = worker + i * workers;
        if (tile >= num_tiles) return false;
        mg = tile % m_groups;
        nt = tile / m_groups;
        return true;
    };

    grid_dependents_launch();
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            // full: one arrive.expect_tx from the TMA lane (+ the dequantisation warps)
            mbar_init(full_bar + s, 1 + GemmWarps<BSrc>::kDequant);
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
    // everything above touched only shared / tensor memory and kernel parameters: under a
    // programmatic dependent launch it overlapped the previous kernel's tail
    grid_dependency_wait();
    if (balanced) {
        for (int t = static_cast<int>(threadIdx.x); t < m_tiles; t += static_cast<int>(blockDim.x)) {
            LiveMaskRow row;
            row.fetch(p.keep_in, t, k_tiles64);
            s_live[t] = row.mask(p.keep_in, t, k_tiles64);
        }
        __syncthreads();
        for (int t = static_cast<int>(threadIdx.x); t < m_tiles; t += static_cast<int>(blockDim.x)) {
            const int mine = live_k_blocks<SwizzleBytes>(s_live[t]);
            int rank_t = 0;
            for (int u = 0; u < m_tiles; ++u) {
                const int other = live_k_blocks<SwizzleBytes>(s_live[u]);
                rank_t += (other > mine || (other == mine && u < t)) ? 1 : 0;
            }
            s_order[rank_t] = static_cast<uint16_t>(t);
        }
        __syncthreads();
    }

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int mg, nt;
            for (int it = 0; ok && work_item(it, mg, nt); ++it) {
                const int m0 = (mg * CtaGroup + static_cast<int>(rank)) * kBlockM * kMTiles;
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
                        // 128-row boxes of A, one per accumulator that has rows
                        const bool second = m0 + kBlockM < p.m;
                        mbar_arrive_expect_tx(full_bar + stage, second ? Smem::kStageA : Smem::kStageA / 2);
                        tma_load_2d(sa, &map_a, full_bar + stage, kb * kBlockK, m0);
                        if (second)
                            tma_load_2d(sa + Smem::kStageA / 2, &map_a, full_bar + stage, kb * kBlockK, m0 + kBlockM);
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
            int mg, nt;
            for (; ok && work_item(local, mg, nt); ++local) {
                const int buf = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                const uint64_t live_mask = group_live_mask(mg);
                if (!mbar_wait_bounded(tmem_empty_bar + buf, acc_phase ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * kMTiles * BlockN);
                [[maybe_unused]] const bool second = (mg * kItemTiles + 1) * kBlockM < p.m;
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
                        if constexpr (kMTiles == 2) {
                            // the second 128 rows of A (16 KB on: 1024 descriptor units) against the same B
                            if (second)
                                tc_mma<Kind>(tmem_d + BlockN, desc_a + 1024u + 2u * j, desc_b + 2u * j, idesc, accumulate);
                        }
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
        // 256 threads: thread dq converts half h = dq / 128 (32 K values = 16 bytes of codes) of
        // row dq % 128 of the 128-row B stage per K block, one fp16 scale per 128 K.
        // W = f16(code * scale) is written straight into the 128-byte-swizzled layout the MMA
        // descriptor expects (16-byte chunk c of row r lives at chunk c ^ (r & 7)), made visible to
        // the async proxy, then the warp arrives on `full`.
        const int dq = static_cast<int>(threadIdx.x) - 32 * (2 + kEpiWarps);
        const int brow = dq & 127;
        const int half = dq >> 7;                 // warp-uniform
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        int mg, nt;
        for (int it = 0; ok && work_item(it, mg, nt); ++it) {
            const int n = nt * BlockN + brow;
            const bool row_ok = n < p.n;
            const uint8_t* codes = p.w4_codes + static_cast<size_t>(row_ok ? n : 0) * (p.k / 2) + half * 16;
            // Software pipeline over groups of 4 K blocks (= one 128-byte line of this row's codes, two
            // scale groups): the next group's codes and scales are in flight while this group is
            // converted, so neither the L2 nor the DRAM latency of the weight stream is exposed.
            uint4 next_raw[4];
            float next_scale[2];
            auto fetch_group = [&](int kg) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    next_raw[j] = (row_ok && kg + j < k_blocks)
                        ? __ldg(reinterpret_cast<const uint4*>(codes + (kg + j) * 32)) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    next_scale[i] = (row_ok && kg + 2 * i < k_blocks)
                        ? __half2float(p.w4_scales[static_cast<size_t>(kg / 2 + i) * p.n + n]) : 0.0f;
            };
            fetch_group(0);
            const __half2 bias2 = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));
            for (int kg = 0; kg < k_blocks && ok; kg += 4) {
                uint4 cur[4];
                float cur_scale[2];
#pragma unroll
                for (int j = 0; j < 4; ++j) cur[j] = next_raw[j];
                cur_scale[0] = next_scale[0];
                cur_scale[1] = next_scale[1];
                if (kg + 4 < k_blocks) fetch_group(kg + 4);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (kg + j >= k_blocks) break;
                    const bool got = mbar_wait_bounded(empty_bar + stage, phase ^ 1u, abort_flag);
                    if (!__all_sync(0xffffffffu, got)) {
                        ok = false;
                        break;
                    }
                    uint8_t* row_base = smem + stage * Smem::kStageBytes + Smem::kStageA + brow * 128;
                    const uint32_t words[4] = {cur[j].x, cur[j].y, cur[j].z, cur[j].w};
                    const __half2 scale2 = __float2half2_rn(cur_scale[j / 2]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {          // chunk c = K values 8c .. 8c+7 = one code word
                        const int c = 4 * half + i;
                        // nibble n -> fp16 (1024 + (n ^ 8)) by OR-ing the biased nibble into the
                        // mantissa of 1024.0, minus 1032.0 = the signed code, exactly; HMUL2 by the
                        // fp16 group scale then rounds once, i.e. f16(code * scale).
                        const uint32_t wbits = words[i] ^ 0x88888888u;   // two's complement -> offset binary
                        // nibbles (e, e + 4) of the word land in the two halves of one register with
                        // one shift and one AND-OR; the byte permutes below put K back in order
                        __half2 v[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t pair = ((wbits >> (4 * e)) & 0x000F000Fu) | 0x64006400u;
                            v[e] = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&pair), bias2), scale2);
                        }
                        const uint32_t* vb = reinterpret_cast<const uint32_t*>(v);
                        uint32_t h[4];
                        h[0] = __byte_perm(vb[0], vb[1], 0x5410);        // K 0, 1
                        h[1] = __byte_perm(vb[2], vb[3], 0x5410);        // K 2, 3
                        h[2] = __byte_perm(vb[0], vb[1], 0x7632);        // K 4, 5
                        h[3] = __byte_perm(vb[2], vb[3], 0x7632);        // K 6, 7
                        *reinterpret_cast<uint4*>(row_base + ((c ^ (brow & 7)) * 16)) = make_uint4(h[0], h[1], h[2], h[3]);
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
        }
    } else {
        // ---------------------------------------------------------- epilogue
        const int ew = warp - 2;                 // 0 .. kEpiWarps-1
        const int quad = warp % 4;               // TMEM lane quadrant this warp may read
        const int sub = (ew / 4) / kParts;       // which 128-row accumulator of the work item
        const int part = (ew / 4) % kParts;      // which slice of its columns
        // Slice of the per-column epilogue constants this warp reads: kSlice scales, then kSlice
        // biases (GLU: value columns first, their gate columns after).  Warp-private, so staging
        // a tile's constants needs no CTA-wide barrier.
        constexpr int kSlice = BlockN / kParts;
        constexpr int kPer = kSlice / 32;
        float* my_scale = s_cols + ew * 2 * kSlice;
        float* my_bias = my_scale + kSlice;
        float pre_s[kPer], pre_b[kPer];
        auto prefetch_cols = [&](int nt_) {
#pragma unroll
            for (int u = 0; u < kPer; ++u) {
                const int i = u * 32 + lane;
                int src;
                if constexpr (Epi == EPI_GLU) {
                    src = i < kColsPerWarp ? nt_ * kBHalf + part * kColsPerWarp + i
                                           : p.n / 2 + nt_ * kBHalf + part * kColsPerWarp + (i - kColsPerWarp);
                } else {
                    src = nt_ * BlockN + part * kColsPerWarp + i;
                }
                const bool in = src < p.n;
                pre_s[u] = (p.col_scales != nullptr && in) ? __ldg(p.col_scales + src) : 1.0f;
                pre_b[u] = (p.bias != nullptr && in) ? __ldg(p.bias + src) : 0.0f;
            }
        };
        int mg, nt;
        if (work_item(0, mg, nt)) prefetch_cols(nt);
        int local = 0;
        bool ok = true;
        for (; ok && work_item(local, mg, nt); ++local) {
            const int mt = (mg * CtaGroup + static_cast<int>(rank)) * kMTiles + sub;   // this warp's 128-row tile
            const int buf = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            const int row = mt * kBlockM + quad * 32 + lane;
            const int n0 = Epi == EPI_GLU ? nt * kBHalf : nt * BlockN;   // first output column
            // this warp's column scales / biases: written from the registers prefetched during
            // the previous tile, then the next tile's are requested
            __syncwarp();
#pragma unroll
            for (int u = 0; u < kPer; ++u) {
                my_scale[u * 32 + lane] = pre_s[u];
                my_bias[u * 32 + lane] = pre_b[u];
            }
            __syncwarp();
            {
                int mg_next, nt_next;
                if (work_item(local + 1, mg_next, nt_next)) prefetch_cols(nt_next);
            }
            const float rs = p.row_scales != nullptr ? (row < p.m ? p.row_scales[row] : 0.0f)
                                                     : p.row_scale;

            bool live = true;
            if (balanced) {
                live = s_live[mt] != 0;
            } else if (p.keep_in != nullptr) {
                // MMAs were issued for this work item iff any K tile of any of its rows is live
                bool any = false;
                for (int t = mg * kItemTiles; t < (mg + 1) * kItemTiles && t < m_tiles; ++t) {
                    const uint8_t* krow = p.keep_in + static_cast<size_t>(t) * k_tiles64;
                    for (int i = lane; i < k_tiles64; i += 32) any |= krow[i] != 0;
                }
                live = __any_sync(0xffffffffu, any);
            }

            // The residual rows of this warp's slice do not depend on the accumulator: the first two
            // pieces are requested before the wait for it and arrive while the MMAs run; each
            // later piece is requested two pieces ahead, into the buffer just consumed.
            constexpr int kPieces = kColsPerWarp / 16;
            constexpr int kAhead = kPieces < 2 ? kPieces : 2;
            [[maybe_unused]] uint4 res_pre[kAhead][2];
            const bool has_residual = Epi == EPI_LINEAR && p.residual != nullptr;
            auto fetch_residual = [&](uint4 (&dst)[2], int c) {
                const int col = n0 + part * kColsPerWarp + c * 16;
                if (has_residual && row < p.m && col < p.n) {
                    const uint4* rp = reinterpret_cast<const uint4*>(
                        p.residual + static_cast<size_t>(row) * p.ld_res + col);
                    dst[0] = rp[0];
                    dst[1] = rp[1];
                }
            };
            if constexpr (Epi == EPI_LINEAR) {
#pragma unroll
                for (int i = 0; i < kAhead; ++i) fetch_residual(res_pre[i], i);
            }

            const bool got = mbar_wait_bounded(tmem_full_bar + buf, acc_phase, abort_flag);
            if (!__all_sync(0xffffffffu, got)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();

            const uint32_t taddr_base = tmem_base + static_cast<uint32_t>((buf * kMTiles + sub) * BlockN) +
                                        (static_cast<uint32_t>(quad * 32) << 16);
            const size_t obytes = out_elem_bytes(p.out_type);

            const bool zero_row = row >= p.valid_rows;
            // Output slice of this warp (32 rows x kColsPerWarp columns): staged in shared memory
            // and written by one TMA store when the host set that up, else stored per thread.
            const bool staged = Smem::kStoreBytes > 0 && p.store_row_bytes != 0;
            uint8_t* stage = store_smem + ew * (Smem::kStoreBytes / kEpiWarps);
            uint8_t* stage_row = stage + lane * p.store_row_bytes;
            const int swz = p.store_row_bytes == 128 ? (lane & 7) : ((lane >> 1) & 3);
            if (staged) {
                if (lane == 0) bulk_wait_read_all();   // the previous tile's store has read the slice
                __syncwarp();
            }
            if constexpr (Epi == EPI_LINEAR) {
#pragma unroll 1
                for (int cg = 0; cg < kPieces; cg += kAhead) {
#pragma unroll
                for (int ci = 0; ci < kAhead; ++ci) {
                    const int c = cg + ci;
                    const int col_local = part * kColsPerWarp + c * 16;
                    uint32_t r[16];
                    tmem_ld_32x16(taddr_base + col_local, r);
                    tmem_ld_wait();
                    const int col = n0 + col_local;
                    if (row < p.m && col < p.n) {
                        // The run-time switches (activation, residual, dead rows) are taken once per
                        // piece, outside the element loops: left inside, every element pays for the
                        // predicated-off SiLU and residual code (22 instructions per element measured).
                        float v[16];
                        const uint4 res_raw[2] = {res_pre[ci][0], res_pre[ci][1]};
                        if (c + kAhead < kPieces) fetch_residual(res_pre[ci], c + kAhead);
                        const float rs_live = live ? rs : 0.0f;
                        if (!live) {              // accumulator never written: any bit pattern
#pragma unroll
                            for (int j = 0; j < 16; ++j) r[j] = 0u;
                        }
#pragma unroll
                        for (int j = 0; j < 16; j += 4) {
                            const float4 cs = *reinterpret_cast<const float4*>(my_scale + c * 16 + j);
                            const float4 bs = *reinterpret_cast<const float4*>(my_bias + c * 16 + j);
                            v[j + 0] = fmaf(acc_to_float<Kind>(r[j + 0]) * rs_live, cs.x, bs.x);
                            v[j + 1] = fmaf(acc_to_float<Kind>(r[j + 1]) * rs_live, cs.y, bs.y);
                            v[j + 2] = fmaf(acc_to_float<Kind>(r[j + 2]) * rs_live, cs.z, bs.z);
                            v[j + 3] = fmaf(acc_to_float<Kind>(r[j + 3]) * rs_live, cs.w, bs.w);
                        }
                        if (p.act == ACT_SILU) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] = silu_f(v[j]);
                        } else if (p.act == ACT_RELU) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] = fmaxf(v[j], 0.0f);
                        }
                        if (has_residual) {
                            const __half2* res_h = reinterpret_cast<const __half2*>(res_raw);
#pragma unroll
                            for (int j = 0; j < 16; j += 2) {
                                const float2 rr = __half22float2(res_h[j / 2]);
                                v[j] = fmaf(p.alpha, v[j], rr.x);
                                v[j + 1] = fmaf(p.alpha, v[j + 1], rr.y);
                            }
                        } else if (p.alpha != 1.0f) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] *= p.alpha;
                        }
                        if (zero_row) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                        }
                        if (staged) {
                            stage_piece(stage_row, c, swz, p.out_type, p.out_scale, v);
                        } else {
                            uint8_t* out_row = reinterpret_cast<uint8_t*>(p.out) +
                                (static_cast<size_t>(row) * p.ld_out + col) * obytes;
                            store_piece(out_row, p.out_type, p.out_scale, v);
                        }
                    }
                }
                }
            } else if constexpr (Epi == EPI_GLU) {
                // accumulator columns [0, BlockN/2) hold values, [BlockN/2, BlockN) their gates
#pragma unroll 1
                for (int c = 0; c < kPieces; ++c) {
                    const int col_local = part * kColsPerWarp + c * 16;
                    uint32_t rv[16], rg[16];
                    tmem_ld_32x16(taddr_base + col_local, rv);
                    tmem_ld_32x16(taddr_base + kBHalf + col_local, rg);
                    tmem_ld_wait();
                    const int col = n0 + col_local;
                    if (row < p.m && col < p.n / 2) {
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float value = round_f16(acc_to_float<Kind>(rv[j]) * rs *
                                                          my_scale[c * 16 + j]);
                            const float gate = round_f16(acc_to_float<Kind>(rg[j]) * rs *
                                                         my_scale[kColsPerWarp + c * 16 + j]);
                            v[j] = zero_row ? 0.0f : __fdividef(value, 1.0f + __expf(-gate));
                        }
                        if (staged) {
                            stage_piece(stage_row, c, swz, p.out_type, p.out_scale, v);
                        } else {
                            uint8_t* out_row = reinterpret_cast<uint8_t*>(p.out) +
                                (static_cast<size_t>(row) * p.ld_out + col) * obytes;
                            store_piece(out_row, p.out_type, p.out_scale, v);
                        }
                    }
                }
            } else {
                // EPI_SPARSE_OUT: SiLU, per-(128 x 64) tile max|a| against tau, INT8 store.
                // Each epilogue warp owns one 64-column sparsity tile of its 32 rows.  Kept lean
                // (about 8 instructions per element) because with K = 1024 the MMAs of a tile take
                // only ~4k cycles: SiLU(x) = x/2 * (1 + tanh(x/2)) costs one MUFU (tanh.approx),
                // the x32 of the INT8 encoding is folded into the same FMA, the codes are produced
                // in the first pass and held packed (16 registers).
                static_assert(Epi != EPI_SPARSE_OUT || (BlockN == 256 && kColsPerWarp == 64),
                              "sparse-out: 256-column tiles, one 64-column tile per warp");
                uint32_t q[kPieces][4];                       // INT8 codes, 4 per register
                float tile_max = 0.0f;                        // max |a * out_scale|
                // a * out_scale = s * (1 + tanh(h)) with s = x/2 * out_scale and h = x/2; rows that
                // must read as zero get a zero row factor
                const float rso = (!zero_row && row < p.m) ? rs * 0.5f * p.out_scale : 0.0f;
                const float inv_out = 1.0f / p.out_scale;
#pragma unroll
                for (int c = 0; c < kPieces; ++c) {
                    uint32_t r[16];
                    tmem_ld_32x16(taddr_base + part * kColsPerWarp + c * 16, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        const float4 cs = *reinterpret_cast<const float4*>(my_scale + c * 16 + j);
                        const float csv[4] = {cs.x, cs.y, cs.z, cs.w};
                        uint32_t bits[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float sv = (acc_to_float<Kind>(r[j + e]) * rso) * csv[e];
                            float th;
                            asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(sv * inv_out));
                            const float a = fmaf(sv, th, sv);
                            tile_max = fmaxf(tile_max, fabsf(a));
                            // round-to-nearest-even INT8 code in the low byte: adding 1.5 * 2^23 leaves
                            // the integer in the mantissa (two's complement for negatives).  SiLU >=
                            // -0.279, so only the upper clamp at 127 can bind.
                            bits[e] = __float_as_uint(fminf(a, 127.0f) + 12582912.0f);
                        }
                        q[c][j / 4] = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040),
                                                  __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
                    }
                }
#pragma unroll
                for (int off = 16; off > 0; off /= 2)
                    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, off));
                // (double-buffered by tile parity: a warp can be a whole tile ahead of its peers)
                float* red = s_reduce + (local & 1) * kEpiWarps;
                if (lane == 0) red[ew] = tile_max;
                // the four warps (one per lane quadrant) that share this 64-column tile
                asm volatile("bar.sync %0, 128;" ::"r"(2 + part) : "memory");
                const int n_tiles64 = p.n / 64;
                float mx = 0.0f;
#pragma unroll
                for (int qd = 0; qd < 4; ++qd) mx = fmaxf(mx, red[part * 4 + qd]);
                mx *= 1.0f / p.out_scale;                       // statistic in activation units
                const bool keep = mx >= p.tau;
                // a kept tile whose largest |a * out_scale| exceeds 127 lost information to the clamp:
                // reported as status bit 3 (value 8), nothing else changes
                if (keep && mx * p.out_scale > 127.0f && quad == 0 && lane == 0 && p.status != nullptr)
                    atomicOr(p.status, 8);
                const int tile64 = n0 / 64 + part;
                if (quad == 0 && lane == 0 && tile64 < n_tiles64 && mt < m_tiles) {
                    p.keep_out[static_cast<size_t>(mt) * n_tiles64 + tile64] = keep ? 1 : 0;
                    if (p.stats_out != nullptr)
                        p.stats_out[static_cast<size_t>(mt) * n_tiles64 + tile64] = mx;
                }
                const int col = n0 + part * kColsPerWarp;
                if (staged) {
#pragma unroll
                    for (int c = 0; c < kPieces; ++c)
                        *reinterpret_cast<uint4*>(stage_row + ((c ^ swz) << 4)) =
                            keep ? make_uint4(q[c][0], q[c][1], q[c][2], q[c][3]) : make_uint4(0, 0, 0, 0);
                } else if (row < p.m && col < p.n) {
                    uint4* dst = reinterpret_cast<uint4*>(
                        reinterpret_cast<uint8_t*>(p.out) + static_cast<size_t>(row) * p.ld_out + col);
#pragma unroll
                    for (int c = 0; c < kPieces; ++c)
                        dst[c] = keep ? make_uint4(q[c][0], q[c][1], q[c][2], q[c][3]) : make_uint4(0, 0, 0, 0);
                }
            }
            if (staged) {
                // generic-proxy writes of the slice -> visible to the TMA engine
                fence_proxy_async_smem();
                __syncwarp();
                const int col0 = n0 + part * kColsPerWarp;
                const int row0 = mt * kBlockM + quad * 32;
                if (lane == 0 && row0 < p.m && col0 < (Epi == EPI_GLU ? p.n / 2 : p.n)) {
                    tma_store_2d(&map_out, stage, col0, row0);
                    bulk_commit_group();
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
        if (lane == 0) bulk_wait_all();   // this warp's TMA stores have landed
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
