// Host side of pk100_gemm: argument validation, TMA tensor-map encoding and the
// dispatch table over (operand kind, tile width, swizzle, epilogue family).
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>

#include "gemm_sm100.cuh"
#include "pk100_internal.h"

namespace pk100 {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
                cudaSuccess && qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        }
    });
    return fn;
}

// Descriptor cache.  A tensor map is a pure function of (base, element size, extents, leading
// dimension, box, swizzle), and a host that runs the same layers on the same buffers request after
// request asks for the same few hundred maps again and again; encoding one costs a driver call.
// Direct-mapped table keyed by a hash of those fields, guarded by one mutex (launchers are
// thread-compatible, not thread-hot).  The 128-byte maps are copied out, so an evicted entry
// never invalidates a launch already issued.
struct MapKey {
    const void* base; uint64_t rows, cols, ld; int elem_bytes, box_rows, swizzle_bytes;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld &&
               elem_bytes == o.elem_bytes && box_rows == o.box_rows && swizzle_bytes == o.swizzle_bytes;
    }
};
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
constexpr int kMapSlots = 4096;
static MapSlot* g_map_slots = nullptr;
static std::mutex g_map_mutex;
static std::atomic<long long> g_map_hits{0}, g_map_misses{0};

static size_t map_hash(const MapKey& k) {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= (k.rows * 0xC2B2AE3D27D4EB4Full) ^ (k.cols << 17) ^ (k.ld << 29);
    h ^= static_cast<uint64_t>(k.elem_bytes * 31 + k.box_rows * 7 + k.swizzle_bytes);
    h ^= h >> 29;
    return static_cast<size_t>(h * 0xBF58476D1CE4E5B9ull >> 32) % kMapSlots;
}

static int encode_map(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows,
                      uint64_t cols, uint64_t ld, int box_rows, int swizzle_bytes);

// 2-D row-major matrix [rows, cols] with `ld` elements between rows; box =
// [box_rows, swizzle_bytes / elem_bytes] elements, swizzle mode = box width.
static int make_map(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows,
                    uint64_t cols, uint64_t ld, int box_rows, int swizzle_bytes) {
    const MapKey key{base, rows, cols, ld, elem_bytes, box_rows, swizzle_bytes};
    const size_t slot = map_hash(key);
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        if (g_map_slots == nullptr) g_map_slots = new MapSlot[kMapSlots]();
        MapSlot& s = g_map_slots[slot];
        if (s.used && s.key == key) {
            *map = s.map;
            g_map_hits.fetch_add(1, std::memory_order_relaxed);
            return PK100_OK;
        }
    }
    const int rc = encode_map(map, base, elem_bytes, rows, cols, ld, box_rows, swizzle_bytes);
    if (rc != PK100_OK) return rc;
    g_map_misses.fetch_add(1, std::memory_order_relaxed);
    std::lock_guard<std::mutex> lock(g_map_mutex);
    MapSlot& s = g_map_slots[slot];
    s.key = key; s.map = *map; s.used = true;
    return PK100_OK;
}

static int encode_map(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows,
                      uint64_t cols, uint64_t ld, int box_rows, int swizzle_bytes) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return PK100_ERR_DRIVER;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(swizzle_bytes / elem_bytes),
                               static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUtensorMapDataType dtype =
        elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const CUtensorMapSwizzle swz =
        swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    const CUresult res = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box,
                            elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return res == CUDA_SUCCESS ? PK100_OK : PK100_ERR_DRIVER;
}

// Tensor map of the output for the staged TMA store (256-column kernels, 128-column linear kernels): every epilogue
// warp owns 32 rows x (tile columns / 4).  Only slices with 64- or 128-byte rows leave that way
// (their swizzle modes); anything else keeps per-thread stores.  Returns the row bytes or 0.
template <int Epi, int BlockN = 256>
static int make_out_map(CUtensorMap* map, const GemmParams& p) {
    const int out_cols = Epi == EPI_GLU ? p.n / 2 : p.n;
    const int cols_per_warp = (Epi == EPI_GLU ? BlockN / 2 : BlockN) / (GemmWarps<BSRC_TMA>::kEpilogue / 4);
    const int obytes = p.out_type == OUT_F16 ? 2 : (p.out_type == OUT_F32 ? 4 : 1);
    const int row_bytes = cols_per_warp * obytes;
    if (row_bytes != 64 && row_bytes != 128) return 0;
    if (BlockN == 128 && row_bytes != 64) return 0;      // its staging holds 64-byte rows only
    if ((reinterpret_cast<uintptr_t>(p.out) & 15u) != 0) return 0;
    if ((static_cast<size_t>(p.ld_out) * obytes) % 16 != 0) return 0;
    if (make_map(map, p.out, obytes, p.m, out_cols, p.ld_out, 32, row_bytes) != PK100_OK) return 0;
    return row_bytes;
}

static int sm_count() {
    static int count = 0;
    if (count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
        if (count <= 0) count = 148;
    }
    return count;
}

// CTA pairs (cta_group::2) for the 256-column kernels.  Off by default: on B200 the pair
// path measured 5-15 % slower than one CTA per tile (the peer's B half arrives over the same
// SM ingress as the TMA traffic it saves), so it is kept as a validated alternative.
static std::atomic<int> g_use_pairs{0};
extern "C" void pk100_set_gemm_cta_pairs(int enable) { g_use_pairs.store(enable != 0); }

// Process-wide cap on the persistent CTAs of a GEMM whose own max_ctas is <= 0 (0 = one per SM).
static std::atomic<int> g_dependent_launch{1};
static std::atomic<int> g_cta_cap{0};
extern "C" void pk100_set_gemm_cta_cap(int ctas) { g_cta_cap.store(ctas > 0 ? ctas : 0); }
static int cta_budget(const pk100_gemm_args& a) {
    if (a.max_ctas > 0) return a.max_ctas;
    const int cap = g_cta_cap.load(std::memory_order_relaxed);
    return cap > 0 && cap < sm_count() ? cap : sm_count();
}
extern "C" void pk100_set_dependent_launch(int enable) { g_dependent_launch.store(enable != 0); }
extern "C" void pk100_tensor_map_cache_stats(long long* hits, long long* misses) {
    if (hits != nullptr) *hits = g_map_hits.load(std::memory_order_relaxed);
    if (misses != nullptr) *misses = g_map_misses.load(std::memory_order_relaxed);
}

template <int Kind, int SwizzleBytes, int Epi>
static int launch_pair(const pk100_gemm_args& a, const GemmParams& p_in, cudaStream_t stream) {
    constexpr int BlockN = 256;
    using Smem = GemmSmem<BlockN / 2, SwizzleBytes, BlockN, gemm_store_bytes<Epi, BSRC_TMA, BlockN>()>;
    GemmParams p = p_in;
    auto kernel = gemm_kernel<Kind, BlockN, SwizzleBytes, Epi, BSRC_TMA, 2>;
    static bool configured = false;
    if (!configured) {
        const cudaError_t err = cudaFuncSetAttribute(
            kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal);
        if (err != cudaSuccess) return static_cast<int>(err);
        configured = true;
    }
    constexpr int elem = Kind == KIND_F16 ? 2 : 1;
    CUtensorMap map_a, map_b;
    int rc = make_map(&map_a, a.a, elem, a.m, a.k, a.lda, kBlockM, SwizzleBytes);
    if (rc != PK100_OK) return rc;
    rc = make_map(&map_b, a.b, elem, a.n, a.k, a.ldb, BlockN / 2, SwizzleBytes);
    if (rc != PK100_OK) return rc;
    CUtensorMap map_out = map_a;
    p.store_row_bytes = make_out_map<Epi>(&map_out, p);
    const int m_groups = (a.m + 2 * kBlockM - 1) / (2 * kBlockM);
    const int n_tiles = (p.n + BlockN - 1) / BlockN;
    int pairs = cta_budget(a) / 2;
    if (pairs > m_groups * n_tiles) pairs = m_groups * n_tiles;
    if (pairs < 1) pairs = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(GemmWarps<BSRC_TMA>::kThreads);
    cfg.dynamicSmemBytes = Smem::kTotal;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, map_out, p);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return static_cast<int>(err);
    }
    pk100_count_launch();
    return PK100_OK;
}

template <int Kind, int BlockN, int SwizzleBytes, int Epi>
static int launch(const pk100_gemm_args& a, const GemmParams& p_in, cudaStream_t stream) {
    if constexpr (BlockN == 256) {
        if (g_use_pairs.load() != 0 && a.m > kBlockM) return launch_pair<Kind, SwizzleBytes, Epi>(a, p_in, stream);
    }
    using Smem = GemmSmem<BlockN, SwizzleBytes, BlockN, gemm_store_bytes<Epi, BSRC_TMA, BlockN>()>;
    GemmParams p = p_in;
    auto kernel = gemm_kernel<Kind, BlockN, SwizzleBytes, Epi, BSRC_TMA>;
    static bool configured = false;
    if (!configured) {
        const cudaError_t err = cudaFuncSetAttribute(
            kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal);
        if (err != cudaSuccess) return static_cast<int>(err);
        configured = true;
    }
    constexpr int elem = Kind == KIND_F16 ? 2 : 1;
    CUtensorMap map_a, map_b;
    int rc = make_map(&map_a, a.a, elem, a.m, a.k, a.lda, kBlockM, SwizzleBytes);
    if (rc != PK100_OK) return rc;
    rc = make_map(&map_b, a.b, elem, a.n, a.k, a.ldb, BlockN / 2, SwizzleBytes);
    if (rc != PK100_OK) return rc;
    CUtensorMap map_out = map_a;
    if constexpr (gemm_store_bytes<Epi, BSRC_TMA, BlockN>() > 0) p.store_row_bytes = make_out_map<Epi, BlockN>(&map_out, p);
    const int m_tiles = (a.m + kBlockM - 1) / kBlockM;
    const int n_tiles = (p.n + BlockN - 1) / BlockN;
    int ctas = cta_budget(a);
    if (ctas > m_tiles * n_tiles) ctas = m_tiles * n_tiles;
    pk100_launch_chained(kernel, dim3(ctas), dim3(GemmWarps<BSRC_TMA>::kThreads), Smem::kTotal, stream, map_a, map_b, map_out, p);
    return pk100_launch_status();
}

// fp16 activations x INT4 group-128 weights, dequantised in shared memory by producer warps.
static int launch_w4(const pk100_gemm_args& a, const GemmParams& p, cudaStream_t stream) {
    constexpr int BlockN = 128;
    constexpr int kMTiles = GemmWarps<BSRC_W4G128>::kMTiles;
    using Smem = GemmSmem<BlockN, 128, BlockN * kMTiles, 0, kBlockM * kMTiles>;
    auto kernel = gemm_kernel<KIND_F16, BlockN, 128, EPI_LINEAR, BSRC_W4G128>;
    static bool configured = false;
    if (!configured) {
        const cudaError_t err = cudaFuncSetAttribute(
            kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal);
        if (err != cudaSuccess) return static_cast<int>(err);
        configured = true;
    }
    CUtensorMap map_a;
    const int rc = make_map(&map_a, a.a, 2, a.m, a.k, a.lda, kBlockM, 128);
    if (rc != PK100_OK) return rc;
    const int m_items = (a.m + kBlockM * kMTiles - 1) / (kBlockM * kMTiles);   // 256-row work items
    const int n_tiles = (p.n + BlockN - 1) / BlockN;
    int ctas = cta_budget(a);
    if (ctas > m_items * n_tiles) ctas = m_items * n_tiles;
    // neither B nor the output has a tensor map
    pk100_launch_chained(kernel, dim3(ctas), dim3(GemmWarps<BSRC_W4G128>::kThreads), Smem::kTotal, stream, map_a, map_a, map_a, p);
    return pk100_launch_status();
}

static bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

}  // namespace pk100

using namespace pk100;

int pk100_tensor_map_2d(void* map, const void* base, int elem_bytes, unsigned long long rows,
                        unsigned long long cols, unsigned long long ld, int box_rows, int swizzle_bytes) {
    return make_map(static_cast<CUtensorMap*>(map), base, elem_bytes, rows, cols, ld, box_rows, swizzle_bytes);
}

bool pk100_dependent_launch_enabled() { return pk100::g_dependent_launch.load(std::memory_order_relaxed) != 0; }

static std::atomic<long long> g_launches{0};
void pk100_count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
extern "C" long long pk100_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int pk100_gemm(void* stream_v, const pk100_gemm_args* a) {
    if (a == nullptr || a->a == nullptr || a->b == nullptr || a->out == nullptr) return PK100_ERR_NULL;
    if (a->m < 0 || a->n <= 0 || a->k <= 0) return PK100_ERR_SHAPE;
    if (a->m == 0) return PK100_OK;
    if (a->kind < PK100_KIND_F16 || a->kind > PK100_KIND_F16_W4G128) return PK100_ERR_UNSUPPORTED;
    const bool w4 = a->kind == PK100_KIND_F16_W4G128;
    const int elem = (a->kind == PK100_KIND_F16 || w4) ? 2 : 1;
    if ((static_cast<long long>(a->k) * elem) % 16 != 0 ||
        (static_cast<long long>(a->lda) * elem) % 16 != 0 || a->lda < a->k)
        return PK100_ERR_SHAPE;
    if (!w4 && ((static_cast<long long>(a->ldb) * elem) % 16 != 0 || a->ldb < a->k)) return PK100_ERR_SHAPE;
    if (w4) {
        if (a->b_group_scales == nullptr) return PK100_ERR_NULL;
        if (a->k % 128 != 0 || a->epilogue != PK100_EPI_LINEAR || a->keep_in != nullptr)
            return PK100_ERR_SHAPE;
    }
    if (a->n % 32 != 0) return PK100_ERR_SHAPE;
    if (!aligned16(a->a) || !aligned16(a->b) || !aligned16(a->out)) return PK100_ERR_ALIGN;
    if (a->out_type < PK100_OUT_F16 || a->out_type > PK100_OUT_S8) return PK100_ERR_UNSUPPORTED;
    const int out_elem = a->out_type == PK100_OUT_F16 ? 2 : (a->out_type == PK100_OUT_F32 ? 4 : 1);
    const int out_cols = a->epilogue == PK100_EPI_GLU ? a->n / 2 : a->n;
    if (a->ld_out < out_cols || (static_cast<long long>(a->ld_out) * out_elem) % 16 != 0)
        return PK100_ERR_SHAPE;
    if (a->residual != nullptr) {
        if (!aligned16(a->residual)) return PK100_ERR_ALIGN;
        if (a->ld_res < out_cols || a->ld_res % 8 != 0) return PK100_ERR_SHAPE;
        if (a->epilogue != PK100_EPI_LINEAR) return PK100_ERR_UNSUPPORTED;
    }
    if (a->keep_in != nullptr) {
        if (elem != 1 || a->k % 64 != 0 || a->k > 4096) return PK100_ERR_SHAPE;
    }
    if (a->epilogue == PK100_EPI_GLU && (a->n % 128 != 0)) return PK100_ERR_SHAPE;
    if (a->epilogue == PK100_EPI_SPARSE_OUT) {
        if (a->keep_out == nullptr) return PK100_ERR_NULL;
        if (a->n % 64 != 0 || a->out_type != PK100_OUT_S8) return PK100_ERR_SHAPE;
    }

    GemmParams p{};
    p.m = a->m;
    p.n = a->n;
    p.k = a->k;
    p.row_scales = a->row_scales;
    p.row_scale = a->row_scale;
    p.col_scales = a->col_scales;
    p.bias = a->bias;
    p.act = a->act;
    p.residual = static_cast<const __half*>(a->residual);
    p.ld_res = a->ld_res;
    p.alpha = a->alpha;
    p.valid_rows = a->valid_rows > 0 ? a->valid_rows : a->m;
    p.out = a->out;
    p.ld_out = a->ld_out;
    p.out_type = a->out_type;
    p.out_scale = a->out_scale;
    p.tau = a->tau;
    p.keep_out = a->keep_out;
    p.stats_out = a->stats_out;
    p.keep_in = a->keep_in;
    p.w4_codes = w4 ? static_cast<const uint8_t*>(a->b) : nullptr;
    p.w4_scales = w4 ? static_cast<const __half*>(a->b_group_scales) : nullptr;
    p.status = a->status;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    // Tile width: the one with the shorter schedule, counting whole waves over the CTAs available and a
    // 128-column tile as 0.7 of a 256-column one (measured: at 3072 x 1024 one wave of 96 wide tiles
    // takes 17.6 us against 20.3 us for two waves of 192 narrow ones; at 6144 x 1024 two wide waves
    // take 24.3 us against 28.7 us for three narrow ones; a single partial wave prefers the narrow tile).
    const int m_tiles = (a->m + kBlockM - 1) / kBlockM;
    bool narrow = a->n % 256 != 0;
    if (!narrow) {
        const long long ctas = cta_budget(*a);
        const long long wide = (static_cast<long long>(m_tiles) * (a->n / 256) + ctas - 1) / ctas;
        const long long thin = (static_cast<long long>(m_tiles) * (a->n / 128) + ctas - 1) / ctas;
        narrow = thin * 7 < wide * 10;
    }

    if (w4) return launch_w4(*a, p, stream);
    switch (a->epilogue) {
    case PK100_EPI_LINEAR:
        if (a->kind == PK100_KIND_F16) {
            return narrow ? launch<KIND_F16, 128, 128, EPI_LINEAR>(*a, p, stream)
                          : launch<KIND_F16, 256, 128, EPI_LINEAR>(*a, p, stream);
        }
        if (a->kind == PK100_KIND_E4M3) {
            return narrow ? launch<KIND_F8, 128, 128, EPI_LINEAR>(*a, p, stream)
                          : launch<KIND_F8, 256, 128, EPI_LINEAR>(*a, p, stream);
        }
        // A tile-sparse A operand (keep_in) runs on the same 128-byte K blocks: a block is skipped
        // when both of its 64-wide sparsity tiles are dead (dead tiles hold zeros, so a half-dead
        // block is computed correctly).  64-byte K blocks matched the skip granularity but
        // measured 14 % slower: TMA moves rows of a box at the same rate whatever their width.
        return narrow ? launch<KIND_I8, 128, 128, EPI_LINEAR>(*a, p, stream)
                      : launch<KIND_I8, 256, 128, EPI_LINEAR>(*a, p, stream);
    case PK100_EPI_GLU:
        if (a->kind == PK100_KIND_E4M3) {
            return (a->n % 256 != 0) ? launch<KIND_F8, 128, 128, EPI_GLU>(*a, p, stream)
                                     : launch<KIND_F8, 256, 128, EPI_GLU>(*a, p, stream);
        }
        if (a->kind == PK100_KIND_F16) {
            return (a->n % 256 != 0) ? launch<KIND_F16, 128, 128, EPI_GLU>(*a, p, stream)
                                     : launch<KIND_F16, 256, 128, EPI_GLU>(*a, p, stream);
        }
        return PK100_ERR_UNSUPPORTED;
    case PK100_EPI_SPARSE_OUT:
        if (a->kind == PK100_KIND_E4M3) return launch<KIND_F8, 256, 128, EPI_SPARSE_OUT>(*a, p, stream);
        if (a->kind == PK100_KIND_F16) return launch<KIND_F16, 256, 128, EPI_SPARSE_OUT>(*a, p, stream);
        return PK100_ERR_UNSUPPORTED;
    default:
        return PK100_ERR_UNSUPPORTED;
    }
}
