// Shared between the translation units of libpk100: status codes, enums that are
// also part of the C ABI (see include/pk100.h) and the launch-status helper.
#pragma once

#include <cuda_runtime.h>

#include "../../include/pk100.h"

// Maps the sticky-free launch error of the last kernel launch to the ABI's
// convention: 0 ok, positive = CUDA runtime error code.
// Number of kernels launched through this library by the calling process (monotonic).
extern "C" long long pk100_launch_count(void);
void pk100_count_launch();

static inline int pk100_launch_status() {
    const cudaError_t err = cudaPeekAtLastError();
    if (err == cudaSuccess) {
        pk100_count_launch();
        return PK100_OK;
    }
    cudaGetLastError();   // clear the non-sticky launch error so later calls are not poisoned
    return static_cast<int>(err);
}

// Programmatic dependent launch for the kernels of the per-block chain (LayerNorm, GEMMs,
// attention, depthwise convolution).  Each of them issues griddepcontrol.launch_dependents on
// entry and griddepcontrol.wait before its first access to global memory, so a launch made with
// the attribute below may become resident while its predecessor in the stream drains: the launch
// latency and the prologue (barrier set-up, tensor-memory allocation, descriptor prefetch) leave
// the critical path; the data dependency is still the whole predecessor grid.  On by default;
// pk100_set_dependent_launch(0) restores plain stream order.
bool pk100_dependent_launch_enabled();

template <typename... Params, typename... Args>
static inline void pk100_launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem_bytes,
                                        cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = pk100_dependent_launch_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

// 2-D TMA descriptor of a row-major matrix [rows, cols] (`ld` elements between rows) with a box of
// [box_rows, swizzle_bytes / elem_bytes] elements; served from the library's descriptor cache
// (gemm_host.cu).  `map` points to a CUtensorMap.
int pk100_tensor_map_2d(void* map, const void* base, int elem_bytes, unsigned long long rows,
                        unsigned long long cols, unsigned long long ld, int box_rows, int swizzle_bytes);
