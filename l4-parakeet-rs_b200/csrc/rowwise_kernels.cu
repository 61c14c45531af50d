// Memory-bound row-wise operators of the FastConformer block for sm_100a:
// LayerNorm (+ fused quantisers), activation / weight quantisers, masked GLU,
// depthwise conv + BatchNorm + SiLU (+ fused per-row E4M3 packing).
// One warp owns one 1024-wide row: 16-byte vector loads, the row stays in
// registers between the statistics passes, reductions are warp shuffles.
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "pk100_internal.h"
#include "ptx_sm100.cuh"

namespace pk100 {

constexpr int kWidth = 1024;

__device__ __forceinline__ float warp_sum_all(float v) {
#pragma unroll
    for (int off = 16; off > 0; off /= 2) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ float warp_max_all(float v) {
#pragma unroll
    for (int off = 16; off > 0; off /= 2) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 p = __half22float2(h[i]);
        f[2 * i] = p.x;
        f[2 * i + 1] = p.y;
    }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 raw;
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return raw;
}

__device__ __forceinline__ uint2 e4m3x8(const float (&f)[8]) {
    uint2 out;
    out.x = __nv_cvt_float2_to_fp8x2(make_float2(f[0], f[1]), __NV_SATFINITE, __NV_E4M3) |
            (static_cast<uint32_t>(
                 __nv_cvt_float2_to_fp8x2(make_float2(f[2], f[3]), __NV_SATFINITE, __NV_E4M3)) << 16);
    out.y = __nv_cvt_float2_to_fp8x2(make_float2(f[4], f[5]), __NV_SATFINITE, __NV_E4M3) |
            (static_cast<uint32_t>(
                 __nv_cvt_float2_to_fp8x2(make_float2(f[6], f[7]), __NV_SATFINITE, __NV_E4M3)) << 16);
    return out;
}

__device__ __forceinline__ int clamp_s8(float v) { return max(-127, min(127, __float2int_rn(v))); }

__device__ __forceinline__ uint2 s8x8(const float (&f)[8]) {
    uint2 out;
    out.x = (clamp_s8(f[0]) & 255) | ((clamp_s8(f[1]) & 255) << 8) | ((clamp_s8(f[2]) & 255) << 16) |
            ((clamp_s8(f[3]) & 255) << 24);
    out.y = (clamp_s8(f[4]) & 255) | ((clamp_s8(f[5]) & 255) << 8) | ((clamp_s8(f[6]) & 255) << 16) |
            ((clamp_s8(f[7]) & 255) << 24);
    return out;
}

// Row geometry of a batch of utterances concatenated along the row axis:
// segment s owns rows [s*seg_stride, (s+1)*seg_stride); its first `valid` rows
// carry data (seg_valid[s] when given, else the uniform `valid_rows`).
__device__ __forceinline__ int segment_valid(const int* seg_valid, int seg, int valid_rows) {
    return seg_valid != nullptr ? seg_valid[seg] : valid_rows;
}

// ------------------------------------------------------------- LayerNorm
// Normalise one row held as 4 x 8 values per lane; returns f16-rounded values.
__device__ __forceinline__ void normalise_row(float (&x)[4][8], const __half* gamma,
                                              const __half* beta, int lane, float eps) {
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += x[i][j];
    const float mean = warp_sum_all(sum) * (1.0f / kWidth);
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float d = x[i][j] - mean;
            sq = fmaf(d, d, sq);
        }
    const float rstd = rsqrtf(warp_sum_all(sq) * (1.0f / kWidth) + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int col = i * 256 + lane * 8;
        float g[8], b[8];
        unpack8(*reinterpret_cast<const uint4*>(gamma + col), g);
        unpack8(*reinterpret_cast<const uint4*>(beta + col), b);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            x[i][j] = __half2float(__float2half_rn((x[i][j] - mean) * rstd * g[j] + b[j]));
    }
}

// Write one normalised row in the requested encoding.
__device__ __forceinline__ void emit_row(const float (&x)[4][8], int mode, float inv_scale,
                                         void* out, float* scales, size_t row, int lane) {
    if (mode == PK100_LN_F16) {
        __half* o = reinterpret_cast<__half*>(out) + row * kWidth;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint4*>(o + i * 256 + lane * 8) = pack8(x[i]);
        return;
    }
    uint8_t* o = reinterpret_cast<uint8_t*>(out) + row * kWidth;
    float mult = inv_scale;
    bool divide = false;
    float scale = 1.0f;
    if (mode == PK100_LN_S4_ROW) {
        // every signed 4-bit code is used: the scale is the larger of max/7 and -min/8
        float mx = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fmaxf(__fdiv_rn(x[i][j], 7.0f), __fdiv_rn(-x[i][j], 8.0f)));
        mx = warp_max_all(mx);
        scale = mx > 0.0f ? mx : 1.0f;
        if (lane == 0) scales[row] = scale;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t w[2] = {0u, 0u};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int q = max(-8, min(7, __float2int_rn(__fdiv_rn(x[i][j], scale))));
                w[j / 4] |= static_cast<uint32_t>(q & 255) << (8 * (j % 4));
            }
            *reinterpret_cast<uint2*>(o + i * 256 + lane * 8) = make_uint2(w[0], w[1]);
        }
        return;
    }
    if (mode == PK100_LN_E4M3_ROW || mode == PK100_LN_S8_ROW) {
        float mx = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(x[i][j]));
        mx = warp_max_all(mx);
        const float top = mode == PK100_LN_E4M3_ROW ? 448.0f : 127.0f;
        scale = mx > 0.0f ? __fdiv_rn(mx, top) : 1.0f;
        if (lane == 0) scales[row] = scale;
        divide = true;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = divide ? __fdiv_rn(x[i][j], scale) : x[i][j] * mult;
        const uint2 bytes = (mode == PK100_LN_S8_ROW) ? s8x8(q) : e4m3x8(q);
        *reinterpret_cast<uint2*>(o + i * 256 + lane * 8) = bytes;
    }
}

__device__ __forceinline__ void emit_zero_row(int mode, void* out, float* scales, size_t row,
                                              int lane) {
    if (mode == PK100_LN_F16) {
        __half* o = reinterpret_cast<__half*>(out) + row * kWidth;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint4*>(o + i * 256 + lane * 8) = make_uint4(0, 0, 0, 0);
    } else {
        uint8_t* o = reinterpret_cast<uint8_t*>(out) + row * kWidth;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint2*>(o + i * 256 + lane * 8) = make_uint2(0, 0);
        if (scales != nullptr && lane == 0) scales[row] = 1.0f;
    }
}

// mode / second_mode: PK100_LN_*.  When gamma2 != nullptr a second LayerNorm is
// applied to the f16-rounded first result and written to out2 (the "pair" form:
// block-output norm + next block's first norm in one pass over the row).
__global__ void __launch_bounds__(256)
layer_norm_kernel(const __half* __restrict__ in, const __half* __restrict__ gamma,
                  const __half* __restrict__ beta, void* __restrict__ out, float* scales,
                  int mode, float inv_scale, const __half* __restrict__ gamma2,
                  const __half* __restrict__ beta2, void* __restrict__ out2, float* scales2,
                  int mode2, float inv_scale2, int total_rows, int seg_stride, int valid_rows,
                  const int* __restrict__ seg_valid, float eps) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int lane = threadIdx.x % 32;
    const int row = blockIdx.x * 8 + threadIdx.x / 32;
    if (row >= total_rows) return;
    const int seg = row / seg_stride;
    const int local = row - seg * seg_stride;
    if (local >= segment_valid(seg_valid, seg, valid_rows)) {
        emit_zero_row(mode, out, scales, row, lane);
        if (gamma2 != nullptr) emit_zero_row(mode2, out2, scales2, row, lane);
        return;
    }
    float x[4][8];
    const __half* src = in + static_cast<size_t>(row) * kWidth;
#pragma unroll
    for (int i = 0; i < 4; ++i)
        unpack8(*reinterpret_cast<const uint4*>(src + i * 256 + lane * 8), x[i]);
    normalise_row(x, gamma, beta, lane, eps);
    emit_row(x, mode, inv_scale, out, scales, row, lane);
    if (gamma2 != nullptr) {
        normalise_row(x, gamma2, beta2, lane, eps);
        emit_row(x, mode2, inv_scale2, out2, scales2, row, lane);
    }
}

// ------------------------------------------------- 2:4 structured sparsity of E4M3 activations
// The reference's FF2 input format (kernels/sm89/encoder.cu:685-704, :1037-1054): per four
// consecutive bytes the two largest 7-bit magnitudes are kept, ties to the lower index.
// Returns the two kept bytes (low 16 bits, index order) and their 2-bit indices (bits 16-19).
__device__ __forceinline__ uint32_t compress_quartet(uint32_t packed) {
    uint32_t data = 0, meta = 0;
    int count = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t mag = (packed >> (8 * i)) & 127u;
        int rank = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t other = (packed >> (8 * j)) & 127u;
            rank += (other > mag || (other == mag && j < i)) ? 1 : 0;
        }
        if (rank < 2) {
            data |= ((packed >> (8 * i)) & 255u) << (8 * count);
            meta |= static_cast<uint32_t>(i) << (2 * count);
            ++count;
        }
    }
    return data | (meta << 16);
}

__device__ __forceinline__ uint32_t expand_quartet(uint32_t two_bytes, uint32_t meta4) {
    return ((two_bytes & 255u) << (8 * (meta4 & 3u))) | (((two_bytes >> 8) & 255u) << (8 * ((meta4 >> 2) & 3u)));
}

// mode 0: dense -> dense with the dropped bytes zeroed; 1: dense -> data [rows, cols/2] + metadata
// [rows, cols/8] behind it; 2: that layout -> dense.  One thread per 16 dense bytes (4 quartets).
__global__ void sparse24_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int rows, int cols,
                                int mode) {
    const size_t chunk = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t chunks_per_row = static_cast<size_t>(cols) / 16;
    if (chunk >= chunks_per_row * rows) return;
    const size_t row = chunk / chunks_per_row, c16 = chunk % chunks_per_row;
    const size_t data_bytes = static_cast<size_t>(rows) * (cols / 2);
    if (mode == 2) {
        const uint2 data = *reinterpret_cast<const uint2*>(in + row * (cols / 2) + c16 * 8);
        const uint32_t meta = *reinterpret_cast<const uint16_t*>(in + data_bytes + row * (cols / 8) + c16 * 2);
        uint4 dense;
        dense.x = expand_quartet(data.x & 0xFFFFu, meta & 15u);
        dense.y = expand_quartet(data.x >> 16, (meta >> 4) & 15u);
        dense.z = expand_quartet(data.y & 0xFFFFu, (meta >> 8) & 15u);
        dense.w = expand_quartet(data.y >> 16, (meta >> 12) & 15u);
        *reinterpret_cast<uint4*>(out + row * cols + c16 * 16) = dense;
        return;
    }
    const uint4 v = *reinterpret_cast<const uint4*>(in + row * cols + c16 * 16);
    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
    uint32_t packed[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) packed[i] = compress_quartet(words[i]);
    if (mode == 0) {
        uint4 dense;
        dense.x = expand_quartet(packed[0] & 0xFFFFu, packed[0] >> 16);
        dense.y = expand_quartet(packed[1] & 0xFFFFu, packed[1] >> 16);
        dense.z = expand_quartet(packed[2] & 0xFFFFu, packed[2] >> 16);
        dense.w = expand_quartet(packed[3] & 0xFFFFu, packed[3] >> 16);
        *reinterpret_cast<uint4*>(out + row * cols + c16 * 16) = dense;
    } else {
        uint2 data;
        data.x = (packed[0] & 0xFFFFu) | (packed[1] << 16);
        data.y = (packed[2] & 0xFFFFu) | (packed[3] << 16);
        *reinterpret_cast<uint2*>(out + row * (cols / 2) + c16 * 8) = data;
        const uint32_t meta = (packed[0] >> 16) | ((packed[1] >> 16) << 4) | ((packed[2] >> 16) << 8) |
                              ((packed[3] >> 16) << 12);
        *reinterpret_cast<uint16_t*>(out + data_bytes + row * (cols / 8) + c16 * 2) = static_cast<uint16_t>(meta);
    }
}

// Packed INT4 codes (low nibble = even index, two's complement) -> one INT8 byte per code.
__global__ void unpack_s4_kernel(const uint8_t* __restrict__ packed, int8_t* __restrict__ out, size_t bytes) {
    const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (i + 4 <= bytes) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(packed + i);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int byte = (w >> (8 * b)) & 255;
            const int even = (byte & 15) >= 8 ? (byte & 15) - 16 : (byte & 15);
            const int odd = (byte >> 4) >= 8 ? (byte >> 4) - 16 : (byte >> 4);
            const uint32_t pair = static_cast<uint32_t>(even & 255) | (static_cast<uint32_t>(odd & 255) << 8);
            if (b < 2) lo |= pair << (16 * b); else hi |= pair << (16 * (b - 2));
        }
        *reinterpret_cast<uint2*>(out + 2 * i) = make_uint2(lo, hi);
    } else {
        for (size_t j = i; j < bytes; ++j) {
            const int byte = packed[j];
            out[2 * j] = static_cast<int8_t>((byte & 15) >= 8 ? (byte & 15) - 16 : (byte & 15));
            out[2 * j + 1] = static_cast<int8_t>((byte >> 4) >= 8 ? (byte >> 4) - 16 : (byte >> 4));
        }
    }
}

// ------------------------------------------------------------ quantisers
__global__ void quantize_fixed_kernel(const __half* __restrict__ in, uint8_t* __restrict__ out,
                                      size_t elements, float inv_scale, int to_s8) {
    const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
    if (i + 8 <= elements) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(in + i), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= inv_scale;
        *reinterpret_cast<uint2*>(out + i) = to_s8 ? s8x8(f) : e4m3x8(f);
    } else {
        for (size_t j = i; j < elements; ++j) {
            const float v = __half2float(in[j]) * inv_scale;
            out[j] = to_s8 ? static_cast<uint8_t>(clamp_s8(v) & 255)
                           : static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
        }
    }
}

// Per-row weight packers, run once at load.  One CTA per output row.
// format: 0 E4M3 (absmax/448), 1 S8 (absmax/127), 2 S4 per row (max(v/7,-v/8), -8..7),
//         3 S4 with one fp16 scale per 128 K (absmax/7, -7..7; scales [K/128, N]).
__global__ void __launch_bounds__(256)
pack_weight_rows_kernel(const __half* __restrict__ w, int n, int k, int ldw, int format,
                        uint8_t* __restrict__ out, float* __restrict__ scales,
                        __half* __restrict__ group_scales) {
    __shared__ float s_part[8];
    __shared__ float s_scale;
    const int row = blockIdx.x;
    const int tid = threadIdx.x;
    const __half* src = w + static_cast<size_t>(row) * ldw;
    if (format == 3) {
        // one warp per group of 128
        const int warp = tid / 32, lane = tid % 32;
        for (int g = warp; g < k / 128; g += 8) {
            float v[4];
            float mx = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[j] = __half2float(src[g * 128 + lane * 4 + j]);
                mx = fmaxf(mx, fabsf(v[j]));
            }
            mx = warp_max_all(mx);
            __half s16 = __float2half_rn(mx > 0.0f ? __fdiv_rn(mx, 7.0f) : 1.0f);
            float s = __half2float(s16);
            if (!(s > 0.0f)) { s = 1.0f; s16 = __float2half_rn(1.0f); }
            if (lane == 0) group_scales[static_cast<size_t>(g) * n + row] = s16;
            int q[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) q[j] = max(-7, min(7, __float2int_rn(__fdiv_rn(v[j], s))));
            const uint16_t packed = static_cast<uint16_t>((q[0] & 15) | ((q[1] & 15) << 4) |
                                                          ((q[2] & 15) << 8) | ((q[3] & 15) << 12));
            *reinterpret_cast<uint16_t*>(out + static_cast<size_t>(row) * (k / 2) + g * 64 + lane * 2) =
                packed;
        }
        return;
    }
    float mx = 0.0f;
    for (int c = tid; c < k; c += 256) {
        const float v = __half2float(src[c]);
        mx = fmaxf(mx, format == 2 ? fmaxf(__fdiv_rn(v, 7.0f), __fdiv_rn(-v, 8.0f)) : fabsf(v));
    }
    mx = warp_max_all(mx);
    if (tid % 32 == 0) s_part[tid / 32] = mx;
    __syncthreads();
    if (tid == 0) {
        float m = 0.0f;
        for (int i = 0; i < 8; ++i) m = fmaxf(m, s_part[i]);
        float s;
        if (format == 0) s = m > 0.0f ? __fdiv_rn(m, 448.0f) : 1.0f;
        else if (format == 1) s = m > 0.0f ? __fdiv_rn(m, 127.0f) : 1.0f;
        else s = m > 0.0f ? m : 1.0f;
        s_scale = s;
        scales[row] = s;
    }
    __syncthreads();
    const float s = s_scale;
    if (format == 2) {
        for (int c = tid * 2; c < k; c += 512) {
            const int a = max(-8, min(7, __float2int_rn(__fdiv_rn(__half2float(src[c]), s))));
            const int b = max(-8, min(7, __float2int_rn(__fdiv_rn(__half2float(src[c + 1]), s))));
            out[static_cast<size_t>(row) * (k / 2) + c / 2] =
                static_cast<uint8_t>((a & 15) | ((b & 15) << 4));
        }
    } else {
        for (int c = tid; c < k; c += 256) {
            const float v = __fdiv_rn(__half2float(src[c]), s);
            out[static_cast<size_t>(row) * k + c] = format == 1
                ? static_cast<uint8_t>(clamp_s8(v) & 255)
                : static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
        }
    }
}

// INT4 group-128 codes -> fp16 weights W[n,k] = f16(code * scale[k/128, n]).
__global__ void dequant_w4g128_kernel(const uint8_t* __restrict__ codes,
                                      const __half* __restrict__ group_scales, int n, int k,
                                      __half* __restrict__ out) {
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // byte index
    const size_t total = static_cast<size_t>(n) * (k / 2);
    if (idx >= total) return;
    const int row = static_cast<int>(idx / (k / 2));
    const int kk = static_cast<int>(idx % (k / 2)) * 2;
    const float s = __half2float(group_scales[static_cast<size_t>(kk / 128) * n + row]);
    const uint8_t b = codes[idx];
    int lo = b & 15, hi = b >> 4;
    lo = lo >= 8 ? lo - 16 : lo;
    hi = hi >= 8 ? hi - 16 : hi;
    *reinterpret_cast<__half2*>(out + static_cast<size_t>(row) * k + kk) =
        __floats2half2_rn(static_cast<float>(lo) * s, static_cast<float>(hi) * s);
}

// ------------------------------------------------------------------- GLU
__global__ void glu_masked_kernel(const __half* __restrict__ in, __half* __restrict__ out,
                                  int total_rows, int seg_stride, int valid_rows,
                                  const int* __restrict__ seg_valid) {
    const size_t idx = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
    if (idx >= static_cast<size_t>(total_rows) * kWidth) return;
    const int row = static_cast<int>(idx / kWidth);
    const int col = static_cast<int>(idx % kWidth);
    const int seg = row / seg_stride;
    uint4 result = make_uint4(0, 0, 0, 0);
    if (row - seg * seg_stride < segment_valid(seg_valid, seg, valid_rows)) {
        float a[8], g[8], r[8];
        unpack8(*reinterpret_cast<const uint4*>(in + static_cast<size_t>(row) * 2 * kWidth + col), a);
        unpack8(*reinterpret_cast<const uint4*>(in + static_cast<size_t>(row) * 2 * kWidth + kWidth + col), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = __fdividef(a[j], 1.0f + __expf(-g[j]));
        result = pack8(r);
    }
    *reinterpret_cast<uint4*>(out + idx) = result;
}

// ------------------------------------------------- depthwise + BN + SiLU
// One CTA = 256 threads x 4 channels = all 1024 channels of a strip of 8 rows (short strips:
// 768 CTAs at 6144 rows keep enough loads in flight; the 8 halo rows come from L2).
// A 9-row window of the thread's 4 channels slides down the strip in registers.
constexpr int kDwStrip = 8;

__global__ void __launch_bounds__(256)
depthwise_bn_silu_kernel(const __half* __restrict__ in, const __half* __restrict__ wdw,
                         const float* __restrict__ bn_gamma, const float* __restrict__ bn_beta,
                         const float* __restrict__ bn_mean, const float* __restrict__ bn_var,
                         void* __restrict__ out, float* __restrict__ row_scales, int quantize,
                         int seg_stride, int valid_rows, const int* __restrict__ seg_valid,
                         float eps) {
    __shared__ float s_max[8][8];
    grid_dependents_launch();
    grid_dependency_wait();
    const int tid = threadIdx.x;
    const int lane = tid % 32, warp = tid / 32;
    const int c0 = tid * 4;
    const int strips_per_seg = (seg_stride + kDwStrip - 1) / kDwStrip;
    const int seg = blockIdx.x / strips_per_seg;
    const int r0 = (blockIdx.x % strips_per_seg) * kDwStrip;
    const int rows = segment_valid(seg_valid, seg, valid_rows);
    const size_t base = static_cast<size_t>(seg) * seg_stride;

    // this thread's 4 x 9 taps are 72 contiguous bytes (8-byte aligned): 9 vector loads
    float w[4][9], rstd[4], gam[4], add[4], mean[4];
    {
        __half taps[36];
        const uint2* src = reinterpret_cast<const uint2*>(wdw + static_cast<size_t>(c0) * 9);
#pragma unroll
        for (int i = 0; i < 9; ++i) reinterpret_cast<uint2*>(taps)[i] = __ldg(src + i);
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int t = 0; t < 9; ++t) w[c][t] = __half2float(taps[c * 9 + t]);
        const float4 var = __ldg(reinterpret_cast<const float4*>(bn_var + c0));
        const float4 g4 = __ldg(reinterpret_cast<const float4*>(bn_gamma + c0));
        const float4 b4 = __ldg(reinterpret_cast<const float4*>(bn_beta + c0));
        const float4 m4 = __ldg(reinterpret_cast<const float4*>(bn_mean + c0));
        rstd[0] = rsqrtf(var.x + eps); rstd[1] = rsqrtf(var.y + eps);
        rstd[2] = rsqrtf(var.z + eps); rstd[3] = rsqrtf(var.w + eps);
        gam[0] = g4.x; gam[1] = g4.y; gam[2] = g4.z; gam[3] = g4.w;
        add[0] = b4.x; add[1] = b4.y; add[2] = b4.z; add[3] = b4.w;
        mean[0] = m4.x; mean[1] = m4.y; mean[2] = m4.z; mean[3] = m4.w;
    }

    auto load_row = [&](int r, float (&dst)[4]) {
        if (r >= 0 && r < rows) {
            const uint2 raw = *reinterpret_cast<const uint2*>(in + (base + r) * kWidth + c0);
            const __half2* h = reinterpret_cast<const __half2*>(&raw);
            const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
            dst[0] = a.x; dst[1] = a.y; dst[2] = b.x; dst[3] = b.y;
        } else {
            dst[0] = dst[1] = dst[2] = dst[3] = 0.0f;
        }
    };

    float win[9][4];
#pragma unroll
    for (int t = 0; t < 8; ++t) load_row(r0 - 4 + t, win[t + 1]);   // slots 1..8 = rows r0-4..r0+3

    for (int blk = 0; blk < kDwStrip / 8; ++blk) {
        float y[8][4];
        float mx[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = r0 + blk * 8 + i;
            // slide: drop the oldest row, fetch row r+4
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int c = 0; c < 4; ++c) win[t][c] = win[t + 1][c];
            load_row(r + 4, win[8]);
            mx[i] = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float acc = 0.0f;
#pragma unroll
                for (int t = 0; t < 9; ++t) acc = fmaf(win[t][c], w[c][t], acc);
                float v = (acc - mean[c]) * rstd[c] * gam[c] + add[c];
                v = __fdividef(v, 1.0f + __expf(-v));
                v = __half2float(__float2half_rn(v));
                if (r >= rows) v = 0.0f;
                y[i][c] = v;
                mx[i] = fmaxf(mx[i], fabsf(v));
            }
        }
        if (quantize) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                mx[i] = warp_max_all(mx[i]);
                if (lane == 0) s_max[warp][i] = mx[i];
            }
            __syncthreads();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float m = 0.0f;
#pragma unroll
                for (int q = 0; q < 8; ++q) m = fmaxf(m, s_max[q][i]);
                mx[i] = m;
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = r0 + blk * 8 + i;
            if (r >= seg_stride) continue;
            const size_t grow = base + r;
            if (quantize) {
                const float scale = mx[i] > 0.0f ? __fdiv_rn(mx[i], 448.0f) : 1.0f;
                if (tid == 0) row_scales[grow] = scale;
                const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                    make_float2(__fdiv_rn(y[i][0], scale), __fdiv_rn(y[i][1], scale)),
                    __NV_SATFINITE, __NV_E4M3);
                const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                    make_float2(__fdiv_rn(y[i][2], scale), __fdiv_rn(y[i][3], scale)),
                    __NV_SATFINITE, __NV_E4M3);
                *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(out) + grow * kWidth + c0) =
                    lo | (hi << 16);
            } else {
                uint2 raw;
                __half2* h = reinterpret_cast<__half2*>(&raw);
                h[0] = __floats2half2_rn(y[i][0], y[i][1]);
                h[1] = __floats2half2_rn(y[i][2], y[i][3]);
                *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(out) + grow * kWidth + c0) = raw;
            }
        }
    }
}

}  // namespace pk100

// ------------------------------------------------------------ C-ABI entry
using namespace pk100;

extern "C" int pk100_layer_norm(void* stream, const void* input, const void* gamma,
                                const void* beta, void* output, float* scales, int mode,
                                float inv_scale, int total_rows, int seg_stride, int valid_rows,
                                const int* seg_valid, float eps) {
    if (!input || !gamma || !beta || !output) return PK100_ERR_NULL;
    if (total_rows <= 0) return total_rows == 0 ? PK100_OK : PK100_ERR_SHAPE;
    if (seg_stride <= 0 || mode < 0 || mode > PK100_LN_S4_ROW) return PK100_ERR_SHAPE;
    if (mode >= PK100_LN_E4M3_ROW && !scales) return PK100_ERR_NULL;
    pk100_launch_chained(layer_norm_kernel, dim3((total_rows + 7) / 8), dim3(256), 0, static_cast<cudaStream_t>(stream),
        static_cast<const __half*>(input), static_cast<const __half*>(gamma),
        static_cast<const __half*>(beta), output, scales, mode, inv_scale, nullptr, nullptr,
        nullptr, nullptr, 0, 0.0f, total_rows, seg_stride, valid_rows, seg_valid, eps);
    return pk100_launch_status();
}

extern "C" int pk100_layer_norm_pair(void* stream, const void* input, const void* gamma,
                                     const void* beta, void* output, const void* next_gamma,
                                     const void* next_beta, void* next_output, float* next_scales,
                                     int next_mode, float next_inv_scale, int total_rows,
                                     int seg_stride, int valid_rows, const int* seg_valid,
                                     float eps) {
    if (!input || !gamma || !beta || !output || !next_gamma || !next_beta || !next_output)
        return PK100_ERR_NULL;
    if (total_rows <= 0) return total_rows == 0 ? PK100_OK : PK100_ERR_SHAPE;
    if (seg_stride <= 0 || next_mode < 0 || next_mode > PK100_LN_S4_ROW) return PK100_ERR_SHAPE;
    if (next_mode >= PK100_LN_E4M3_ROW && !next_scales)
        return PK100_ERR_NULL;
    pk100_launch_chained(layer_norm_kernel, dim3((total_rows + 7) / 8), dim3(256), 0, static_cast<cudaStream_t>(stream),
        static_cast<const __half*>(input), static_cast<const __half*>(gamma),
        static_cast<const __half*>(beta), output, nullptr, PK100_LN_F16, 0.0f,
        static_cast<const __half*>(next_gamma), static_cast<const __half*>(next_beta), next_output,
        next_scales, next_mode, next_inv_scale, total_rows, seg_stride, valid_rows, seg_valid, eps);
    return pk100_launch_status();
}

extern "C" int pk100_quantize_fp8_fixed(void* stream, const void* input, void* output,
                                        long long elements, float inverse_scale) {
    if (!input || !output) return PK100_ERR_NULL;
    if (elements <= 0) return elements == 0 ? PK100_OK : PK100_ERR_SHAPE;
    const long long threads = (elements + 7) / 8;
    quantize_fixed_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0,
                            static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(input), static_cast<uint8_t*>(output),
        static_cast<size_t>(elements), inverse_scale, 0);
    return pk100_launch_status();
}

extern "C" int pk100_quantize_int8(void* stream, const void* input, void* output,
                                   float inverse_scale, long long elements) {
    if (!input || !output) return PK100_ERR_NULL;
    if (elements <= 0) return elements == 0 ? PK100_OK : PK100_ERR_SHAPE;
    const long long threads = (elements + 7) / 8;
    quantize_fixed_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0,
                            static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(input), static_cast<uint8_t*>(output),
        static_cast<size_t>(elements), inverse_scale, 1);
    return pk100_launch_status();
}

extern "C" int pk100_pack_weight_rows(void* stream, const void* weight, int n, int k, int ldw,
                                      int format, void* packed, float* scales,
                                      void* group_scales) {
    if (!weight || !packed) return PK100_ERR_NULL;
    if (n <= 0 || k <= 0 || ldw < k || format < 0 || format > 3) return PK100_ERR_SHAPE;
    if (format == 3 && group_scales == nullptr) return PK100_ERR_NULL;
    if (format != 3 && scales == nullptr) return PK100_ERR_NULL;
    if (format == 3 && k % 128 != 0) return PK100_ERR_SHAPE;
    if (format == 2 && k % 2 != 0) return PK100_ERR_SHAPE;
    pack_weight_rows_kernel<<<n, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(weight), n, k, ldw, format, static_cast<uint8_t*>(packed),
        scales, static_cast<__half*>(group_scales));
    return pk100_launch_status();
}

extern "C" int pk100_dequant_w4g128(void* stream, const void* codes, const void* group_scales,
                                    int n, int k, void* weight_f16) {
    if (!codes || !group_scales || !weight_f16) return PK100_ERR_NULL;
    if (n <= 0 || k <= 0 || k % 128 != 0) return PK100_ERR_SHAPE;
    const size_t total = static_cast<size_t>(n) * (k / 2);
    dequant_w4g128_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0,
                            static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(codes), static_cast<const __half*>(group_scales), n, k,
        static_cast<__half*>(weight_f16));
    return pk100_launch_status();
}

extern "C" int pk100_unpack_s4(void* stream, const void* packed, void* codes, long long packed_bytes) {
    if (!packed || !codes) return PK100_ERR_NULL;
    if (packed_bytes < 0) return PK100_ERR_SHAPE;
    if (packed_bytes == 0) return PK100_OK;
    if ((reinterpret_cast<uintptr_t>(packed) & 3u) || (reinterpret_cast<uintptr_t>(codes) & 7u)) return PK100_ERR_ALIGN;
    const size_t threads = (static_cast<size_t>(packed_bytes) + 3) / 4;
    unpack_s4_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(packed), static_cast<int8_t*>(codes), static_cast<size_t>(packed_bytes));
    return pk100_launch_status();
}

static int sparse24_launch(void* stream, const void* input, void* output, int rows, int cols, int mode) {
    if (!input || !output) return PK100_ERR_NULL;
    if (rows < 0 || cols <= 0 || cols % 16 != 0) return PK100_ERR_SHAPE;
    if (rows == 0) return PK100_OK;
    if ((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(output)) & 15u) return PK100_ERR_ALIGN;
    const size_t chunks = static_cast<size_t>(rows) * (cols / 16);
    sparse24_kernel<<<static_cast<unsigned>((chunks + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(input), static_cast<uint8_t*>(output), rows, cols, mode);
    return pk100_launch_status();
}

extern "C" int pk100_prune_2of4_e4m3(void* stream, const void* dense, void* pruned, int rows, int cols) {
    return sparse24_launch(stream, dense, pruned, rows, cols, 0);
}
extern "C" int pk100_compress_2of4_e4m3(void* stream, const void* dense, void* compressed, int rows, int cols) {
    return sparse24_launch(stream, dense, compressed, rows, cols, 1);
}
extern "C" int pk100_decompress_2of4_e4m3(void* stream, const void* compressed, void* dense, int rows, int cols) {
    return sparse24_launch(stream, compressed, dense, rows, cols, 2);
}

extern "C" int pk100_glu_masked(void* stream, const void* input, void* output, int total_rows,
                                int seg_stride, int valid_rows, const int* seg_valid) {
    if (!input || !output) return PK100_ERR_NULL;
    if (total_rows <= 0) return total_rows == 0 ? PK100_OK : PK100_ERR_SHAPE;
    if (seg_stride <= 0) return PK100_ERR_SHAPE;
    const size_t threads = static_cast<size_t>(total_rows) * kWidth / 8;
    glu_masked_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0,
                        static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(input), static_cast<__half*>(output), total_rows, seg_stride,
        valid_rows, seg_valid);
    return pk100_launch_status();
}

extern "C" int pk100_depthwise_bn_silu(void* stream, const void* input, const void* dw_weight,
                                       const float* bn_gamma, const float* bn_beta,
                                       const float* bn_mean, const float* bn_var, void* output,
                                       float* row_scales, int quantize, int segments,
                                       int seg_stride, int valid_rows, const int* seg_valid,
                                       float eps) {
    if (!input || !dw_weight || !bn_gamma || !bn_beta || !bn_mean || !bn_var || !output)
        return PK100_ERR_NULL;
    if (quantize && !row_scales) return PK100_ERR_NULL;
    if (segments <= 0) return segments == 0 ? PK100_OK : PK100_ERR_SHAPE;
    if (seg_stride <= 0) return PK100_ERR_SHAPE;
    auto misaligned = [](const void* ptr, uintptr_t mask) { return (reinterpret_cast<uintptr_t>(ptr) & mask) != 0; };
    if (misaligned(dw_weight, 7) || misaligned(bn_gamma, 15) || misaligned(bn_beta, 15) ||
        misaligned(bn_mean, 15) || misaligned(bn_var, 15) || misaligned(input, 7))
        return PK100_ERR_ALIGN;      // the kernel reads taps 8 bytes and BatchNorm vectors 16 bytes at a time
    const int strips = (seg_stride + kDwStrip - 1) / kDwStrip;
    pk100_launch_chained(depthwise_bn_silu_kernel, dim3(segments * strips), dim3(256), 0, static_cast<cudaStream_t>(stream),
        static_cast<const __half*>(input), static_cast<const __half*>(dw_weight), bn_gamma,
        bn_beta, bn_mean, bn_var, output, row_scales, quantize, seg_stride, valid_rows, seg_valid,
        eps);
    return pk100_launch_status();
}
