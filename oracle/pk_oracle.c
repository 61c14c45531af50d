/* CPU oracle, C restatement of the byte/integer codecs (TEST INFRASTRUCTURE).
 *
 * Cross-checks the numpy versions in oracle/codec.py and serves as the inner
 * loops of the timed CPU baseline.  Each function cites the reference code it
 * restates (paths inside the reference project).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

/* E4M3 decode (OCP FP8, bias 7, no inf, 0x7f = NaN). */
static float e4m3_decode_one(uint8_t code) {
    const int sign = code >> 7, exp = (code >> 3) & 15, man = code & 7;
    float v;
    if (exp == 15 && man == 7) return NAN;
    if (exp == 0) v = ldexpf((float)man / 8.0f, -6);
    else v = ldexpf(1.0f + (float)man / 8.0f, exp - 7);
    return sign ? -v : v;
}

/* `__nv_fp8_e4m3(float)` / `F8E4M3::from_f32`: RNE, saturate to +-448
 * (kernels/sm89/encoder.cu:557; src/cuda/encoder.rs:410). */
static uint8_t e4m3_encode_one(float x) {
    uint32_t bits;
    memcpy(&bits, &x, 4);
    const uint8_t sign = (uint8_t)((bits >> 24) & 0x80);
    const float ax = fabsf(x);
    if (isnan(x)) return sign | 0x7f;
    if (ax >= 448.0f) return sign | 0x7e;
    if (ax < ldexpf(1.0f, -10)) return sign;             /* below half the smallest subnormal */
    int e;
    frexpf(ax, &e);                                       /* ax = f * 2^e, f in [0.5, 1) */
    int exp = e - 1;                                      /* ax in [2^exp, 2^(exp+1)) */
    if (exp < -6) exp = -6;                               /* subnormal range: fixed quantum 2^-9 */
    const float quantum = ldexpf(1.0f, exp - 3);
    const float q = nearbyintf(ax / quantum);             /* RNE (default rounding mode), exact scaling */
    const float r = q * quantum;
    if (r >= 448.0f) return sign | 0x7e;
    if (r < ldexpf(1.0f, -6)) return sign | (uint8_t)q;   /* subnormal: mantissa = q */
    int e2;
    const float f2 = frexpf(r, &e2);                      /* r = f2 * 2^e2 */
    const int bexp = e2 - 1 + 7;
    const int man = (int)((f2 * 2.0f - 1.0f) * 8.0f);
    return sign | (uint8_t)(bexp << 3) | (uint8_t)man;
}

void pk_e4m3_encode(const float* x, uint8_t* out, long n) {
    for (long i = 0; i < n; ++i) out[i] = e4m3_encode_one(x[i]);
}

void pk_e4m3_decode(const uint8_t* in, float* out, long n) {
    for (long i = 0; i < n; ++i) out[i] = e4m3_decode_one(in[i]);
}

/* quantize_i8 (src/cuda/quant_benchmark.rs:827-829; kernels/sm89/linear.cu:549-560). */
void pk_quantize_int8(const float* x, float inverse_scale, int8_t* out, long n) {
    for (long i = 0; i < n; ++i) {
        float v = nearbyintf(x[i] * inverse_scale);
        if (v > 127.0f) v = 127.0f;
        if (v < -127.0f) v = -127.0f;
        out[i] = (int8_t)v;
    }
}

/* decision_key (kernels/sm89/decoder.cu:41-46): order-preserving key whose integer
 * maximum is the best score, ties -> the lower token id. */
uint64_t pk_decision_key(float score, int id) {
    if (score == 0.0f) score = 0.0f;
    uint32_t bits;
    memcpy(&bits, &score, 4);
    const uint32_t ordered = (bits & 0x80000000u) ? ~bits : (bits ^ 0x80000000u);
    return ((uint64_t)ordered << 32) | (uint64_t)(0xffffffffu - (uint32_t)id);
}

/* S8 x S8 -> S32 dot-product GEMM, acc[m,n] = sum_k a[m,k]*b[n,k]
 * (the accumulate of kernels/sm89/linear.cu:378-429), OpenMP over rows. */
void pk_gemm_s8(const int8_t* a, const int8_t* b, int32_t* acc, int m, int n, int k) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            int32_t s = 0;
            const int8_t* ar = a + (long)i * k;
            const int8_t* br = b + (long)j * k;
            for (int t = 0; t < k; ++t) s += (int32_t)ar[t] * (int32_t)br[t];
            acc[(long)i * n + j] = s;
        }
    }
}
