/*
 * libpk100 -- sm_100a (B200) kernels for the FastConformer / TDT hot path of
 * l4-parakeet-rs behind a plain C ABI.
 *
 * Every entry point replaces one kernel (or host launch helper) of the
 * reference's `kernels/sm89` translation units; the reference interface each
 * one stands in for is cited as path:line inside the reference project.
 *
 * Conventions (the reference's, src/cuda.rs:698-778, src/cuda/cublas.rs:67-113):
 *   - pointers are DEVICE pointers unless the name says host; the caller owns
 *     every allocation, the library never allocates or frees device memory;
 *   - activations are row-major [rows, width]; weights are row-major
 *     [out (N), in (K)];
 *   - `stream` is a CUstream / cudaStream_t passed as void*; every call is
 *     asynchronous and stream-ordered, performs no synchronisation and no
 *     allocation;
 *   - return value: 0 success, negative = argument error found on the host
 *     (nothing was launched), positive = CUDA error code of the launch.
 *   - A batch of utterances is laid out as `segments` consecutive blocks of
 *     `seg_stride` rows; the first valid rows of each block carry data
 *     (`seg_valid[s]` when that device array is given, else `valid_rows`), the
 *     remaining rows are zero -- the reference's rows / valid_rows /
 *     padded_rows geometry (src/cuda/pipeline.rs:438-442) per utterance.
 */
#ifndef PK100_H_
#define PK100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    PK100_OK = 0,
    PK100_ERR_NULL = -1,      /* a required pointer is null */
    PK100_ERR_SHAPE = -2,     /* a dimension violates the documented constraint */
    PK100_ERR_ALIGN = -3,     /* pointer / leading dimension not 16-byte aligned */
    PK100_ERR_UNSUPPORTED = -4,
    PK100_ERR_DRIVER = -5,    /* tensor-map encoding failed */
    PK100_ERR_LIMIT = -6,     /* size beyond a documented fixed capacity */
    PK100_ERR_FORMAT = -7,    /* artifact file or packer input violates the format */
    PK100_ERR_IO = -8         /* artifact file cannot be opened or mapped */
};

/* Operand kinds of pk100_gemm. */
enum {
    PK100_KIND_F16 = 0, PK100_KIND_E4M3 = 1, PK100_KIND_S8 = 2,
    /* A fp16 [m,k]; b = INT4 codes [n, k/2] (low nibble = even k), b_group_scales = fp16
     * [k/128, n]; the weights are dequantised to fp16 in shared memory by producer warps
     * (W = f16(code * scale)) and multiplied with kind::f16 MMAs. */
    PK100_KIND_F16_W4G128 = 3
};
/* Output encodings of pk100_gemm. */
enum { PK100_OUT_F16 = 0, PK100_OUT_F32 = 1, PK100_OUT_E4M3 = 2, PK100_OUT_S8 = 3 };
/* Activations (kernels/sm89/linear.cu:65-73). */
enum { PK100_ACT_NONE = 0, PK100_ACT_SILU = 1, PK100_ACT_RELU = 2 };
/* Epilogue families. */
enum { PK100_EPI_LINEAR = 0, PK100_EPI_GLU = 1, PK100_EPI_SPARSE_OUT = 2 };
/* LayerNorm output encodings. */
enum {
    PK100_LN_F16 = 0,        /* fp16 */
    PK100_LN_E4M3_FIXED = 1, /* E4M3(y * inv_scale)                          */
    PK100_LN_E4M3_ROW = 2,   /* E4M3(y / s), s = absmax/448 per row (0 -> 1) */
    PK100_LN_S8_ROW = 3,     /* clamp(rne(y / s)), s = absmax/127 per row    */
    PK100_LN_S4_ROW = 4      /* INT4 codes clamp(rne(y / s), -8, 7), s = max(y/7, -y/8) per row (0 -> 1), one
                              * code per INT8 byte: pk_sm89_layer_norm_quantize_int4_dynamic
                              * (kernels/sm89/encoder.cu:211-306) without the nibble packing, so that the
                              * INT4 x INT4 products of its consumer run exactly on kind::i8 */
};
/* Weight packing formats of pk100_pack_weight_rows. */
enum { PK100_PACK_E4M3 = 0, PK100_PACK_S8 = 1, PK100_PACK_S4_ROW = 2, PK100_PACK_S4_G128 = 3 };

/*
 * General tensor-core linear:  D[m,n] = epilogue(A[m,k] . B[n,k]^T).
 * tcgen05.mma (kind::f16 / kind::f8f6f4 / kind::i8), TMA-staged operands, TMEM
 * accumulators.  Replaces the GEMM family of the reference:
 *   pk_sm89_fp16_linear_epilogue(_m64)   kernels/sm89/linear.cu:83-171, :243-320
 *   pk_sm89_fp8_linear_epilogue          kernels/sm89/linear.cu:325-374
 *   pk_sm89_int8_linear_epilogue         kernels/sm89/linear.cu:378-429
 *   ffn_fp8_async<> and its 13 wrappers  kernels/sm89/encoder.cu:787-1127, :1313-1319, :2099-2107
 *   pk_sm89_ffn_expand_async             kernels/sm89/encoder.cu:427-547
 *   Cublas::linear (cublasGemmEx)        src/cuda/cublas.rs:67-113
 * Epilogue algebra (kernels/sm89/encoder.cu:961-1005):
 *   v = acc * row_scale(s)[m] * col_scales[n] + bias[n];  v = act(v);
 *   v = residual ? fma(alpha, v, residual[m,n]) : alpha * v;   rows >= valid_rows -> 0
 *   PK100_EPI_GLU: B rows [0,n/2) are values, [n/2,n) gates; out[m,c] =
 *     f16(value) / (1 + exp(-f16(gate))), out has n/2 columns (encoder.cu:936-944).
 *   PK100_EPI_SPARSE_OUT: v = SiLU(...); per [128-row x 64-col] tile t = max|v|;
 *     keep_out[tile] = t >= tau; kept tiles are stored as INT8
 *     clamp(rne(v * out_scale)), dropped tiles as zeros; stats_out[tile] = t.  SiLU is
 *     evaluated as v/2 * (1 + tanh(v/2)) with the hardware tanh approximation (rel. 2^-11).
 *   keep_in: when given ([ceil(m/128), k/64] bytes) K tiles flagged 0 are skipped
 *     (their A bytes must be zero).
 * Constraints: k * elem_size, lda/ldb * elem_size multiples of 16 bytes;
 *   n % 32 == 0; 16-byte aligned pointers; ld_out * out_elem_size % 16 == 0.
 */
typedef struct pk100_gemm_args {
    int kind;                 /* PK100_KIND_* (A and B share it) */
    int epilogue;             /* PK100_EPI_* */
    int m, n, k;
    const void* a;  int lda;  /* [m, k], leading dimension in elements */
    const void* b;  int ldb;  /* [n, k] */
    const float* row_scales;  /* [m] or NULL */
    float row_scale;          /* used when row_scales == NULL */
    const float* col_scales;  /* [n] or NULL */
    const float* bias;        /* [n] or NULL */
    int act;                  /* PK100_ACT_* */
    const void* residual;     /* fp16 [m, ld_res] or NULL; may alias out */
    int ld_res;
    float alpha;
    int valid_rows;           /* <= 0 means m */
    void* out;      int ld_out;
    int out_type;             /* PK100_OUT_* */
    float out_scale;
    float tau;
    uint8_t* keep_out;
    float* stats_out;
    const uint8_t* keep_in;
    int* status;              /* device int, may be NULL: becomes 1 if a bounded wait expired; bit 3 (value 8) is
                               * OR-ed in when PK100_EPI_SPARSE_OUT clamped a code of a kept tile at +127
                               * (|v * out_scale| > 127: choose a smaller out_scale) */
    int max_ctas;             /* <= 0: one CTA per SM */
    const void* b_group_scales; /* PK100_KIND_F16_W4G128 only */
} pk100_gemm_args;

int pk100_gemm(void* stream, const pk100_gemm_args* args);

/* enable != 0: 256-column GEMM tiles run on CTA pairs (tcgen05 cta_group::2, 2-CTA clusters,
 * 256 x 256 tiles); default 0 = one CTA per 128 x 256 tile, which measured faster on B200. */
void pk100_set_gemm_cta_pairs(int enable);

/* Process-wide cap on the persistent CTAs of every pk100_gemm launch whose own max_ctas is <= 0
 * (the sequencers pk100_run_layers / pk100_run_subsampling included); 0 = one CTA per SM.  For a
 * host that keeps another persistent kernel resident beside the encoder (the cluster decoder holds
 * 16 SMs per call): persistent GEMM CTAs that cannot be placed at once queue behind the first wave
 * and double the kernel's time, a smaller grid does not.  Takes effect on launches issued after it. */
void pk100_set_gemm_cta_cap(int ctas);

/* Programmatic dependent launch of the kernels of the per-block chain (LayerNorm, GEMMs,
 * attention, depthwise convolution): each launch may become resident while its predecessor in the
 * stream drains (its set-up overlaps that tail) and waits for the whole predecessor grid before it
 * touches global memory, so results do not change.  Default 1; 0 = plain stream order. */
void pk100_set_dependent_launch(int enable);

/* Tensor maps (TMA descriptors) are cached per (pointer, shape, leading dimension, box): hits and
 * misses of that cache since the library was loaded.  Either pointer may be NULL. */
void pk100_tensor_map_cache_stats(long long* hits, long long* misses);

/* Number of kernels this library has launched in the calling process (monotonic). */
long long pk100_launch_count(void);

/* pk_sm89_layer_norm (kernels/sm89/encoder.cu:81-126) and
 * pk_sm89_layer_norm_quantize_fp8_dynamic (:294-299); launcher launch_norm /
 * launch_norm_quantize_fp8 (src/cuda/encoder.rs:1361-1468).  Width is 1024. */
int pk100_layer_norm(void* stream, const void* input, const void* gamma, const void* beta,
                     void* output, float* scales, int mode, float inv_scale, int total_rows,
                     int seg_stride, int valid_rows, const int* seg_valid, float eps);

/* pk_sm89_layer_norm_pair (kernels/sm89/encoder.cu:128-209; launch_norm_pair
 * src/cuda/encoder.rs:1394-1433): fp16 first output, second LayerNorm of the
 * rounded first output in `next_mode`. */
int pk100_layer_norm_pair(void* stream, const void* input, const void* gamma, const void* beta,
                          void* output, const void* next_gamma, const void* next_beta,
                          void* next_output, float* next_scales, int next_mode,
                          float next_inv_scale, int total_rows, int seg_stride, int valid_rows,
                          const int* seg_valid, float eps);

/* pk_sm89_quantize_fp8_fixed (kernels/sm89/encoder.cu:549-559). */
int pk100_quantize_fp8_fixed(void* stream, const void* input, void* output, long long elements,
                             float inverse_scale);

/* pk_sm89_quantize_int8 (kernels/sm89/linear.cu:549-560); argument order as there. */
int pk100_quantize_int8(void* stream, const void* input, void* output, float inverse_scale,
                        long long elements);

/* Load-time weight packing.  Replaces QuantizedFfnWeights::load_for
 * (src/cuda/encoder.rs:361-422, CPU) and pk_sm89_quantize_rows1024 / _rows256 /
 * _ffn_contract (kernels/sm89/encoder.cu:1129-1180, per request in the
 * reference).  weight: fp16 [n, ldw]; packed: [n, k] bytes (E4M3, S8) or
 * [n, k/2] (S4, low nibble = even k); scales fp32 [n]; group_scales fp16
 * [k/128, n] (PK100_PACK_S4_G128 only). */
int pk100_pack_weight_rows(void* stream, const void* weight, int n, int k, int ldw, int format,
                           void* packed, float* scales, void* group_scales);

/* INT4-g128 codes -> fp16 weights (the dequantisation the INT4 GEMM performs;
 * idea of pk_sm89_q4_k_dequantize, kernels/sm89/linear.cu:458-472). */
int pk100_dequant_w4g128(void* stream, const void* codes, const void* group_scales, int n, int k,
                         void* weight_f16);

/* Packed INT4 codes (two per byte, low nibble = even index, two's complement: the storage of
 * PK100_PACK_S4_ROW weights and of the reference's INT4 activations, kernels/sm89/encoder.cu:279-290) ->
 * one INT8 byte per code, the operand form of kind::i8.  The reference's INT4 x INT4 FF1
 * (pk_sm89_ffn_expand_int4_sparse, mma m16n8k64 s4, :1079-1085) is then pk100_layer_norm mode
 * PK100_LN_S4_ROW + pk100_gemm kind S8 on the unpacked weight codes (row_scales, col_scales, SiLU,
 * PK100_OUT_E4M3 x 16) + pk100_compress_2of4_e4m3: the same integer sums, exactly. */
int pk100_unpack_s4(void* stream, const void* packed, void* codes, long long packed_bytes);

/* 2:4 structured sparsity of E4M3 activations: the input format of the reference's sparse FF2
 * (pk_sm89_ffn_expand_int4_sparse epilogue 7, kernels/sm89/encoder.cu:685-704, :1037-1054, consumed by
 * pk_sm89_ffn_contract_fp8_sparse :1087-1095 with mma.sp).  Per four consecutive bytes the two largest
 * 7-bit magnitudes are kept, ties to the lower index.  cols % 16 == 0, 16-byte aligned pointers.
 *   prune:      dense [rows, cols] -> dense [rows, cols] with the dropped bytes zero (may be in place);
 *   compress:   dense -> the reference's arena: data [rows, cols/2] then metadata [rows, cols/8]
 *               (rows * cols * 5 / 8 bytes);
 *   decompress: that arena -> dense [rows, cols].
 * The reference-parity FF2 on B200 is decompress (or prune) + pk100_gemm kind E4M3 with row_scale 1/16,
 * the weight's column scales, alpha 0.5 and the residual in place: dense math on the same values. */
int pk100_prune_2of4_e4m3(void* stream, const void* dense, void* pruned, int rows, int cols);
int pk100_compress_2of4_e4m3(void* stream, const void* dense, void* compressed, int rows, int cols);
int pk100_decompress_2of4_e4m3(void* stream, const void* compressed, void* dense, int rows, int cols);

/* pk_sm89_glu_masked (kernels/sm89/encoder.cu:308-330). input [rows, 2048]. */
int pk100_glu_masked(void* stream, const void* input, void* output, int total_rows,
                     int seg_stride, int valid_rows, const int* seg_valid);

/* pk_sm89_depthwise_batchnorm_silu (kernels/sm89/encoder.cu:1182-1233) and, with
 * quantize != 0, pk_sm89_depthwise_pack (:1235-1311): E4M3 bytes + per-row scales. */
int pk100_depthwise_bn_silu(void* stream, const void* input, const void* dw_weight,
                            const float* bn_gamma, const float* bn_beta, const float* bn_mean,
                            const float* bn_var, void* output, float* row_scales, int quantize,
                            int segments, int seg_stride, int valid_rows, const int* seg_valid,
                            float eps);

/* pk_sm89_local_relpos_attention (kernels/sm89/encoder.cu:1338-1461): the fp32
 * CUDA-core statement of the operator, one warp per (query, head).  query /
 * key / value are fp16 with row strides ldq / ldk / ldv (elements) so that the
 * planes of a fused QKV projection can be passed directly; position is the
 * head-major table [8, 272, 128]; bias_u / bias_v are [8, 128]. */
int pk100_local_relpos_attention_simple(void* stream, const void* query, int ldq, const void* key,
                                        int ldk, const void* value, int ldv, const void* position,
                                        const void* bias_u, const void* bias_v, void* output,
                                        int ldo, int segments, int seg_stride, int valid_rows,
                                        const int* seg_valid);

/* pk_sm89_local_relpos_attention_tc_scores / _packed (kernels/sm89/encoder.cu:1500-2052;
 * launch_attention_arena src/cuda/encoder.rs:1839-1963): the tensor-core kernel of the
 * hot path.  Same arguments and semantics as the _simple entry point; Q.K^T, Q.P^T and
 * P.V run as fp16 MMAs with fp32 accumulation and an fp32 online softmax. */
int pk100_local_relpos_attention(void* stream, const void* query, int ldq, const void* key, int ldk,
                                 const void* value, int ldv, const void* position,
                                 const void* bias_u, const void* bias_v, void* output, int ldo,
                                 int segments, int seg_stride, int valid_rows, const int* seg_valid);

/* The same operator on tcgen05 tensor cores (the kernel of the hot path on B200): one CTA per 128
 * queries of a head, Q.P^T, Q.K^T and Pr.V as tcgen05.mma kind::f16 with the accumulators in tensor
 * memory, operands staged by TMA (the value rows as they lie in memory: an MN-major B operand, no
 * transposed copy), fp32 softmax.  Arguments as above plus
 *   status:  device int, set to 1 when a bounded wait expired (may be NULL).
 * Needs seg_stride % 128 == 0 (PK100_ERR_SHAPE otherwise: use pk100_local_relpos_attention). */
int pk100_local_relpos_attention_tcgen05(void* stream, const void* query, int ldq, const void* key, int ldk,
                                         const void* value, int ldv, const void* position,
                                         const void* bias_u, const void* bias_v, void* output, int ldo,
                                         int segments, int seg_stride, int valid_rows, const int* seg_valid,
                                         int* status);

/* pk_sm89_pack_position_heads (kernels/sm89/encoder.cu:1321-1336):
 * [272, 1024] -> head-major [8, 272, 128]. */
int pk100_pack_position_heads(void* stream, const void* input, void* output);

/* ------------------------------------------------------------------------
 * Encoder layer sequencer -- the host side of one FastConformer block.
 * Replaces LayerWeights (src/cuda/encoder.rs:530-601), LayerBuffers (:432-439)
 * and run_layer / run_layers (:484-528, :604-1126).
 *
 * Precision map of this build (one table for every layer and every size; the
 * reference switches kernels by row count, src/cuda/encoder.rs:618-633):
 *   FF modules   LN -> E4M3 (x56) | W1 E4M3 per-row scales, SiLU, 128x64 tile
 *                threshold tau, INT8 (x32) | W2 INT8 per-row scales, tile skip,
 *                x += 0.5 * y
 *   attention    LN -> INT8 per-row | Wqkv INT8 per-row scales -> fp16 Q|K|V
 *                [rows, 3072] | local rel-pos attention fp16 | Wo INT4 group-128
 *                dequantised to fp16, x += y
 *   conv module  LN -> E4M3 per-row | Wpw1 E4M3 + GLU + pad mask | depthwise k=9
 *                + BatchNorm + SiLU -> E4M3 per-row | Wpw2 E4M3, x += y
 *   output       LayerNorm (fused with the next block's first LayerNorm)
 */
typedef struct pk100_ff_weights {
    const void* ln_gamma;  const void* ln_beta;      /* fp16 [1024] */
    const void* w1;        const float* w1_scales;   /* E4M3 [4096,1024], fp32 [4096] */
    const void* w2;        const float* w2_scales;   /* S8 [1024,4096], fp32 [1024] */
    float tau;                                       /* tile threshold on max|SiLU| */
} pk100_ff_weights;

typedef struct pk100_layer_weights {
    pk100_ff_weights ff1;
    const void* ln_att_gamma;  const void* ln_att_beta;
    const void* wqkv;          const float* wqkv_scales;   /* S8 [3072,1024] rows Q|K|V */
    const void* position;                                   /* fp16 [8,272,128] */
    const void* bias_u;        const void* bias_v;          /* fp16 [8,128] */
    const void* wo_f16;                                     /* fp16 [1024,1024] (dequantised INT4-g128); used when wo_codes == NULL */
    const void* wo_codes;      const void* wo_group_scales; /* INT4 codes [1024,512] + fp16 scales [8,1024] */
    const void* ln_conv_gamma; const void* ln_conv_beta;
    const void* wpw1;          const float* wpw1_scales;   /* E4M3 [2048,1024] */
    const void* dw_weight;                                  /* fp16 [1024,9] */
    const float* bn_gamma; const float* bn_beta; const float* bn_mean; const float* bn_var;
    const void* wpw2;          const float* wpw2_scales;   /* E4M3 [1024,1024] */
    pk100_ff_weights ff2;
    const void* ln_out_gamma;  const void* ln_out_beta;
} pk100_layer_weights;

/* Caller-owned scratch for `rows` = segments * seg_stride rows.  Sizes in bytes:
 * q8 rows*1024, row_scales rows*4, hidden8 rows*4096, keep ceil(rows/128)*64,
 * qkv rows*3072*2, att rows*1024*2, glu rows*1024*2, dw8 rows*1024,
 * dw_scales rows*4, status 4.  All 256-byte aligned. */
typedef struct pk100_encoder_workspace {
    void* q8; float* row_scales; void* hidden8; uint8_t* keep; void* qkv; void* att;
    void* glu; void* dw8; float* dw_scales; int* status;
    /* Optional timing hook (HOST array of cudaEvent_t, may be NULL): the FF-expand GEMM of
     * layer l, module m (0/1) is bracketed by events[2*(2*l+m)] and [2*(2*l+m)+1] when
     * 2*(2*l+m)+1 < profile_events_len.  Recording an event does not synchronise. */
    void** profile_events; int profile_events_len;
} pk100_encoder_workspace;

/* Bytes needed for one arena holding every field above. */
long long pk100_encoder_workspace_bytes(int rows);
/* Carves `base` (256-byte aligned, >= pk100_encoder_workspace_bytes(rows)). */
int pk100_encoder_workspace_carve(void* base, int rows, pk100_encoder_workspace* out);

/* Runs layers [0, n_layers).  state_a holds the input rows [rows,1024] fp16 and is
 * updated in place (residual stream); layer i writes its output norm to state_b
 * (i even) or state_a (i odd) and the next layer continues from there;
 * *output receives the buffer that holds the final result.  tile_stats, when not
 * NULL, receives max|SiLU| per 128x64 tile: [n_layers][2][ceil(rows/128)*64].
 * attention_impl: 0 = tensor-core kernel (tcgen05 when seg_stride is a multiple of 128, else the
 * mma.sync kernel), 1 = fp32 CUDA-core kernel, 2 = the mma.sync kernel. */
int pk100_run_layers(void* stream, const pk100_layer_weights* layers, int n_layers, void* state_a,
                     void* state_b, const pk100_encoder_workspace* ws, int segments,
                     int seg_stride, int valid_rows, const int* seg_valid, float* tile_stats,
                     int attention_impl, void** output);

/* ------------------------------------------------------------------------
 * TDT greedy decoder.  Replaces DecoderWeights (src/cuda/decoder.rs:227-271),
 * launch_decode (:274-353) and the persistent kernels pk_sm89_tdt_persistent_v2
 * / _fp8_ih (kernels/sm89/decoder.cu:165-447, :452-784) for a BATCH of
 * utterances.  `layers` is 1 or 2 LSTM layers (the reference model has 2).
 * The encoder projection (enc_proj = state . W_enc^T + b, fp16 [rows, 640]) is
 * an ordinary pk100_gemm call made by the caller, as in decoder.rs:298-313.
 */
#define PK100_DECODER_MAX_UTTERANCES 8

typedef struct pk100_decoder_weights {
    int layers;
    const void* embedding;                 /* fp16 [1025, 640] */
    const void* w_ih[2]; const void* w_hh[2];   /* fp16 [2560, 640], gate order i f g o */
    const float* b_ih[2]; const float* b_hh[2]; /* fp32 [2560] */
    const void* w_pred; const float* b_pred;    /* fp16 [640, 640], fp32 [640] */
    const void* w_joint; const float* b_joint;  /* fp16 [1030, 640], fp32 [1030]: 1025 tokens + 5 durations */
} pk100_decoder_weights;

/* Scratch bytes for `utterances` (<= PK100_DECODER_MAX_UTTERANCES); 0 if out of range. */
long long pk100_tdt_workspace_bytes(int utterances);

/* Byte offset inside the workspace of an int32 that the cluster and exchange kernels set, when they
 * finish, to the number of lockstep rounds the call took (a round = one joint evaluation per live
 * utterance; the latency unit of the decoder: src/cuda/decoder.rs:274-353 has one grid barrier per
 * such step).  -1 when `utterances` is out of range.  For measurement; the grid-barrier kernel
 * leaves the word at zero. */
long long pk100_tdt_rounds_offset(int utterances);

/* How many 16-CTA clusters of the cluster decoder (1 or 2 LSTM layers) the current device can hold
 * at once (a cluster has to fit one GPC; 7 on a B200), 0 when that kernel cannot run here.  A host
 * that decodes several groups of utterances side by side on separate streams, each with its own
 * workspace, should not start more calls than this: a call beyond it waits for a whole earlier one. */
int pk100_tdt_cluster_capacity(int lstm_layers);

/* Decodes `utterances` sequences in lockstep.  Chooses the cluster kernel when the device can
 * host a 16-CTA cluster, else the exchange kernel (both
 * below; same results up to the summation order of the fp32 partial sums).
 * enc_proj rows of utterance u start at
 * u * seg_stride; frames[u] (device int array) frames are consumed.  tokens /
 * durations: [utterances, max_tokens] int32 (durations may be NULL), counts:
 * [utterances].  workspace: >= pk100_tdt_workspace_bytes(utterances), 256-byte
 * aligned; it is cleared by the call.  frames[u] beyond seg_stride is read as seg_stride (a
 * decode never leaves its utterance's block).  *status (device int, may be NULL) becomes 2 if
 * a bounded wait expired; bit 4 is set when every token score of a round was NaN (that round
 * decodes as a blank, so no id outside [0, 1024] is ever produced).  Token rule: highest joint score, ties to the lower
 * id; duration: first strict maximum of 5 logits; at most 10 symbols per frame; blank
 * (1024) never updates the prediction network (kernels/sm89/decoder.cu:35-46, :416-445). */
int pk100_tdt_decode(void* stream, const pk100_decoder_weights* weights, const void* enc_proj,
                     int utterances, int seg_stride, const int* frames, void* workspace,
                     int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                     int* status);

/* Decoder for hosts that may not allocate device memory.  It has no counterpart in the
 * reference (there the Rust host allocates the decoder workspace itself,
 * src/cuda/pipeline.rs:280-350).  Meant for embedders whose process owns a fixed CUDA memory
 * arena and rejects cudaMalloc from plug-ins: pre-sized serving workers, real-time audio
 * hosts, code called while another component is capturing the stream.
 * Same arguments as pk100_tdt_decode_exchange (whose kernel it runs) minus `workspace`: the exchange scratch is a fixed
 * 288 KiB device array inside the library image, present on every GPU that loads the
 * library for the life of the process.  Limits and rules:
 *   - at most PK100_DECODER_MAX_UTTERANCES utterances; more returns PK100_ERR_LIMIT and
 *     launches nothing;
 *   - the first call on each device looks the array's device address up (with that device
 *     current) and remembers it; make that first call outside any stream capture; the remembered
 *     address does not survive a cudaDeviceReset (reload the library after one);
 *   - the array is shared by every call and keeps the previous call's contents; each call
 *     clears the part it uses before its kernel starts (stream-ordered), so back-to-back
 *     calls on one stream are fine, but two calls that overlap on the GPU (different
 *     streams or threads) race on it -- serialise them;
 *   - performs no cudaMalloc / cudaFree and calls no allocating library routine. */
int pk100_tdt_decode_static(void* stream, const pk100_decoder_weights* weights, const void* enc_proj,
                            int utterances, int seg_stride, const int* frames, int32_t* tokens,
                            int32_t* durations, int32_t* counts, int max_tokens, int* status);

/* Same contract, one kernel design each.
 * _cluster: one thread-block cluster of 16 CTAs; the phases of a round exchange their vectors
 *   through distributed shared memory (remote stores that complete on the receiver's mbarrier);
 *   joint rows resident in shared memory, layer 0's recurrent weights resident in tensor memory,
 *   prediction weights streamed from L2, all from a fragment-ordered copy that the call writes
 *   into the workspace.  With two LSTM layers the joint rows and the second layer's weights are
 *   streamed as well (the second layer's state takes the room of the joint rows).  PK100_ERR_UNSUPPORTED when the device cannot
 *   co-schedule 16 CTAs of that much shared memory as a cluster.
 * _exchange: one CTA per SM, all weights resident in shared memory, phases exchange through
 *   tagged global-memory slots that the consumers poll (bounded).  One or two LSTM layers.  Uses
 *   only the first 280 KB of the workspace. */
int pk100_tdt_decode_cluster(void* stream, const pk100_decoder_weights* weights, const void* enc_proj,
                             int utterances, int seg_stride, const int* frames, void* workspace,
                             int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                             int* status);
int pk100_tdt_decode_exchange(void* stream, const pk100_decoder_weights* weights, const void* enc_proj,
                              int utterances, int seg_stride, const int* frames, void* workspace,
                              int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                              int* status);

/* Same contract, earliest design kept as a cross-check: weights in shared memory and a
 * bounded grid barrier between the phases (the structure of the reference kernel,
 * kernels/sm89/decoder.cu:227-414).  pk100_tdt_decode falls back to it on devices whose SM
 * count does not fit the register-resident slicing. */
int pk100_tdt_decode_barrier(void* stream, const pk100_decoder_weights* weights, const void* enc_proj,
                             int utterances, int seg_stride, const int* frames, void* workspace,
                             int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                             int* status);

/* Long-request numerics.  From 1024 encoder frames on (FP8_MIN_FRAMES, src/cuda/decoder.rs:15,
 * :88, :292-321) the reference launches another kernel (pk_sm89_tdt_persistent_fp8_ih,
 * kernels/sm89/decoder.cu:452-784, :805-824) that computes a different function: w_hh of both
 * layers and w_ih of layer 1 become per-tensor symmetric INT8 codes (scale = max|w| / 127, derived
 * inside every request, :517-575), the hidden state that multiplies them is rne(h * 127) (:644,
 * :668), and the layer-0 input term is read from an fp16 table embedding . w_ih[0]^T
 * (launch_input_table, src/cuda/decoder.rs:355-383).  Prediction projection and joint keep the fp32
 * state.  The entry points below reproduce those numerics (integer dot products exactly), with the
 * contract of pk100_tdt_decode:
 * _long: the cluster kernel where available, else the grid-barrier kernel;
 * _long_cluster / _long_barrier: one kernel each (PK100_ERR_UNSUPPORTED as for _cluster);
 * _auto: the reference's rule applied per utterance -- utterances with frames[u] < 1024 are decoded
 *   with the short-request numerics, the others with the long-request numerics, as two launches on
 *   `stream` that each skip the other's utterances.  A host that knows every utterance is short
 *   calls pk100_tdt_decode and saves the second launch. */
int pk100_tdt_decode_long(void* stream, const pk100_decoder_weights* weights, const void* enc_proj,
                          int utterances, int seg_stride, const int* frames, void* workspace,
                          int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                          int* status);
int pk100_tdt_decode_long_cluster(void* stream, const pk100_decoder_weights* weights, const void* enc_proj,
                                  int utterances, int seg_stride, const int* frames, void* workspace,
                                  int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                                  int* status);
int pk100_tdt_decode_long_barrier(void* stream, const pk100_decoder_weights* weights, const void* enc_proj,
                                  int utterances, int seg_stride, const int* frames, void* workspace,
                                  int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                                  int* status);
int pk100_tdt_decode_auto(void* stream, const pk100_decoder_weights* weights, const void* enc_proj,
                          int utterances, int seg_stride, const int* frames, void* workspace,
                          int32_t* tokens, int32_t* durations, int32_t* counts, int max_tokens,
                          int* status);

/* ------------------------------------------------------------------------
 * 8x convolution subsampling for a batch of utterances: mel fp32
 * [utterances, frames, 128] -> fp16 rows [utterances * seg_stride, 1024].
 * Replaces run_subsampling (src/cuda/subsampling.rs:436-804) and
 * pk_sm89_subsample_first / _depthwise / _flatten
 * (kernels/sm89/subsampling.cu:11-226); the pointwise layers and the projection
 * are pk100_gemm calls (fp16, bias, ReLU) like launch_linear_view there.
 * mel_frames (device int [utterances], may be NULL = `frames` for all) gives each
 * utterance's true frame count; utterance u yields ceil(ceil(ceil(f/2)/2)/2) rows,
 * the remaining rows of its block are "don't care" (every consumer masks them). */
typedef struct pk100_subsampling_weights {
    const void* conv0_w; const void* conv0_b;   /* fp16 [256,9] (3x3), fp16 [256] */
    const void* dw1_w;   const void* dw1_b;     /* fp16 [256,9], fp16 [256] */
    const void* pw1_w;   const float* pw1_b;    /* fp16 [256,256], fp32 [256] */
    const void* dw2_w;   const void* dw2_b;
    const void* pw2_w;   const float* pw2_b;
    const void* proj_w;  const float* proj_b;   /* fp16 [1024,4096], fp32 [1024] */
} pk100_subsampling_weights;

long long pk100_subsampling_workspace_bytes(int utterances, int frames, int seg_stride);

int pk100_run_subsampling(void* stream, const pk100_subsampling_weights* weights, const float* mel,
                          int utterances, int frames, const int* mel_frames, void* workspace,
                          void* output, int seg_stride, int* status);

/* The reference's variant for requests of 1024 output frames or more (FP8_MIN_FRAMES, src/cuda/subsampling.rs:22,
 * :551-630, :718-775): the fp16 output of the first depthwise convolution is quantised per row to E4M3
 * (absmax / 448; pk_sm89_subsample_depthwise_fp8 kernels/sm89/subsampling.cu:126-165) and its pointwise layer
 * runs E4M3 x E4M3 against per-row E4M3 weights (pk_sm89_subsample_pointwise_fp8 kernels/sm89/encoder.cu:1113-1119);
 * the second stage stays fp16; the flattened rows are quantised per row (pk_sm89_quantize_ffn_contract :1161-1180)
 * and projected E4M3 x E4M3 (pk_sm89_subsample_projection_fp8 :1105-1111).  The packed weights come from
 * pk100_pack_weight_rows(PK100_PACK_E4M3) of pw1_w and proj_w once at load (the reference re-quantises them in
 * every request).  Workspace: pk100_subsampling_fp8_workspace_bytes. */
typedef struct pk100_subsampling_fp8 {
    const void* pw1_q;  const float* pw1_scales;    /* E4M3 [256,256], fp32 [256] */
    const void* proj_q; const float* proj_scales;   /* E4M3 [1024,4096], fp32 [1024] */
} pk100_subsampling_fp8;

long long pk100_subsampling_fp8_workspace_bytes(int utterances, int frames, int seg_stride);

int pk100_run_subsampling_fp8(void* stream, const pk100_subsampling_weights* weights,
                              const pk100_subsampling_fp8* fp8, const float* mel, int utterances, int frames,
                              const int* mel_frames, void* workspace, void* output, int seg_stride, int* status);

/* ------------------------------------------------------------------------
 * ".pkl4" weight artifact: reader and layout packers (host code, no GPU).
 * Replaces AotArtifactIndex::open / read_f32 and validate_header
 * (src/artifact.rs:98-187, :514-593, :687-724) and the encoders encode_fp16,
 * encode_fp16_linear, encode_fp32_bias, align_up (src/artifact.rs:413-484, :734-739).
 * The file is mapped read-only; `data` pointers stay valid until pk100_artifact_close.
 * A file written by the reference (target "sm_89") is accepted as is: its storages are the
 * layouts these kernels read (fp16 [out^128, in^128] row-major, fp32 bias ^128).
 * Load-time FP8 / INT8 / INT4 packing of the linears is pk100_pack_weight_rows. */
typedef struct pk100_artifact pk100_artifact;
enum {
    PK100_STORAGE_FP16 = 0, PK100_STORAGE_FP32 = 1,
    PK100_STORAGE_FP16_LINEAR = 2,   /* "sm89_fp16_linear" */
    PK100_STORAGE_FP32_BIAS = 3      /* "sm89_fp32_bias" */
};
typedef struct pk100_artifact_tensor {
    const char* name;                  /* owned by the artifact */
    int storage;                       /* PK100_STORAGE_* */
    int logical_rank, physical_rank;   /* <= 4 */
    long long logical_shape[4], physical_shape[4];
    unsigned long long offset, bytes;  /* offset from the start of the payload */
    const void* data;                  /* host pointer into the mapping, 256-byte aligned */
} pk100_artifact_tensor;

/* Opens and validates `path`.  On failure returns PK100_ERR_IO / PK100_ERR_FORMAT and writes a
 * message of the reference's wording into `error` (may be NULL). */
int pk100_artifact_open(const char* path, pk100_artifact** out, char* error, int error_len);
void pk100_artifact_close(pk100_artifact* artifact);
int pk100_artifact_tensor_count(const pk100_artifact* artifact);
int pk100_artifact_tensor_at(const pk100_artifact* artifact, int index, pk100_artifact_tensor* out);
int pk100_artifact_find(const pk100_artifact* artifact, const char* name);   /* index or -1 */
int pk100_artifact_vocabulary_size(const pk100_artifact* artifact);
const char* pk100_artifact_vocabulary_at(const pk100_artifact* artifact, int index);
/* key: "target", "profile", "source_repository", "source_revision", "precision_plan" */
const char* pk100_artifact_field(const pk100_artifact* artifact, const char* key);
/* Plain FP32 tensors only; fails on a non-finite value (src/artifact.rs:158-187). */
int pk100_artifact_read_f32(const pk100_artifact* artifact, const char* name, float* out, long long capacity);

/* fp32 -> fp16 round-to-nearest-even; non-finite input is PK100_ERR_FORMAT. */
int pk100_encode_fp16(const float* source, long long elements, uint16_t* out);
int pk100_encode_fp16_linear(const float* source, long long logical_out, long long logical_in,
                             long long padded_out, long long padded_in, uint16_t* out);
int pk100_encode_fp32_bias(const float* source, long long logical, long long padded, float* out);
/* Returns 0 and sets *overflow (may be NULL) when the rounded value does not fit 64 bits. */
unsigned long long pk100_align_up(unsigned long long value, unsigned long long alignment, int* overflow);

/* ------------------------------------------------------------------------
 * Packed-layout size contract: padded shapes and byte counts of the candidate weight formats
 * (host code, pure integers).  Replaces LinearFormat / LinearLayout / estimate_linear /
 * TILE_ALIGNMENT (src/packing.rs:5-130) and Exl3Layout (src/exl3.rs:14-75), with which a host
 * sizes weight buffers before anything is packed.
 *   FP16: 2 * in^128 * out^128 payload bytes; FP8_E4M3 / INT8: in^128 * out^128 payload + 4 * out^128
 *   bytes of fp32 row scales; Q4_K: out * (in / 256) * 144 bytes, unpadded, not available when
 *   in % 256 != 0 (`available` = 0, the reference's Ok(None)); EXL3: in^128 * out^128 * bits / 8
 *   trellis bytes + 2 * (in^128 + out^128) scale bytes, trellis shape [in^128/16, out^128/16, 16*bits].
 * Errors: PK100_ERR_SHAPE for a zero dimension (PackingError::Empty), PK100_ERR_UNSUPPORTED for an
 * unknown format or an EXL3 rate outside 1..8 bits (InvalidBitRate), PK100_ERR_LIMIT on overflow. */
enum {
    PK100_FORMAT_FP16 = 0, PK100_FORMAT_FP8_E4M3 = 1, PK100_FORMAT_INT8 = 2,
    PK100_FORMAT_Q4_K = 3, PK100_FORMAT_EXL3 = 4
};
typedef struct pk100_linear_layout {
    long long logical_in, logical_out, padded_in, padded_out;
    unsigned long long payload_bytes, metadata_bytes;
    int available;
} pk100_linear_layout;
typedef struct pk100_exl3_layout_t {
    long long padded_in, padded_out, trellis_shape[3];
    unsigned long long trellis_bytes, scale_bytes;
} pk100_exl3_layout_t;
int pk100_estimate_linear(int format, long long logical_in, long long logical_out, int exl3_bits,
                          pk100_linear_layout* out);
int pk100_exl3_layout(long long logical_in, long long logical_out, int qbits, pk100_exl3_layout_t* out);

/* ------------------------------------------------------------------------
 * Log-mel frontend: PCM fp32 [utterances, sample_stride] (sample_counts[u] samples each,
 * device int array) -> normalised log-mel fp32 [utterances, frame_cap, 128], the input
 * layout of pk100_run_subsampling.  Utterance u has sample_counts[u] / 160 + 1 frames of
 * which the first sample_counts[u] / 160 are valid; every other row of its block is zero;
 * valid_frames (device int [utterances], may be NULL) receives the valid counts.
 * Needs frame_cap >= sample_stride / 160 + 1.
 * Replaces run_frontend (src/cuda/frontend.rs:230-316) with pk_sm89_frame_window, the cuFFT
 * R2C plan, pk_sm89_mel_log_sparse and pk_sm89_normalize_mel (kernels/sm89/frontend.cu);
 * definition: CpuMelFrontend::compute (src/frontend.rs:114-215).  The pinned configuration
 * only: 512-point FFT, hop 160, 128 mel bins, centred, power spectrum, per-feature
 * normalisation (src/config.rs:154-173).
 * window: the 400-tap window centred in 512 values (center_window, src/frontend.rs:218-223);
 * filters: the non-zero entries of the [128, 257] filter bank row by row (offsets [129],
 * bins and values [offsets[128]]), as sparse_filters builds them (src/cuda/frontend.rs:196-228). */
typedef struct pk100_frontend_weights {
    const float* window;            /* device fp32 [512] */
    const int* filter_offsets;      /* device int [129] */
    const int* filter_bins;         /* device int [nonzeros] */
    const float* filter_values;     /* device fp32 [nonzeros] */
    float preemphasis, log_zero_guard, normalize_epsilon;   /* 0.97, 2^-24, 1e-5 */
} pk100_frontend_weights;

int pk100_mel_frames_for(int samples);   /* samples / 160 + 1, or 0 for no samples */
int pk100_mel_frontend(void* stream, const pk100_frontend_weights* weights, const float* samples,
                       int utterances, long long sample_stride, const int* sample_counts, float* mel,
                       int frame_cap, int* valid_frames);

#ifdef __cplusplus
}
#endif

#endif /* PK100_H_ */
