/*
 * mgx_cuda.h - C ABI of the sm_100a kernel library behind the MIGraphX `cuda` target.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t; NULL = the legacy default stream),
 * enqueues work on that stream and returns without synchronising.
 *
 * Return value: 0 on success; a negative MGX_E_* code when the arguments are
 * rejected on the host before anything is launched; a positive value is a
 * cudaError_t reported by the CUDA runtime/driver.  Nothing throws across
 * this boundary.  There is no CPU fallback: an unsupported case is an error.
 *
 * Device-side problems (a bounded wait inside a kernel ran out) are recorded
 * in a per-device status word, read with mgx_cuda_device_status().
 *
 * The reference has no C ABI at this level: its GPU target calls rocBLAS /
 * hipBLASLt / MLIR-generated kernels from C++ operator structs.  Each entry
 * point below names the reference interface it stands in for.
 */
#ifndef MGX_CUDA_H
#define MGX_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MGX_API __attribute__((visibility("default")))

/* ---- status codes ------------------------------------------------------ */
#define MGX_OK 0
#define MGX_E_INVALID_ARG (-1)   /* null pointer, negative size, bad enum           */
#define MGX_E_UNSUPPORTED (-2)   /* valid request this library has no kernel for    */
#define MGX_E_ALIGNMENT (-3)     /* pointer / leading dimension not aligned as req. */
#define MGX_E_WORKSPACE (-4)     /* workspace missing or too small                  */
#define MGX_E_TOO_LARGE (-5)     /* size beyond a documented fixed maximum          */
#define MGX_E_DRIVER (-6)        /* could not obtain a driver entry point           */
#define MGX_E_DEVICE_TIMEOUT (-7) /* a kernel's bounded wait expired (status word)  */

/* ---- element types (values are part of the ABI) ------------------------ */
typedef enum mgx_dtype
{
    MGX_F32        = 0,
    MGX_F16        = 1,
    MGX_I8         = 2,
    MGX_U8         = 3,
    MGX_I32        = 4,
    MGX_FP8_E4M3FN = 5,
    MGX_I64        = 6 /* indices of mgx_cuda_gather only */
} mgx_dtype;

/* How the fp32 scale operand of a fused dequantizelinear is indexed.  After
 * simplify_qdq the scale reaches the op as a full [M,N] broadcast view
 * (reference: src/simplify_qdq.cpp:243-248); the host recovers the mode from
 * the view's strides. */
typedef enum mgx_scale_mode
{
    MGX_SCALE_NONE       = 0, /* raw accumulator out (quant_dot alone)          */
    MGX_SCALE_PER_TENSOR = 1, /* scale[0]                                       */
    MGX_SCALE_PER_COL    = 2, /* scale[n], n = output column (per out channel)  */
    MGX_SCALE_PER_ROW    = 3  /* scale[m]                                       */
} mgx_scale_mode;

/* Activation applied after scale and bias (the fused `pointwise` module). */
typedef enum mgx_act
{
    MGX_ACT_NONE     = 0,
    MGX_ACT_RELU     = 1,
    MGX_ACT_GELU_ERF = 2, /* 0.5*x*(1+erf(x/sqrt(2)))  (src/op/builder/gelu.cpp:58-74) */
    MGX_ACT_GELU_TANH = 3,
    MGX_ACT_SILU     = 4
} mgx_act;

/* ---- quantizelinear ---------------------------------------------------- *
 * y[r,c] = clamp(rne(x[r,c] / scale[r,c]) + zp[r,c], lowest, max)  for int8/uint8,
 * y[r,c] = fp8(clamp(x/scale + zp, -448, 448))                     for fp8 e4m3fn.
 * Stands in for op::quantizelinear::compute
 * (src/include/migraphx/op/quantizelinear.hpp:71-108).
 * x is [rows, cols] with row stride ldx (elements); y likewise with ldy.
 * scale has x's type and is indexed scale[r*scale_strides[0] + c*scale_strides[1]]
 * (stride 0 = broadcast, as MIGraphX passes broadcast views); zp has y's type,
 * may be NULL (zero) and is indexed the same way with zp_strides.
 * x_type: MGX_F32 | MGX_F16.  y_type: MGX_I8 | MGX_U8 | MGX_FP8_E4M3FN. */
MGX_API int mgx_cuda_quantizelinear(const void* x,
                                    int x_type,
                                    int64_t ldx,
                                    const void* scale,
                                    const int64_t scale_strides[2],
                                    const void* zp,
                                    const int64_t zp_strides[2],
                                    void* y,
                                    int y_type,
                                    int64_t ldy,
                                    int64_t rows,
                                    int64_t cols,
                                    void* stream);

/* ---- generic element-wise operator ("next" row: the non-GEMM part of a program) --------- *
 * Evaluates a short list of scalar instructions per output element, the way
 * op::pointwise::compute (src/include/migraphx/op/pointwise.hpp:81-114) evaluates the
 * instructions of its sub-module: value i is input i for i < ninputs, otherwise the result of
 * instruction i - ninputs; the last instruction's result is the output.  Every result is
 * converted to its instruction's type before it is used again (MGX_F16: truncating, as
 * migraphx::half converts, src/include/migraphx/generic_float.hpp:180-230), so a chain of
 * fp16 operators rounds where the reference rounds.  Inputs are strided views of the output's
 * index space (stride 0 = broadcast); the output is a packed row-major tensor of `lens`. */
#define MGX_PW_MAXDIMS 5
#define MGX_PW_MAXIN 8
#define MGX_PW_MAXINSN 32

typedef enum mgx_pw_op {
    MGX_PW_ADD = 0, MGX_PW_SUB, MGX_PW_MUL, MGX_PW_DIV, MGX_PW_MIN, MGX_PW_MAX, MGX_PW_POW,
    MGX_PW_NEG, MGX_PW_ABS, MGX_PW_EXP, MGX_PW_LOG, MGX_PW_SQRT, MGX_PW_RSQRT, MGX_PW_RECIP,
    MGX_PW_TANH, MGX_PW_SIGMOID, MGX_PW_ERF, MGX_PW_RELU, MGX_PW_SIN, MGX_PW_COS,
    MGX_PW_FLOOR, MGX_PW_CEIL, MGX_PW_ROUND, MGX_PW_NEARBYINT,
    MGX_PW_CONVERT,    /* to the instruction's type */
    MGX_PW_WHERE,      /* src0 != 0 ? src1 : src2 */
    MGX_PW_CLIP,       /* min(max(src0, src1), src2) */
    MGX_PW_EQUAL, MGX_PW_GREATER, MGX_PW_LESS,
    MGX_PW_LEAKY_RELU, /* src0 > 0 ? src0 : src0 * imm */
    MGX_PW_CONST,      /* imm */
    MGX_PW_IDENTITY,
    MGX_PW_OP_COUNT
} mgx_pw_op;

typedef struct mgx_pw_insn {
    int32_t op;       /* mgx_pw_op */
    int32_t type;     /* mgx_dtype of the result (MGX_I8 also stands for bool) */
    int32_t src[3];   /* indices of the operand values */
    float imm;
} mgx_pw_insn;

typedef struct mgx_pw_desc {
    int32_t ndim;                       /* 1 .. MGX_PW_MAXDIMS */
    int32_t ninputs;                    /* 0 .. MGX_PW_MAXIN */
    int32_t ninsns;                     /* 1 .. MGX_PW_MAXINSN */
    int32_t reserved;
    int64_t lens[MGX_PW_MAXDIMS];       /* output dimensions */
    int32_t in_type[MGX_PW_MAXIN];      /* mgx_dtype of every input */
    int64_t in_strides[MGX_PW_MAXIN][MGX_PW_MAXDIMS]; /* in elements */
    mgx_pw_insn insn[MGX_PW_MAXINSN];
} mgx_pw_desc;

/* inputs: ninputs device pointers.  out: packed tensor of the last instruction's type. */
MGX_API int mgx_cuda_pointwise(const mgx_pw_desc* d, const void* const* inputs, void* out, void* stream);

/* ---- reductions over the last axis and softmax ("next" rows: LayerNorm, attention) ------ *
 * x is [rows, cols] with row stride ldx (elements), y[rows] packed.  Stands in for
 * op::reduce_sum / reduce_mean / reduce_max / reduce_min (src/include/migraphx/op/reduce_op.hpp:
 * 180-203: the reference accumulates in double; here fp32 partial sums are combined as a tree,
 * within 1e-6 relative of it) restricted to the innermost axis.  Types: MGX_F32 | MGX_F16,
 * the result has x's type (fp16: truncating conversion). */
typedef enum mgx_reduce_op { MGX_REDUCE_SUM = 0, MGX_REDUCE_MEAN = 1, MGX_REDUCE_MAX = 2, MGX_REDUCE_MIN = 3 } mgx_reduce_op;

MGX_API int mgx_cuda_reduce(const void* x, int type, int64_t ldx, int64_t rows, int64_t cols, int op,
                            void* y, void* stream);

/* y[r, c] = exp(x[r, c] - max_c x[r, :]) / sum_c exp(...), over the innermost axis, with the
 * reference's intermediate roundings (ref_softmax, src/targets/ref/lowering.cpp:253-320: the
 * exponentials are stored in the output type before they are summed and divided). */
MGX_API int mgx_cuda_softmax(const void* x, int type, int64_t ldx, void* y, int64_t ldy, int64_t rows,
                             int64_t cols, void* stream);

/* ---- LayerNorm over the last axis, one launch ("next" row: the encoder's LayerNorms) ----- *
 * y = (x - mean) * rsqrt(var + eps) * gamma + beta per row of x [rows, cols] (row strides in
 * elements), optionally followed by a per-tensor quantizelinear of y written to q (int8 or
 * fp8 e4m3fn, the next quantized linear's input); y or q may be NULL when only the other is
 * wanted.  gamma / beta: [cols] in x's type, or NULL.  Stands in for the instruction chain of
 * src/onnx/parse_layernorm.cpp:100-140 (reduce_mean, sub, mul, reduce_mean, add, rsqrt, mul, mul,
 * add) and keeps those operators' roundings: with MGX_F16 every intermediate is truncated to half
 * like migraphx::half arithmetic.  Types: MGX_F32 | MGX_F16; cols a multiple of 4 (fp32) / 8
 * (fp16) and at most 8192 / 16384 (mgx_cuda_layernorm_supported); 16-byte aligned rows.  A warp per row,
 * or a block per row where there are few rows or long ones. */
typedef struct mgx_layernorm_desc
{
    int64_t rows, cols;
    int64_t ldx, ldy, ldq;
    int32_t type;   /* mgx_dtype of x, gamma, beta and y */
    float eps;
    int32_t q_type; /* mgx_dtype of q (MGX_I8 | MGX_FP8_E4M3FN); ignored when q == NULL */
    float q_scale;
    float q_zero_point;
    int32_t flags;  /* 0 | MGX_LAYERNORM_RMS */
} mgx_layernorm_desc;
/* RMS normalisation as the SimplifiedLayerNormalization parser decomposes it
 * (src/onnx/parse_simplified_layer_normalization.cpp:91-106): y = x * rsqrt(mean(float(x)^2) + eps) *
 * gamma; the squares and their mean in fp32, the mean, the sum with eps, the rsqrt and the two products
 * stored in x's type.  beta must be NULL. */
#define MGX_LAYERNORM_RMS 1

MGX_API int mgx_cuda_layernorm_supported(int type, int64_t cols);
MGX_API int mgx_cuda_layernorm(const mgx_layernorm_desc* d, const void* x, const void* gamma, const void* beta,
                               void* y, void* q, void* stream);
/* The same with a third result: dq = dequantizelinear(q, dq_scale, zero point) in x's type
 * ((q - zero point) * dq_scale, fp16: truncated), the dequantised copy simplify_qdq makes other
 * readers of a quantised tensor use (src/simplify_qdq.cpp:401-432).  Needs q, int8 only. */
MGX_API int mgx_cuda_layernorm_ex(const mgx_layernorm_desc* d, const void* x, const void* gamma, const void* beta,
                                  void* y, void* q, void* dq, int64_t lddq, float dq_scale, void* stream);

/* ---- multi-head attention on fp16 tensors, one launch ("next" row: encoder attention) ---- *
 * o[b*seq + i, h*64 .. h*64+63] = softmax_j(scale * <q_i, k_j>) . v_j per batch b and head h,
 * no mask.  q, k, v: row-strided [batch*seq, heads*64] fp16 matrices (a head is a 64-column
 * slice of a row; ld* in elements, 16-byte aligned rows), read in place.  o (fp16) and / or oq
 * (int8: the per-tensor quantizelinear of the fp16 result) receive the merged-heads result.
 * Stands in for reshape -> transpose -> dot -> mul -> softmax -> dot -> transpose -> reshape of an
 * encoder layer (the reference fuses the same chain for its GPU target,
 * src/targets/gpu/fuse_mlir.cpp:1161-1234).  head_dim must be 64.  The kernel keeps the chain's own
 * roundings (scores, exponentials and probabilities rounded to half where the operators store them,
 * ref_softmax's order of operations): results are the reference's halves except for about one
 * element in a hundred (neighbouring halves, from the order of the fp32 sums and the last bit of
 * exp). */
typedef struct mgx_attention_desc
{
    int64_t batch, seq, heads, head_dim;
    int64_t ldq, ldk, ldv, ldo, ldoq;
    float scale;
    float q_scale;      /* quantizelinear scale / zero point of oq; ignored when oq == NULL */
    float q_zero_point;
    int32_t flags;      /* MGX_ATTENTION_* bits, 0 for none */
} mgx_attention_desc;

/* Run the softmax in fp32 over key blocks (running maximum and sum, one pass over the keys)
 * instead of making the operator chain's half roundings: results within the fp16
 * tolerance (rtol 2e-2 / atol 1e-2) of the chain instead of (nearly) its bits. */
#define MGX_ATTENTION_FP32_SOFTMAX 1
/* The chain's roundings without the score buffer in shared memory that sequences of up to 1024
 * keys use: three passes over the keys, the scores recomputed on the tensor cores in each.  What
 * longer sequences always run (measured at 384 keys: 42 us against 39 us with the buffer). */
#define MGX_ATTENTION_THREE_PASS 2

MGX_API int mgx_cuda_attention(const mgx_attention_desc* d, const void* q, const void* k, const void* v, void* o,
                               void* oq, void* stream);

/* ---- decoder KV cache and rotary embedding ("next" rows: Llama-shaped layers) ------------- *
 * concat_past_present: the new keys / values of a step, present [batch, kv_heads, seq, head]
 * (byte strides along batch / head / row in present_strides, rows contiguous), are copied into
 * the cache past [batch, kv_heads, cache_seq, head] in place: at row seqlens[b] of every head when
 * seq == 1 (decode), at row 0 otherwise (prompt).  Stands in for op::concat_past_present::compute
 * (src/include/migraphx/op/concat_past_present.hpp:84-155).  Rows that would fall beyond
 * cache_seq are not written.  seqlens_type: MGX_I32 | MGX_I64. */
MGX_API int mgx_cuda_concat_past_present(const void* present, const int64_t present_strides[3], int64_t batch,
                                         int64_t kv_heads, int64_t seq, int64_t head_bytes, const void* seqlens,
                                         int seqlens_type, void* past, int64_t cache_seq, void* stream);

/* gqa_rotary_embedding: rotary position embedding of the Q and K heads of a packed
 * [batch, heads + 2 kv_heads, seq, head] tensor (V heads and columns beyond rotary_dim pass
 * through), positions s (prompt) or seqlens[b] (decode, seq == 1), cos / sin caches
 * [max_seq, rotary_dim / 2] in the tensor's type.  Stands in for
 * op::gqa_rotary_embedding::compute (src/include/migraphx/op/gqa_rotary_embedding.hpp:72-221) with
 * its roundings.  type: MGX_F16 | MGX_F32. */
MGX_API int mgx_cuda_gqa_rotary_embedding(const void* qkv, int type, int64_t batch, int64_t heads, int64_t kv_heads,
                                          int64_t seq, int64_t head, const void* cos_cache, const void* sin_cache,
                                          int64_t max_seq, int64_t rotary_dim, const void* seqlens, int seqlens_type,
                                          int interleaved, void* out, void* stream);

/* The rotation of the rotary_embedding builder, non-interleaved
 * (src/op/builder/rotary_embedding.cpp:60-230: gathernd of the cos / sin rows at the positions,
 * rotate-half, mul, mul, mul, add) as one launch with that chain's roundings: out = x * cos +
 * concat(x[half:], x[:half]) * (signs * sin), every product and the sum stored in the tensor's type.
 * x: [batch, heads, seq, head] with element strides x_strides = {batch, head, row} (rows
 * contiguous); positions [batch * seq] (MGX_I32 | MGX_I64); caches [max_pos, head / 2] in x's type;
 * out packed.  type: MGX_F16 | MGX_F32. */
MGX_API int mgx_cuda_rotary_embedding(const void* x, int type, const int64_t x_strides[3], int64_t batch,
                                      int64_t heads, int64_t seq, int64_t head, const void* positions,
                                      int positions_type, const void* cos_cache, const void* sin_cache,
                                      int64_t max_pos, void* out, void* stream);

/* Decode-step attention against the fp16 KV cache, one launch: for every batch entry b and query
 * head h (sharing KV head h / (heads / kv_heads)), softmax(scale * q K^T) V over the cache
 * positions 0 .. seqlens[b], positions beyond it masked out.  Stands in for the operator chain
 * the GroupQueryAttention parser emits after concat_past_present
 * (src/onnx/parse_group_query_attention.cpp:184-262: KV-head broadcast, dot, mul, where, softmax,
 * dot) with that chain's fp16 roundings.  q: rows of `head` halves at q + b * q_batch_stride +
 * h * q_head_stride (elements); caches packed [batch, kv_heads, cache_seq, head], 16-byte aligned;
 * out packed [batch, heads * head].  head: 64 | 128; heads / kv_heads: 1 | 2 | 4 | 8.
 * MGX_E_TOO_LARGE when a CTA's share of the cache positions does not fit shared memory
 * (mgx_cuda_gqa_decode_supported tells beforehand). */
typedef struct mgx_gqa_decode_desc
{
    int64_t batch, heads, kv_heads, head, cache_seq;
    int64_t q_batch_stride, q_head_stride;
    float scale;
    int32_t seqlens_type; /* MGX_I32 | MGX_I64 */
} mgx_gqa_decode_desc;
MGX_API int mgx_cuda_gqa_decode_attention(const mgx_gqa_decode_desc* d, const void* q, const void* k_cache,
                                          const void* v_cache, const void* seqlens, void* out, void* stream);
MGX_API int mgx_cuda_gqa_decode_supported(int64_t batch, int64_t heads, int64_t kv_heads, int64_t head,
                                          int64_t cache_seq);

/* ---- gather, concat (byte movers of the "next" rows: embeddings, KV-cache append) -------- *
 * out[o, j, :] = data[o, indices[j], :] for o < outer, j < nidx, rows of inner_bytes bytes:
 * op::gather (src/include/migraphx/op/gather.hpp:107-150) on a packed tensor whose dimensions
 * before / after the axis are folded into outer / inner_bytes.  Negative indices count from the
 * end; an index out of range gives zeros (the reference throws on the host).
 * index_type: MGX_I32 | MGX_I64. */
MGX_API int mgx_cuda_gather(const void* data, int64_t outer, int64_t axis_len, int64_t inner_bytes,
                            const void* indices, int index_type, int64_t nidx, void* out, void* stream);

/* dst[r, 0:row_bytes] = src[r, 0:row_bytes] for r < rows with independent row pitches (bytes):
 * one input of op::concat (src/include/migraphx/op/concat.hpp:147-163) copied into its slice of
 * the packed result. */
MGX_API int mgx_cuda_copy_rows(const void* src, int64_t src_pitch, void* dst, int64_t dst_pitch,
                               int64_t rows, int64_t row_bytes, void* stream);

/* ---- dequantizelinear -------------------------------------------------- *
 * y = (x - zp) * scale, output type = scale type (MGX_F32 | MGX_F16).
 * Stands in for op::dequantizelinear::compute
 * (src/include/migraphx/op/dequantizelinear.hpp:60-82).
 * x_type: MGX_I8 | MGX_U8 | MGX_I32 | MGX_FP8_E4M3FN. */
MGX_API int mgx_cuda_dequantizelinear(const void* x,
                                      int x_type,
                                      int64_t ldx,
                                      const void* scale,
                                      int scale_type,
                                      const int64_t scale_strides[2],
                                      const void* zp,
                                      const int64_t zp_strides[2],
                                      void* y,
                                      int64_t ldy,
                                      int64_t rows,
                                      int64_t cols,
                                      void* stream);

/* ---- unpack_int4 / pack_int4 (stand-alone form) ------------------------ *
 * unpack: out[r, 2i] = in[r,i] & 0xF, out[r, 2i+1] = in[r,i] >> 4 (sign-extended
 * when type is MGX_I8).  Reference: op::unpack_int4::compute
 * (src/include/migraphx/op/unpack_int4.hpp:75-120), HIP kernel
 * src/targets/gpu/kernels/include/migraphx/kernels/unpack_int4.hpp:33-54.
 * pack is the inverse with clipping to the 4-bit range
 * (src/include/migraphx/op/pack_int4.hpp:79-123).  The axis is the last one. */
MGX_API int mgx_cuda_unpack_int4(const void* in, void* out, int type, int64_t rows,
                                 int64_t packed_cols, void* stream);
MGX_API int mgx_cuda_pack_int4(const void* in, void* out, int type, int64_t rows,
                               int64_t packed_cols, void* stream);

/* ---- quant_dot (+ fused dequantizelinear / bias / activation / residual) *
 * D[b] = epilogue(A[b] . B[b]) for b < batch.
 * A is [M,K], row stride lda, K contiguous.  B is the quant_dot right operand:
 *   b_layout = MGX_B_KN : [K,N], row stride ldb, N contiguous (MIGraphX default)
 *   b_layout = MGX_B_NK : [N,K], row stride ldb, K contiguous (a transpose view)
 * ab_type MGX_I8 accumulates exactly in int32; MGX_FP8_E4M3FN accumulates in fp32.
 * ab_type MGX_F16 is op::dot on fp16 operands (attention, un-quantised linears): fp32
 * accumulation, out_type MGX_F16 (truncating conversion) or MGX_F32, scale_mode NONE as a rule,
 * no fused quantizelinear; lda, ldb and the batch strides are multiples of 8 elements.
 * Epilogue, in this order (it is the order of the fused pointwise module
 * `dequantizelinear -> add(bias) -> act -> add(residual)`):
 *   v = acc                                   (int32 or fp32)
 *   if scale_mode != NONE: v = float(acc) * scale[..]   (fp32 multiply, one rounding)
 *   if bias:     v = v + bias[n]              (fp32 vector of N, separate add)
 *   v = act(v)
 *   if residual: v = v + float(residual[m,n]) (same type/ld as D)
 *   D = out_type(v)
 * out_type: MGX_I32 (only ab_type I8, scale NONE, no bias/act/residual: the raw
 * quant_dot result), MGX_F32, MGX_F16.
 * Stands in for rocblas_gemm<op::quant_dot>::compute
 * (src/targets/gpu/include/migraphx/gpu/gemm.hpp:109-127), hip_gemm for fp8
 * (src/targets/gpu/include/migraphx/gpu/hip_gemm.hpp:44-141) and the
 * gemm+pointwise fusion of src/targets/gpu/fuse_mlir.cpp:709-807; arithmetic
 * follows ref_quant_gemm (src/targets/ref/lowering.cpp:205-249, src/gemm.cpp:43-63).
 * Requirements: A, B, D 16-byte aligned; lda, ldb multiples of 16 elements.
 * With b_layout = MGX_B_KN a workspace of mgx_cuda_qgemm_workspace() bytes is
 * needed (B is re-laid out K-contiguous once per call); constant weights should
 * be transposed once with mgx_cuda_transpose_8bit() and passed as MGX_B_NK. */
typedef enum mgx_b_layout
{
    MGX_B_KN = 0,
    MGX_B_NK = 1
} mgx_b_layout;

typedef struct mgx_qgemm_desc
{
    int64_t M, N, K;
    int64_t batch;
    int64_t lda, ldb, ldd;                 /* row strides, elements          */
    int64_t stride_a, stride_b, stride_d;  /* batch strides, elements        */
    int32_t ab_type;                       /* MGX_I8 | MGX_FP8_E4M3FN | MGX_F16 */
    int32_t out_type;                      /* MGX_I32 | MGX_F32 | MGX_F16    */
    int32_t b_layout;                      /* mgx_b_layout                   */
    int32_t scale_mode;                    /* mgx_scale_mode                 */
    int32_t act;                           /* mgx_act                        */
    int32_t flags;                         /* MGX_QGEMM_* bits, 0 for none   */
} mgx_qgemm_desc;

/* out_type MGX_F16 only: the operators after dequantizelinear run in half, as in an fp16 model
 * (src/simplify_qdq.cpp:283-287 converts the dequantised value to half first): the dequantised
 * value, the bias sum, every step of the erf-GELU ((x * 0.5) * (erf(x / half(sqrt 2)) + 1),
 * src/op/builder/gelu.cpp:58-74) and the residual sum are each truncated to half like
 * migraphx::half arithmetic.  Without the flag they are fp32 operations and only the final
 * value is converted. */
#define MGX_QGEMM_HALF_MATH 1

MGX_API size_t mgx_cuda_qgemm_workspace(const mgx_qgemm_desc* desc);
MGX_API int mgx_cuda_qgemm(const mgx_qgemm_desc* desc,
                           const void* A,
                           const void* B,
                           void* D,
                           const float* scale,
                           const float* bias,
                           const void* residual,
                           void* workspace,
                           size_t workspace_bytes,
                           void* stream);

/* quant_dot whose epilogue also (or only) writes quantizelinear(D): the pointwise module
 * `dequantizelinear -> add -> act -> [add] -> quantizelinear` that fuse_pointwise forms when
 * the next operator is another quantized GEMM (src/fuse_pointwise.cpp:91-139).  The
 * quantizelinear has a per-tensor scale (given in D's type, as the operator takes it) and
 * zero point: q = saturate(rne(D / scale) + zero_point) for MGX_I8, fp8(clamp(D / scale +
 * zero_point)) for MGX_FP8_E4M3FN, computed from the value D holds (after the conversion to
 * out_type).  D may be NULL when only the quantized tensor is needed. */
typedef struct mgx_qgemm_qout
{
    void* q;            /* [M,N] per batch, 8-bit                 */
    int64_t ldq;        /* row stride, elements                   */
    int64_t stride_q;   /* batch stride, elements                 */
    int32_t q_type;     /* MGX_I8 | MGX_FP8_E4M3FN                */
    float scale;        /* > 0                                    */
    float zero_point;   /* integral for MGX_I8                    */
    int32_t flags;      /* 0 | MGX_QOUT_LUT                       */
    /* MGX_QOUT_LUT (fp16 result with MGX_QGEMM_HALF_MATH, q is the only output, no residual): the
     * activation and the quantizelinear are one table look-up.  lut[h] is the quantised byte for the
     * value whose fp16 bit pattern is h after dequantizelinear and bias: 65536 bytes in device memory
     * that the caller filled with activation + quantizelinear of every half (what a chain of fp16
     * operators makes of it, desc->act included).  The table is used where the launch takes the
     * epilogue's vector path (M a multiple of 128, N of 16, aligned rows), otherwise the same values
     * are computed.  Read only when the flag is set. */
    const void* lut;
} mgx_qgemm_qout;
#define MGX_QOUT_LUT 1

MGX_API int mgx_cuda_qgemm_ex(const mgx_qgemm_desc* desc,
                              const void* A,
                              const void* B,
                              void* D,
                              const float* scale,
                              const float* bias,
                              const void* residual,
                              const mgx_qgemm_qout* qout,
                              void* workspace,
                              size_t workspace_bytes,
                              void* stream);

/* The same operation for callers that must not allocate device memory and have no buffer
 * of their own to lend: a runtime that carved up all device memory when the model was
 * compiled (MIGraphX plans one arena per program and never allocates during eval), a
 * serving loop in which cudaMalloc's implicit device synchronisation is not acceptable, or
 * a host with a fixed memory budget.  It has no counterpart in the reference.
 * The scratch of the call - the re-laid-out copy of a [K,N] right operand (b_layout =
 * MGX_B_KN), or the tile counters and partial sums of the weight-streaming kernel that
 * [N,K] operands with at most 16 rows take - goes into a fixed
 * 16 MiB array that is part of this library's device image: every GPU that loads the
 * library holds those 16 MiB until the process exits.  Requests whose
 * mgx_cuda_qgemm_workspace() exceeds mgx_cuda_qgemm_static_scratch_limit() are rejected
 * with MGX_E_TOO_LARGE when the operand is [K,N]; with [N,K] operands (whose scratch is
 * optional) they run as tiles without scratch instead.  No cudaMalloc / cudaFree / allocating library routine is called.
 * The first call on each device looks the array's device address up (one cheap runtime
 * query); make that first call before starting a stream capture on that device.
 * All calls on a device share the one array: two calls whose kernels may overlap on the
 * GPU (different streams without an ordering between them) race on it; calls on one stream
 * are safe.  The array keeps the previous call's bytes; what has to start at
 * zero (the tile counters of the weight-streaming kernel) is cleared by the call itself,
 * and every other byte the kernels read is rewritten by the same call first. */
MGX_API size_t mgx_cuda_qgemm_static_scratch_limit(void);
MGX_API int mgx_cuda_qgemm_static_scratch(const mgx_qgemm_desc* desc,
                                          const void* A,
                                          const void* B,
                                          void* D,
                                          const float* scale,
                                          const float* bias,
                                          const void* residual,
                                          void* stream);

/* [rows, cols] bytes -> [cols, rows] bytes, per batch (dense, ld = cols / rows).
 * Used once per constant weight so that quant_dot's [K,N] operand becomes
 * K-contiguous (the reference does the equivalent with its column-major trick,
 * src/targets/gpu/gemm_impl.cpp:343-351). */
MGX_API int mgx_cuda_transpose_8bit(const void* src, void* dst, int64_t rows, int64_t cols,
                                    int64_t batch, void* stream);

/* ---- weight-only int4 linear: unpack_int4 + dequantizelinear + dot ------ *
 * D[M,N] = A[M,K] (fp16) . W^T where W[n,k] = fp16((q[n,k] - zp) * s[n, k/group]),
 * q unpacked from Bp[N, K/2] bytes (low nibble = even k;
 * src/include/migraphx/op/unpack_int4.hpp:108-115), s fp16 [N, K/group], zp either
 * the constant zp_const (zp == NULL; 8 is the MatMulNBits default,
 * src/onnx/parse_matmulnbits.cpp:122) or uint8 [N, K/group].  fp32 accumulate,
 * fp16 out.  This is the IR parse_matmulnbits emits
 * (src/onnx/parse_matmulnbits.cpp:85-158) and what the reference fuses in
 * src/targets/gpu/fuse_mlir.cpp:1236-1276.
 * gemv: decode (M <= 16), split-K through the workspace (mgx_cuda_w4a16_workspace bytes).
 * gemm: any M (prefill); needs K % 128 == 0 and group % 128 == 0.  mgx_cuda_w4a16() picks. */
typedef struct mgx_w4_desc
{
    int64_t M, N, K;
    int64_t lda, ldd;  /* row strides of A and D, elements */
    int32_t group;     /* quantisation group along K (multiple of 32; 128 typical) */
    int32_t zp_const;  /* used when zp == NULL */
    int32_t act;       /* mgx_act, applied to the fp32 accumulator before the fp16 store */
    int32_t reserved;
} mgx_w4_desc;

MGX_API size_t mgx_cuda_w4a16_workspace(const mgx_w4_desc* desc);
MGX_API int mgx_cuda_w4a16_gemv(const mgx_w4_desc* desc, const void* A, const void* Bp,
                                const void* scales, const void* zp, void* D, void* workspace,
                                size_t workspace_bytes, void* stream);
MGX_API int mgx_cuda_w4a16_gemm(const mgx_w4_desc* desc, const void* A, const void* Bp,
                                const void* scales, const void* zp, void* D, void* workspace,
                                size_t workspace_bytes, void* stream);
MGX_API int mgx_cuda_w4a16(const mgx_w4_desc* desc, const void* A, const void* Bp,
                           const void* scales, const void* zp, void* D, void* workspace,
                           size_t workspace_bytes, void* stream);

/* ---- tensor-parallel exchange -------------------------------------------- *
 * In-place sum all-reduce over NCCL (NVLink / NVSwitch) on the caller's stream: the exchange
 * step after the row-split linears (o_proj, down_proj) of a tensor-parallel int4 decoder.
 * The reference has no collective; there is no counterpart.  NCCL is loaded at run time
 * (libnccl.so.2 or $MGX_NCCL_LIB); MGX_E_DRIVER if it cannot be found, 2000 + ncclResult_t
 * on an NCCL error.  One communicator per process (one process per GPU): rank 0 obtains a
 * 128-byte id with mgx_cuda_comm_unique_id() and hands it to the other ranks out of band.
 * comm == NULL in mgx_cuda_all_reduce means the process default set with
 * mgx_cuda_comm_set_default() (what the cuda::all_reduce operator uses). */
MGX_API int mgx_cuda_comm_unique_id(void* id128);
MGX_API int mgx_cuda_comm_create(const void* id128, int nranks, int rank, void** comm);
MGX_API int mgx_cuda_comm_destroy(void* comm);
MGX_API void mgx_cuda_comm_set_default(void* comm);
MGX_API void* mgx_cuda_comm_default(void);
MGX_API int mgx_cuda_all_reduce(void* buf, size_t count, int dtype, void* comm, void* stream);

/* ---- device status ------------------------------------------------------ *
 * Reads and clears the current device's status word (synchronises the device).
 * *status = 0 when no kernel reported a problem; otherwise a code whose low 8
 * bits say which wait gave up (1 = TMA full barrier, 2 = stage-empty barrier,
 * 3 = accumulator-ready barrier, 4 = accumulator-free barrier). */
MGX_API int mgx_cuda_device_status(int* status);

/* Self-test of the bounded waits: launches one thread that waits at most limit_ns
 * (1 .. 1e8) nanoseconds on a barrier phase that nothing completes.  The wait gives up the
 * way every kernel's waits do: it records code 99 in the device status word (read it with
 * mgx_cuda_device_status) and the kernel returns normally; *gave_up (a device uint32, may
 * be NULL) receives 99.  Nothing faults and the context stays usable.  No counterpart in
 * the reference (its kernels have no bounded waits). */
MGX_API int mgx_cuda_selftest_bounded_wait(uint64_t limit_ns, void* gave_up, void* stream);

/* Human-readable text for a return value of this library. */
MGX_API const char* mgx_cuda_status_string(int code);

/* Library build tag: "sm_100a" plus the kernel set version. */
MGX_API const char* mgx_cuda_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MGX_CUDA_H */
