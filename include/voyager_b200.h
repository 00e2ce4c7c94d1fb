/*
 * voyager_b200 -- C ABI of the B200 (sm_100a) kernels behind the `quantized_ops` operators of
 * voyager-compiler.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (as void*), returns 0
 * on success or a negative vq_status, never throws and never synchronises the stream.  After a
 * non-zero return vq_last_error() gives a message for the calling thread.  All tensors are
 * dense and contiguous in logical (row-major) order; outputs are written in full and inputs are
 * never modified.  Citations name the upstream function each entry point replaces, by path
 * inside the voyager-compiler source tree.
 */
#ifndef VOYAGER_B200_H
#define VOYAGER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VQ_ABI_VERSION 2

#if defined(__GNUC__)
#define VQ_API __attribute__((visibility("default")))
#else
#define VQ_API
#endif

typedef enum vq_status {
    VQ_OK = 0,
    VQ_ERR_INVALID = -1,      /* bad argument (null pointer, size, alignment, dtype) */
    VQ_ERR_UNSUPPORTED = -2,  /* valid upstream usage this build has no kernel for */
    VQ_ERR_CUDA = -3,         /* a CUDA runtime call or launch failed */
    VQ_ERR_DEVICE = -4        /* a kernel reported a bounded wait that ran out */
} vq_status;

typedef enum vq_dtype { VQ_F32 = 0, VQ_BF16 = 1 } vq_dtype;

/* How a 16-bit bf16 pattern is turned into an output value (upstream: the 65 536-entry `qmap`
 * argument, src/voyager_compiler/quantization/fake_quantize.py:30-98). */
typedef enum vq_table_kind {
    VQ_TABLE_NONE = 0,
    VQ_TABLE_LUT16 = 1,  /* lut16[pattern] is the bf16 bit pattern of the output value */
    VQ_TABLE_INT = 2,    /* table is known to equal clamp(round_half_even(v), lo, hi), NaN -> NaN */
    VQ_TABLE_RUNS = 3    /* piecewise constant over the ordered finite bf16 line with <= 512 runs:
                            branchless binary search over run starts held in shared memory;
                            +inf, -inf and NaN inputs have their own outputs */
} vq_table_kind;

typedef struct vq_table {
    int32_t kind;
    int32_t n_runs;            /* RUNS: number of runs (1..512) */
    const uint16_t* lut16;     /* LUT16: device pointer, 65 536 entries */
    const uint8_t* lut8;       /* optional (any kind but INT): device pointer, 65 536 packed codes */
    float lo, hi;              /* INT */
    const uint16_t* run_keys;  /* RUNS: device pointer, n_runs-1 ascending run starts, in the
                                  order-preserving key space key = bits ^ (bits&0x8000 ? 0xFFFF : 0x8000) */
    const uint16_t* run_vals;  /* RUNS: device pointer, n_runs output bf16 patterns */
    const uint8_t* run_codes;  /* RUNS, optional: n_runs packed codes */
    uint16_t nan_val;          /* RUNS: output patterns for NaN, +inf and -inf inputs */
    uint16_t pinf_val;
    uint16_t ninf_val;
    uint8_t nan_code;          /* RUNS: packed codes for NaN, +inf and -inf inputs */
    uint8_t pinf_code;
    uint8_t ninf_code;
    uint8_t nan_uniform;       /* LUT16: non-zero when every NaN input pattern has the same output, which
                                  lets the kernels use the hardware bf16 conversion (NaN -> 0x7FFF) */
    uint8_t flat_tiny;         /* LUT16: non-zero when the table is constant over the patterns 0x0000..0x0400 and
                                  over 0x8000..0x8400 (|value| <= 2^-119), so that the rounding of a quotient
                                  in the subnormal range cannot change the result; lets bf16 kernels divide
                                  by multiplying with a reciprocal without scanning for tiny elements.
                                  0 is always safe. */
    uint8_t reserved[5];
    const float* levels2;      /* optional, with lut8: device pointer, 512 fp32 entries: the output value of packed
                                  code c for an input pattern without the sign bit at [c], with it at [256 + c].
                                  Only set when lut16[p] == levels2[lut8[p] + 256 * (p >> 15)] holds for every
                                  pattern p (the host checks it): the value then follows from the code and the
                                  input's sign, and kernels need the 64 KB code table alone in shared memory. */
} vq_table;

/* Where the scale (and zero point) of element i lives (upstream `expand`,
 * src/voyager_compiler/ops/quantized.py:82-95, and plain broadcasting when block_size is None). */
typedef enum vq_scale_mode {
    VQ_SCALE_SCALAR = 0,    /* one scale for the whole tensor */
    VQ_SCALE_ROWBLOCK = 1,  /* tensor viewed as [rows, K]; scale is [rows, ceil(K/block)] */
    VQ_SCALE_STRIDED = 2    /* general: per-dimension block divisor and scale stride */
} vq_scale_mode;

typedef struct vq_scale_layout {
    int32_t mode;
    int32_t ndim;            /* STRIDED: 1..6 */
    int64_t rows, K, block;  /* ROWBLOCK */
    int64_t size[6];         /* STRIDED: tensor sizes, outermost first */
    int64_t div[6];          /* STRIDED: coordinate divisor per dim (block size, or 1) */
    int64_t stride[6];       /* STRIDED: scale stride per dim in elements (0 = broadcast) */
} vq_scale_layout;

/* Host-derived exponent tables for power-of-two scales (upstream:
 * floor(log2(amax)) - floor(log2(quant_max)) and 2**e with torch CPU arithmetic in the tensor's
 * dtype, src/voyager_compiler/quantization/mx_utils.py:42-47, ops/quantized.py:471-488,498).
 * Index i stands for the true binary exponent e = i - 149 of amax (e in [-149, 127]).
 *   bump_at[i]  : smallest fp32 bit pattern with true exponent e for which the CPU's rounded
 *                 log2 already floors to e+1 (the pattern of 2^(e+1) when there is none);
 *   scale_of[j] : the final scale, as fp32, for a floored exponent j - 149 (278 entries),
 *                 i.e. where(2**(e - floor(log2 qmax)) > 0, ., 1). */
#define VQ_EXP_ENTRIES 277
typedef struct vq_exp_tables {
    const uint32_t* bump_at;  /* device pointer, 277 entries */
    const float* scale_of;    /* device pointer, 278 entries */
} vq_exp_tables;

VQ_API int vq_version(void);
VQ_API const char* vq_last_error(void);
/* Number of kernels this library has launched from the calling process so far. */
VQ_API uint64_t vq_launch_count(void);

/* Host-only self check of the index-division constants the kernels use (0 = exact). */
VQ_API int vq_selftest_fastdiv(uint32_t d, uint32_t n);

/* out[i] = table(bf16_rne(in[i])), stored in the dtype of `in`.
 * Replaces `vmap`, src/voyager_compiler/ops/quantized.py:98-121. */
VQ_API int vq_lut_map(const void* in, int dtype, int64_t n, const vq_table* table, void* out, void* stream);

/* out[i] = table(bf16_rne(in[i] / scale[.] (+ zero_point[.]))) in the dtype of `in`; scale and
 * zero_point have the dtype of `in`.  `out_codes`, when not NULL, also receives the packed code
 * of every element (code_bits 8: one byte each; 4: two per byte, even element in the low nibble).
 * `out` may be NULL when only packed codes are wanted.
 * Replaces `quantize`, src/voyager_compiler/ops/quantized.py:131-172. */
VQ_API int vq_quantize(const void* in, int dtype, int64_t n, const void* scale, const void* zero_point,
                const vq_scale_layout* layout, const vq_table* table, void* out,
                uint8_t* out_codes, int code_bits, void* stream);

/* out[i] = out_table((in_table(in[i]) - zero_point[.]) * scale[.]), either table optional.
 * Replaces `dequantize`, src/voyager_compiler/ops/quantized.py:182-227. */
VQ_API int vq_dequantize(const void* in, int dtype, int64_t n, const void* scale, const void* zero_point,
                  const vq_scale_layout* layout, const vq_table* in_table, const vq_table* out_table,
                  void* out, void* stream);

/* Per-block scale of a tensor viewed as [outer, L, inner] with blocks of `block` elements along
 * L (a ragged tail block is zero padded; L < block is one block).  Output is
 * [outer, ceil(L/block), inner] in the dtype of `in`.
 *   pow2 == 1: scale = exp->scale_of[floor-log2 index of amax]    (needs exp)
 *   pow2 == 0: scale = amax / quant_max, optionally through scale_table, then where(>0, ., 1)
 *   pow2 == 2: the block maximum of |x| itself (NaN kept); chaining such passes axis by axis
 *              gives the maxima of blocks that span several axes.
 * Replaces `calculate_mx_qparam`, src/voyager_compiler/ops/quantized.py:442-499. */
VQ_API int vq_mx_scale(const void* in, int dtype, int64_t outer, int64_t L, int64_t inner, int64_t block,
                double quant_max, int pow2, const vq_exp_tables* exp, const vq_table* scale_table,
                void* out_scale, void* stream);

/* Optional extra outputs of vq_quantize_mx; any pointer may be NULL. */
typedef struct vq_mx_extras {
    float* scale_f32;    /* the scale widened to fp32, same shape as out_scale */
    int8_t* exp_e8;      /* pow2 only: log2(scale) clamped to [-127, 127] */
    uint8_t* codes;      /* packed codes, code_bits per element */
    int32_t code_bits;   /* 8 or 4 */
    void* dequant;       /* table value * scale in the dtype of `in` (value tables only) */
} vq_mx_extras;

/* One pass over `in`: block scale as vq_mx_scale, then codes as vq_quantize with that scale.
 * out_scale / out_codes may be NULL when only the extras are wanted.
 * Replaces `quantize_mx`, src/voyager_compiler/ops/quantized.py:509-529 (outputs: scale, codes). */
VQ_API int vq_quantize_mx(const void* in, int dtype, int64_t outer, int64_t L, int64_t inner, int64_t block,
                   double quant_max, int pow2, const vq_exp_tables* exp, const vq_table* scale_table,
                   const vq_table* table, void* out_scale, void* out_codes,
                   const vq_mx_extras* extras, void* stream);

/* One tensor of a multi-tensor pass: `n` elements laid out as consecutive blocks (a [rows, K]
 * tensor with blocks along K and K a multiple of the block).  Output pointers as in
 * vq_quantize_mx / vq_mx_extras; any may be NULL, at least one must not be. */
typedef struct vq_mx_item {
    const void* in;
    void* out_scale;
    void* out_codes;
    float* scale_f32;
    int8_t* exp_e8;
    uint8_t* codes;
    void* dequant;
    int64_t n;
} vq_mx_item;

/* Bytes of device workspace vq_quantize_mx_multi needs for n_items tensors. */
VQ_API size_t vq_quantize_mx_multi_workspace(int n_items);

/* vq_quantize_mx over many tensors that share dtype, block size, scale rule and tables, in ONE
 * kernel launch (whole-model weight quantization; upstream runs calculate_mx_qparam + quantize per
 * parameter, src/voyager_compiler/quantization/quantize_pt2e.py:485-500).  `items` is a HOST
 * array; it is copied into `workspace` (device memory, 16-byte aligned, at least
 * vq_quantize_mx_multi_workspace(n_items) bytes) on `stream` before the launch.  The workspace
 * must stay untouched until the work queued on `stream` has finished. */
VQ_API int vq_quantize_mx_multi(const vq_mx_item* items, int n_items, int dtype, int64_t block, double quant_max,
                                int pow2, const vq_exp_tables* exp, const vq_table* scale_table,
                                const vq_table* table, int code_bits, void* workspace, size_t workspace_bytes,
                                void* stream);

/* vq_quantize_mx_multi prepared once and run many times (weights re-quantized every calibration or
 * training step; a sharded whole-model pass that repeats): create checks the arguments, picks the
 * kernel and its launch shape and puts the descriptors into `workspace` (same size rule as above;
 * the stream is synchronised once so the descriptors have landed); run is then a single kernel
 * launch on any stream of the same device, with no host work that grows with the tensor count and
 * no copy.  The tensors are read and written where the items pointed at creation time; the tables,
 * the exponent tables and the workspace must stay alive and untouched for the life of the plan.
 * Same upstream counterpart as vq_quantize_mx_multi. */
typedef struct vq_mx_plan vq_mx_plan;
VQ_API int vq_mx_plan_create(const vq_mx_item* items, int n_items, int dtype, int64_t block, double quant_max,
                             int pow2, const vq_exp_tables* exp, const vq_table* scale_table, const vq_table* table,
                             int code_bits, void* workspace, size_t workspace_bytes, void* stream,
                             vq_mx_plan** plan_out);
VQ_API int vq_mx_plan_run(const vq_mx_plan* plan, void* stream);
VQ_API void vq_mx_plan_destroy(vq_mx_plan* plan);

/* Y[M,N] = A[M,K] @ B[N,K]^T (+ bias[N]); A, B, bias, Y bf16, fp32 accumulation on the tensor
 * cores, operands fetched by TMA.  K must be a multiple of 8.  `status` (device int32, may be
 * NULL, zeroed by the caller) receives a non-zero code if a bounded wait inside the kernel ran out.
 * This is the contraction `aten.linear` performs inside linear_mx / matmul_mx
 * (src/voyager_compiler/ops/quantized.py:330-333, 404-406). */
VQ_API int vq_gemm_bf16_tn(const void* A, const void* B, const void* bias, void* Y, int64_t M, int64_t N, int64_t K,
                           int32_t* status, void* stream);

/* out[b, n, k] = bf16(in[b, k, n] * scale[b, k / block, n]) for bf16 tensors: `in` [batch, K, N], `scale`
 * [batch, scale_rows, N] with scale_rows >= ceil(K / block) (NULL: a plain transposition), `out` [batch, N, K].
 * K, N and block even.  Decodes the right operand of `matmul_mx` (blocks along dim -2) or a "ck" linear
 * weight, src/voyager_compiler/ops/quantized.py:330-333, 389-406, straight into the K-major order the GEMM reads. */
VQ_API int vq_dequantize_transpose(const void* in, const void* scale, int64_t batch, int64_t K, int64_t N, int64_t block,
                                   int64_t scale_rows, void* out, void* stream);

/* `batch` independent products Y[b] = A[b] @ B[b]^T with A [batch, M, K], B [batch, N, K] and Y [batch, M, N],
 * all contiguous bf16; a_shared / b_shared != 0: that operand is a single [M, K] / [N, K] matrix used by every
 * batch.  One persistent launch walks the output tiles of all batches.  This is the contraction
 * `aten.matmul` performs inside matmul_mx on batched (attention) operands,
 * src/voyager_compiler/ops/quantized.py:404-406, once the right operand is in [N, K] order
 * (vq_dequantize_transpose). */
VQ_API int vq_gemm_bf16_tn_batched(const void* A, const void* B, void* Y, int64_t batch, int64_t M, int64_t N, int64_t K,
                                   int a_shared, int b_shared, int32_t* status, void* stream);

/* The fp32 form of the contraction above on the tensor cores: Y[b][M,N] = A[b][M,K] @ B[b][N,K]^T (+ bias, batch 1
 * only), all tensors fp32 row-major; the tensor cores read the operands as tf32 (the low 13 bits of every operand
 * are ignored: exact for decoded MX operands -- codes of up to 11 significant bits times a power-of-two scale --
 * and 2^-11 relative otherwise) and accumulate in fp32.  K a multiple of 4, operands 16-byte aligned; a_shared /
 * b_shared as in vq_gemm_bf16_tn_batched.  Serves `linear_mx` / `matmul_mx` / `conv2d_mx` on fp32 operands,
 * src/voyager_compiler/ops/quantized.py:239-432 (upstream calls the fp32 F.linear / matmul / conv2d there). */
VQ_API int vq_gemm_f32_tn_batched(const void* A, const void* B, const void* bias, void* Y, int64_t batch, int64_t M,
                                  int64_t N, int64_t K, int a_shared, int b_shared, int32_t* status, void* stream);

/* The same GEMM writing its [M,N] result into columns [col_offset, col_offset+N) of EVERY buffer in
 * Ys (n_outputs <= 8 device pointers, rows ldy elements apart): a rank of a column-sharded linear
 * passes its own output and its peers' (peer-mapped memory), so the all-gather of the reference-side
 * composition happens as plain stores over NVLink inside the GEMM epilogue.  The caller orders the
 * launch against the peers (a barrier before reuse of Y, another before reading it). */
VQ_API int vq_gemm_bf16_tn_scatter(const void* A, const void* B, const void* bias, void* const* Ys, int n_outputs,
                                   int64_t ldy, int64_t col_offset, int64_t M, int64_t N, int64_t K,
                                   int32_t* status, void* stream);

/* Statistics pass of the learned-codebook fit (src/voyager_compiler/quantization/lcq.py: unit_scale :136-150,
 * Histogram.add :75-105, _accumulate :601-626).  x holds n elements (VQ_F32 or VQ_BF16, widened to fp32);
 * with block > 0 every run of `block` elements is divided by max(amax, 1e-12) / quant_max first, with block == 0
 * the values are taken as they are.  Value v goes to bin clamp(#{edges <= v} - 1, 0, bins - 1) over the bins + 1
 * ascending fp32 `edges` (device) and adds w, w * v and w * v * v, in fp64, to weight / total / square (device,
 * [bins] each, accumulated in place); w = 1 when n_weights == 0, else weights[i % n_weights] for element i (the
 * energy of its channel, channels last).  Sums are formed in an order the scheduler decides; fp64 keeps that
 * below what can move a fitted level, as upstream notes for its own GPU path. */
VQ_API int vq_lcq_accumulate(const void* x, int dtype, int64_t n, int64_t block, double quant_max, const float* weights,
                             int64_t n_weights, const float* edges, int bins, double* weight, double* total,
                             double* square, void* stream);

/* The 65 536-entry bf16 table a fitted codebook is used through: table[p] = the entry nearest to the value of bf16
 * pattern p clamped to [min(entries), max(entries)], distances in fp32, the first of equal distances, entry 0 for a NaN
 * pattern; `entries` are n fp32 numbers on the device (1 <= n <= 8192), rounded to bf16 in the table.
 * Replaces `codebook_qmap`, src/voyager_compiler/quantization/lcq.py:270-291. */
VQ_API int vq_codebook_qmap(const float* entries, int n, uint16_t* table, void* stream);

/* One microscaling block of the GPTQ column walk, all rows at once
 * (src/voyager_compiler/quantization/gptq.py:238-259 with block_scale, :79-137): for every row r of
 * work[rows, ld] (fp32) the scale s_r = where(t > 0, t, 1) with t = scale_table(amax_r / quant_max) over the
 * columns start..start+bw, floored at 1e-12 (with `shrink`: the factor of {1, .93, .86, .79, .72} times that, taken
 * through scale_table, whose salience-weighted squared error is lowest); then column by column
 * q = table(bf16(w / s_r)) * s_r -> out[r, col], delta = (w - q) / max(hinv[col, col], 1e-12) -> deltas[r, col - start]
 * (deltas is [rows, bw]), and w[later columns of the block] -= delta * hinv[col, later].  work is only read: the
 * caller applies work[:, start+bw:] -= deltas @ hinv[start:start+bw, start+bw:].  hinv is the upper Cholesky factor of
 * the inverse Hessian, [K, ldh] fp32; salience [K] = diag(H), needed with `shrink`; scale_out [rows] may be NULL;
 * bw <= 64.  Every step is the fp32 operation upstream's tensor expression performs, in its order. */
VQ_API int vq_gptq_block(const float* work, int64_t ld, int64_t rows, int64_t start, int bw, const float* hinv, int64_t ldh,
                         const float* salience, int shrink, double quant_max, const vq_table* table,
                         const vq_table* scale_table, float* out, int64_t ldo, float* deltas, float* scale_out,
                         void* stream);

/* Patch matrix of a 2-D convolution (groups = 1), so that conv2d_mx becomes the contraction above:
 * out[(n, ho, wo), (i, j, c)] = x[n, ho*stride_h - pad_h + i*dil_h, wo*stride_w - pad_w + j*dil_w, c], zero
 * outside the image; out is [N*Ho*Wo, ldk] in x's dtype (VQ_F32 or VQ_BF16), ldk >= kh*kw*C, the columns from
 * kh*kw*C on are zero-filled; Ho = (H + 2 pad_h - dil_h (kh-1) - 1) / stride_h + 1, Wo alike.  x is addressed
 * by the element strides sn, sh, sw, sc (NCHW: sc = H*W, sw = 1; NHWC: sc = 1).  With `scale` (same dtype, may
 * be NULL) every element is multiplied by scale[n*ssn + h*ssh + w*ssw + (c / block)*ssc] and rounded once in
 * that dtype: `dequantize` of an MX activation with blocks along the channels
 * (src/voyager_compiler/ops/quantized.py:182-227, 267-271) fused into the copy.  The weight goes against the
 * result as [O, ldk] with the same (i, j, c) column order.  Serves `conv2d_mx`,
 * src/voyager_compiler/ops/quantized.py:239-283 (upstream calls aten.conv2d on the decoded operands). */
VQ_API int vq_conv_patches(const void* x, int dtype, int64_t N, int64_t H, int64_t W, int64_t C, int64_t sn, int64_t sh,
                           int64_t sw, int64_t sc, int kh, int kw, int stride_h, int stride_w, int pad_h, int pad_w,
                           int dil_h, int dil_w, const void* scale, int64_t block, int64_t ssn, int64_t ssh, int64_t ssw,
                           int64_t ssc, void* out, int64_t ldk, void* stream);

/* 2-D convolution as an implicit GEMM on the tensor cores (no patch matrix is written):
 *   y[(n, ho, wo), o] = bias[o] + sum over (i, j, c) of
 *       x[n, ho*stride_h - pad_h + i*dil_h, wo*stride_w - pad_w + j*dil_w, g*Cg + c] * wmat[o, (i*kw + j)*Cp + c]
 * for the outputs o of group g (Cg = C / groups input channels, O / groups outputs per group), zero outside the
 * image; fp32 accumulation, one rounding to bf16.  x: bf16, channels contiguous, pixels addressed by the element
 * strides sn, sh, sw; with `x_scale` (bf16, may be NULL) every element is first multiplied by
 * x_scale[n*ssn + h*ssh + w*ssw + channel / block] and rounded to bf16 once (`dequantize` of an MX activation with
 * blocks along the channels, src/voyager_compiler/ops/quantized.py:182-227, fused into the operand staging).  wmat:
 * the decoded bf16 weight as [O, vq_conv2d_weight_columns(Cg, kh, kw)], every tap's channels zero-padded to
 * Cp = 64 * ceil(Cg / 64).  y: [N*Ho*Wo, O] bf16 (NHWC), Ho = (H + 2 pad_h - dil_h (kh-1) - 1) / stride_h + 1, Wo
 * alike; bias bf16 [O] or NULL.  Needs Cg, sn, sh, sw multiples of 8, 16-byte aligned x, wmat, y and a block that
 * is a power of two >= 8 (VQ_ERR_UNSUPPORTED otherwise: use vq_conv_patches + vq_gemm_bf16_tn).  `status` as in
 * vq_gemm_bf16_tn (codes 11..14 name the warp role whose bounded wait ran out).  Serves `conv2d_mx`,
 * src/voyager_compiler/ops/quantized.py:239-283 (upstream calls aten.conv2d on the decoded operands), groups included. */
VQ_API int64_t vq_conv2d_weight_columns(int64_t channels_per_group, int kh, int kw);
VQ_API int vq_conv2d_bf16(const void* x, int64_t N, int64_t H, int64_t W, int64_t C, int64_t sn, int64_t sh, int64_t sw,
                          const void* x_scale, int64_t block, int64_t ssn, int64_t ssh, int64_t ssw, const void* wmat,
                          int64_t O, int kh, int kw, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h,
                          int dil_w, int groups, const void* bias, void* y, int32_t* status, void* stream);

/* Y[M,N] = (a_codes * expand(a_scale))[M,K] @ (b_codes * expand(b_scale))[N,K]^T (+ bias), all
 * tensors bf16, scales [rows, K/block] with blocks along K; each product code*scale is rounded to
 * bf16 once, as the bf16 tensor arithmetic of the reference does, inside the operand staging of
 * the GEMM (no dequantised copy is written).  block must be 32 and K a multiple of 64, otherwise
 * VQ_ERR_UNSUPPORTED.  Replaces `linear_mx`, src/voyager_compiler/ops/quantized.py:295-348
 * (weight_layout "kc", no codebooks, no sparse side path). */
VQ_API int vq_linear_mx(const void* a_codes, const void* a_scale, const void* b_codes, const void* b_scale,
                        const void* bias, void* Y, int64_t M, int64_t N, int64_t K, int64_t block, int32_t* status,
                        void* stream);

/* vq_quantize_mx_multi without a caller workspace and without any allocation.  This entry point has
 * no counterpart in the reference; it exists for callers that must not allocate device memory where
 * they quantize (a plug-in running inside another framework's closed memory pool, a serving loop
 * that sized all buffers at start-up, a thread that may not take the allocator lock).  The tensor
 * descriptors are staged in a fixed array inside the library, so:
 *   - at most vq_quantize_mx_multi_static_max_items() tensors (1024) per call; more is rejected
 *     with VQ_ERR_INVALID;
 *   - the first call on each device looks up the array's device address (with that device current);
 *     make that first call outside any stream capture;
 *   - all calls on a device share the array: calls whose GPU work can overlap (different streams,
 *     or threads racing on one stream) overwrite each other's descriptors.  Serialise them.  Nothing
 *     in the array has to be cleared between calls; each call rewrites what it uses.
 * No cudaMalloc / cudaFree or other allocating routine is called; inputs and outputs are the caller's. */
VQ_API int vq_quantize_mx_multi_static_max_items(void);
VQ_API int vq_quantize_mx_multi_static(const vq_mx_item* items, int n_items, int dtype, int64_t block,
                                       double quant_max, int pow2, const vq_exp_tables* exp,
                                       const vq_table* scale_table, const vq_table* table, int code_bits,
                                       void* stream);

/* out[i] = qmap[bf16(in[i] / scale)] * scale in `dtype`: quantize and dequantize in one pass, the
 * forward of upstream `FakeQuantizeFunction`, src/voyager_compiler/quantization/fake_quantize.py:101-115
 * (`vmap(input / scale, qmap) * scale`).  Scale placement as in vq_quantize. */
VQ_API int vq_fake_quantize(const void* in, int dtype, int64_t n, const void* scale, const vq_scale_layout* layout,
                            const vq_table* table, void* out, void* stream);

/* out[c] = max |in[o, c, i]| over o and i, for a tensor viewed as [outer, C, inner]; fp32 output
 * (the exact widening for bf16 data; NaN if a NaN is present).  One pass, no temporary: the
 * observer's `torch.amax(torch.abs(x))` / per-channel amax,
 * src/voyager_compiler/quantization/fake_quantize.py:320-325.  Per tensor: outer = C = 1. */
VQ_API int vq_amax(const void* in, int dtype, int64_t outer, int64_t C, int64_t inner, float* out, void* stream);

/* The observer's state update as one launch (`_update_amax_scale`,
 * src/voyager_compiler/quantization/fake_quantize.py:327-341): amax = max over history[history_len, channels]
 * before amax_cur enters it; the history is rolled by -1 along its first axis and slot 0 set to
 * amax_cur; scale = amax / quant_max, unchanged where amax is 0, NaN or Inf; pow2 != 0 rounds the
 * scale up to a power of two, 2 ** ceil(log2(scale)).  `pow2_stay` (device, 256 bytes, may be NULL): for every
 * biased fp32 exponent, how many of the values 2^e (1 + m 2^-23), m = 0, 1, ..., the reference arithmetic (the CPU's
 * fp32 log2, rounded) still maps to e; with it the result equals upstream's bit for bit, without it the device's
 * log2f decides those few values.  All fp32, in place. */
VQ_API int vq_observer_update(const float* amax_cur, float* history, float* scale, int history_len, int64_t channels,
                              double quant_max, int pow2, const uint8_t* pow2_stay, void* stream);

/* vq_amax and vq_observer_update as ONE launch: the reduction's CTA that finishes last runs the state update.
 * `amax_scratch`: channels + 1 fp32 words of device memory owned by the observer, ALL ZERO on entry (allocate it zeroed
 * once) and all zero again when the launch completes: the per-channel maxima of this step and a ticket.  No memset and
 * no second launch per step; two steps on the same scratch must not overlap.  Arguments otherwise as the two calls.
 * Replaces `FusedAmaxObsFakeQuantize._update_amax_scale`, src/voyager_compiler/quantization/fake_quantize.py:309-341. */
VQ_API int vq_observer_step(const void* in, int dtype, int64_t outer, int64_t channels, int64_t inner, float* amax_scratch,
                            float* history, float* scale, int history_len, double quant_max, int pow2, const uint8_t* pow2_stay,
                            void* stream);

/* Group-wise affine fake-quantize of a tensor viewed as [rows, K] with blocks of `block` elements along K (the last
 * block of a row may be short; its zero padding takes part in the extrema as upstream pads it):
 *   sf = (max - min) / (quant_max - quant_min), 1 where that is not positive;  zp = -min / sf + quant_min;
 *   both optionally mapped through `scale_table` (65 536 bf16 patterns on the device, or NULL);
 *   out = (clamp(round_half_even(in / sf + zp), quant_min, quant_max) - zp) * sf,
 * every step rounded to `dtype`.  out_scale / out_zero_point: [rows, ceil(K / block)] in `dtype`.
 * Replaces `GroupWiseAffineFakeQuantFunction.forward`,
 * src/voyager_compiler/quantization/fake_quantize.py:160-207. */
VQ_API int vq_group_affine_fake_quantize(const void* in, int dtype, int64_t rows, int64_t K, int64_t block, double quant_min,
                                         double quant_max, const uint16_t* scale_table, void* out_scale, void* out_zero_point,
                                         void* out, void* stream);

/* histogram[b] += number of elements of `in` with floor(log2(|x| as fp32)) == b - 126, b = 0..253, as one fp32
 * addition per bin: the observer's exponent histogram, `histogram += torch.histc(floor(log2(|x|)), 254, min=-126,
 * max=127)`, src/voyager_compiler/quantization/fake_quantize.py:369-371.  Zeros, subnormals, infinities and NaNs are
 * not counted.  `exp` holds the fp32 thresholds (bump_at) of the shared-exponent rule; `workspace` is at least 2032 bytes
 * of device scratch, 8-byte aligned; with 2040 bytes or more, large tensors finish in the counting launch itself (its last
 * CTA adds the counts to `histogram`) instead of a launch of their own. */
VQ_API int vq_exp_histogram(const void* in, int dtype, int64_t n, const vq_exp_tables* exp, float* histogram, void* workspace,
                            size_t workspace_bytes, void* stream);

/* inliers[i] = |in[i]| >= t ? 0 : in[i], with t = *threshold (device, fp32) rounded to the dtype of `in`;
 * *n_outliers (device) receives the number of elements set to zero.  The observer's outlier removal before
 * quantization, `x.masked_fill(x.abs() >= outlier_threshold, 0.0)`,
 * src/voyager_compiler/quantization/fake_quantize.py:388-394. */
VQ_API int vq_outlier_split(const void* in, int dtype, int64_t n, const float* threshold, void* inliers,
                            unsigned long long* n_outliers, void* stream);

/* out[i] = |in[i]| >= t ? in[i] : quantized[i]: the outliers come back after the quantizer ran on the inliers
 * (`torch.where(skip, orig_x, x)`, src/voyager_compiler/quantization/fake_quantize.py:428-430). */
VQ_API int vq_outlier_merge(const void* in, const void* quantized, int dtype, int64_t n, const float* threshold, void* out,
                            void* stream);

/* vq_linear_mx on PACKED operands: a_codes [M,K] and b_codes [N,K] hold one int8 code per byte (as
 * vq_quantize_mx / vq_quantize_mx_multi write them with code_bits 8 for an integer table), a_scale /
 * b_scale are bf16 [rows, K/32].  Codes and scales arrive by TMA; the conversion int8 -> bf16(code *
 * scale) happens inside the operand staging of the CTA-pair kernel, so the operands cost one byte per
 * element of HBM and L2 traffic.  Same product as vq_linear_mx / `linear_mx`
 * (src/voyager_compiler/ops/quantized.py:295-348) on the float codes.  Needs block 32, K a multiple of
 * 256 and M > 128 (VQ_ERR_UNSUPPORTED otherwise). */
VQ_API int vq_linear_mx_packed(const int8_t* a_codes, const void* a_scale, const int8_t* b_codes, const void* b_scale,
                               const void* bias, void* Y, int64_t M, int64_t N, int64_t K, int64_t block,
                               int32_t* status, void* stream);

/* `filter_outlier`, src/voyager_compiler/ops/quantized.py:565-621 (with `_pad_csr`, :538-562), over
 * [batch, rows, cols] matrices: inlier[i] = in[i] where |in[i]| <= threshold (threshold rounded to the
 * tensor dtype), +0 elsewhere; per matrix the non-zero outliers as a CSR in row / column order: values
 * (tensor dtype) and int32 column indices in [batch, max_nnz] padded with 0 / -1, int32 row pointers
 * [batch, rows + 1] starting at indptr_offset.  More than max_nnz outliers: the surplus is dropped and
 * the row pointers are clamped, as upstream does.  `workspace`: vq_filter_outlier_workspace(batch, rows)
 * bytes of device scratch. */
VQ_API size_t vq_filter_outlier_workspace(int64_t batch, int64_t rows);
VQ_API int vq_filter_outlier(const void* in, int dtype, int64_t batch, int64_t rows, int64_t cols, double threshold,
                             int64_t max_nnz, int32_t indptr_offset, void* data, int32_t* indices, int32_t* indptr,
                             void* inlier, void* workspace, size_t workspace_bytes, void* stream);

/* Y[b, r, :] = sum over the CSR entries (r, k, v) of matrix b of v * Bt[b, k, :], fp32 accumulation,
 * one rounding to `dtype`: the sparse correction of `spmm_csr`, src/voyager_compiler/ops/quantized.py:786-862,
 * with the right operand already decoded and in [K, N] order.  Row pointers may start above 0 (a
 * slice of a longer CSR); data / indices then hold only the span they cover.  bt_batch_stride: elements
 * between the Bt of consecutive batches, 0 when it is shared.  addend (optional, [batch, rows, N], may
 * alias Y): Y = addend + product, the product rounded to `dtype` first, as `dense_out + spmm_out` does. */
VQ_API int vq_spmm_csr(const void* data, const int32_t* indices, const int32_t* indptr, const void* Bt, int dtype,
                       int64_t batch, int64_t rows, int64_t K, int64_t N, int64_t max_nnz, int64_t bt_batch_stride,
                       const void* addend, void* Y, void* stream);

/* `slice_csr_tensor`, src/voyager_compiler/ops/quantized.py:745-788, without its three host read-backs: rows
 * (dim 0) or columns (dim 1) [start, end) of a padded CSR (`data` / `indices` of max_nnz entries, int32 `indptr`
 * of rows + 1 entries).  Outputs: `cap` entries (upstream: int(max_nnz * size_factor)) padded with 0 / -1, and the
 * row pointers of the slice (dim 0: end - start + 1 entries rebased to 0; dim 1: rows + 1 entries, column indices
 * rebased to `start`); when more entries survive than fit, the surplus is dropped and the row pointers are clamped
 * to `cap`, as upstream's _pad_csr does.  dim 1 needs vq_slice_csr_workspace(rows) bytes of device scratch. */
VQ_API size_t vq_slice_csr_workspace(int64_t rows);
VQ_API int vq_slice_csr(const void* data, const int32_t* indices, const int32_t* indptr, int dtype, int64_t rows,
                        int64_t max_nnz, int dim, int64_t start, int64_t end, int64_t cap, void* out_data,
                        int32_t* out_indices, int32_t* out_indptr, void* workspace, size_t workspace_bytes, void* stream);

/* One tensor of a per-channel pass, viewed as [channels, length] (a conv weight OIHW is
 * [O, I*H*W]).  Every output may be NULL, at least one must not be.  All tensors in `dtype`. */
typedef struct vq_channel_item {
    const void* input;
    int64_t channels, length;
    const void* scale_in; /* [channels], optional: quantize with this scale instead of amax / quant_max */
    void* amax_out;       /* [channels]: max |x| of the channel (NaN if the channel holds one) */
    void* scale_out;      /* [channels]: amax / quant_max, 1 where amax is 0, NaN or Inf (not written with scale_in) */
    void* values;         /* [channels, length]: qmap[bf16(x / scale)] */
    uint8_t* codes;       /* [channels, length]: packed 8-bit code of that value */
    void* dequant;        /* [channels, length]: values * scale */
} vq_channel_item;

/* Bytes of device workspace for these items (depends on the channel counts and lengths). */
VQ_API size_t vq_channel_quantize_multi_workspace(const vq_channel_item* items, int n_items);

/* Per-channel amax + scale + quantize (+ dequantize) over many tensors in ONE launch: what upstream
 * computes per weight tensor with the observer's scale rule
 * (src/voyager_compiler/quantization/fake_quantize.py:320-333: amax over all axes but the channel
 * axis, / quant_max), `quantize` (src/voyager_compiler/ops/quantized.py:131-172) and `dequantize`
 * (:182-227), each as separate passes.  `items` is a HOST array, copied into `workspace` (device, 16-byte
 * aligned, vq_channel_quantize_multi_workspace(items, n_items) bytes) on `stream`.  Channel lengths
 * below 2^22 elements. */
VQ_API int vq_channel_quantize_multi(const vq_channel_item* items, int n_items, int dtype, double quant_max,
                                     const vq_table* table, void* workspace, size_t workspace_bytes, void* stream);

/* vq_channel_quantize_multi prepared once and run many times (weights re-quantized every calibration or
 * training step): create checks the arguments, cuts the tensors into batches, picks the kernel and puts
 * the descriptors into `workspace` (the stream is synchronised once); run is then a single kernel launch
 * on any stream of the same device, with no host work and no copy.  Tensors are read and written where the
 * items pointed at creation time; the table and the workspace must stay alive and untouched for the life of
 * the plan.  Same upstream counterpart as vq_channel_quantize_multi. */
typedef struct vq_channel_plan vq_channel_plan;
VQ_API int vq_channel_plan_create(const vq_channel_item* items, int n_items, int dtype, double quant_max,
                                  const vq_table* table, void* workspace, size_t workspace_bytes, void* stream,
                                  vq_channel_plan** plan_out);
VQ_API int vq_channel_plan_run(const vq_channel_plan* plan, void* stream);
VQ_API void vq_channel_plan_destroy(vq_channel_plan* plan);

/* Non-zero when a bounded wait inside a bulk-copy per-channel kernel ran out on the current device since the
 * last call; the outputs of that launch are then incomplete.  Streaming-role kernel: 31 the producer waited for
 * a free stage, 32 a reduction team for its batch, 33 a quantization team for the reductions, the batch or the
 * tables.  Group pipeline (channels of 4609..6144 elements): 21 the producer, 22 a consumer group waiting for its
 * batch, 23 for the tables.  Synchronises the device; clears the word. */
VQ_API int vq_channel_status(void);

/* out[i] = levels[code[i]] * scale[i / block] in `dtype` (one rounding), from the packed views that
 * vq_quantize_mx / vq_quantize_mx_multi write: 8-bit codes (one per byte) or 4-bit codes (two per
 * byte, even element in the low nibble), and per block either an fp32 scale or an E8 exponent
 * (scale = 2^e).  `levels`: device array of n_levels fp32 values.  block must be a multiple of 16.
 * The decode + scale half of `linear_mx`'s operand preparation, src/voyager_compiler/ops/quantized.py:313-326,
 * and `dequantize`, :182-227, on packed storage. */
VQ_API int vq_dequantize_packed(const uint8_t* codes, int code_bits, const float* levels, int n_levels,
                                const float* scale_f32, const int8_t* exp_e8, int64_t n, int64_t block, void* out,
                                int dtype, void* stream);

/* Per-row codebook quantization: x is [rows, K] (dtype f32 or bf16, row-major), levels is
 * [rows, n_levels] fp32, each row sorted ascending, n_levels <= 256.  For every element the index of
 * the nearest level of its row goes to idx_out (uint8 [rows, K], may be NULL) and that level to
 * deq_out (same dtype as x, may be NULL).  The rule is upstream `codebook_qmap`,
 * src/voyager_compiler/quantization/lcq.py:270-291, applied per row: clamp to the codebook range,
 * |x - level| in fp32, the first minimum wins, NaN -> index 0.  round_bf16 != 0 rounds the element to
 * bf16 before the search and the returned level to bf16, which is what that table followed by `vmap`
 * (src/voyager_compiler/ops/quantized.py:98-121) gives; round_bf16 == 0 searches the fp32 element and
 * returns the fp32 level.  Upstream codebooks are per tensor; a per-row codebook has no upstream op.
 * `workspace`: device scratch of vq_row_codebook_workspace(rows, n_levels) bytes, 4-byte aligned (the
 * per-row decision thresholds are written there by a first small kernel on the same stream). */
VQ_API size_t vq_row_codebook_workspace(int64_t rows, int n_levels);

/* The fit of those codebooks: out[row, k] (fp32 [rows, n_levels]) = quantile of row `row` of x [rows, K] at
 * (2k + 1) / (2 n_levels), linear interpolation, evaluated in fp32 exactly as torch.quantile does on the
 * CPU; a row holding a NaN gives NaN.  K from 1 to 8192 (VQ_ERR_UNSUPPORTED otherwise).  No upstream
 * counterpart (upstream codebooks are fitted per tensor by quantization/lcq.py). */
VQ_API int vq_row_quantile(const void* x, int dtype, int64_t rows, int64_t K, int n_levels, float* out, void* stream);
VQ_API int vq_row_codebook(const void* x, int dtype, int64_t rows, int64_t K, const float* levels, int n_levels,
                           int round_bf16, uint8_t* idx_out, void* deq_out, void* workspace, size_t workspace_bytes,
                           void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VOYAGER_B200_H */
