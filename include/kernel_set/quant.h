/*
 * Activation quantizer and int4 weight format helpers.
 *
 * Replaces three entries of include/kernel_set/quant.h of the reference
 * project: ks_quantize_fp8_group (:28-40), ks_dequantize_int4 (:53-58) and
 * ks_repack_int4 (:60-66), and adds the import of GPTQ / AWQ checkpoints. The
 * per-tensor fp8, int8 and nvfp4 quantizers of that header are other formats.
 */
#ifndef KERNEL_SET_QUANT_H_
#define KERNEL_SET_QUANT_H_

#include "kernel_set/types.h"

KS_BEGIN_EXTERN_C

/*
 * For every row r and every run g of `group_size` consecutive columns (the
 * last run of a row may be shorter):
 *     amax        = max |input[r,c]| over the run, in fp32
 *     scale[r,g]  = max(amax / qmax, 1e-12)      qmax = 448 (e4m3), 57344 (e5m2)
 *     out[r,c]    = fp8(input[r,c] / scale[r,g]) round-to-nearest-even, saturating
 *
 *   input  [rows, cols]                     f32 / f16 / bf16 (`in_dtype`)
 *   out    [rows, cols]                     `fp8_dtype`
 *   scale  [rows, ceil(cols/group_size)]    fp32, row-major
 *
 * Both divisions are IEEE divisions, which is what the reference's torch
 * statement of the op computes (benchmarks/bench.py:1444-1457, 2339-2344).
 * Contract otherwise as the reference: quant.h:28-40, quant_fp8_group.cu:133-214.
 */
KS_API ks_status_t ks_quantize_fp8_group(void* out, float* scale,
                                         const void* input, int64_t rows,
                                         int64_t cols, int group_size,
                                         ks_dtype_t in_dtype,
                                         ks_dtype_t fp8_dtype,
                                         ks_stream_t stream);

/*
 * out[k,n] = (q[k,n] - zeros[k/gs, n]) * scales[k/gs, n], computed in fp32 and
 * rounded once to `out_dtype` (f32 / f16 / bf16).
 *
 *   qweight_packed  [K/8, N] int32; code of k = 8*row + j sits in bits 4j..4j+3
 *   scales, zeros   [K/gs, N] `out_dtype`; both required
 *   K multiple of 8 and of group_size.
 * Contract as the reference: quant.h:53-58, dequant_int4.cu:78-112.
 */
KS_API ks_status_t ks_dequantize_int4(void* out, const void* qweight_packed,
                                      const void* scales, const void* zeros,
                                      int64_t k, int64_t n, int group_size,
                                      ks_dtype_t out_dtype, ks_stream_t stream);

/*
 * Re-lays the int32 [K/8, N] packing above into the uint8 [K/2, N] packing
 * that ks_gemm_w4a16 reads (even k in the low nibble). `num_bits` must be 4.
 * `perm`: NULL, or int32 [size_k] on the device, a permutation of 0..size_k-1:
 * row k' of the result is then row perm[k'] of the source (activation order;
 * the reference returns KS_ERROR_NOT_IMPLEMENTED for it). An entry outside
 * 0..size_k-1 yields code 0. With perm, size_k and size_n must be multiples
 * of 8. Contract otherwise as the reference: quant.h:60-66, repack_int4.cu:43-70.
 */
KS_API ks_status_t ks_repack_int4(void* out_packed, const void* qweight,
                                  const void* perm, int64_t size_k,
                                  int64_t size_n, int num_bits,
                                  ks_stream_t stream);

/*
 * ks_quantize_fp8_group(group_size = 128) with the scales stored column-major:
 *   scale_t[g * scale_ld + r] = scale of row r, group g   (scale_ld >= rows)
 * so that the rows of a GEMM tile find their scales of one K-block contiguous
 * (one 512-byte run per 128 rows, TMA-loadable when scale_ld is a multiple of
 * 4); ks_gemm_fp8_blockwise_colscale consumes this layout. Codes and scale
 * values are those of ks_quantize_fp8_group. cols must be a multiple of 128.
 * No counterpart in the reference's C ABI (its external providers offer the
 * layout as an option of their own quantizer).
 */
KS_API ks_status_t ks_quantize_fp8_group_colscale(void* out, float* scale_t,
                                                  int64_t scale_ld,
                                                  const void* input,
                                                  int64_t rows, int64_t cols,
                                                  ks_dtype_t in_dtype,
                                                  ks_dtype_t fp8_dtype,
                                                  ks_stream_t stream);

/*
 * Import of int4 checkpoints. No counterpart in the reference's C ABI: its
 * documentation names the missing re-layout as a gap (docs/QUANT_OPERATORS.md:
 * 71-75, 165) and its dispatcher hands the op to external providers
 * (bindings/python/kernel_set/backends/_quant_ext.py:217-241).
 *
 *   GPTQ  qweight [K/8, N] int32, code of k = 8*row + j in bits 4j..4j+3
 *         qzeros  [G, N/8] int32, column 8c+j in bits 4j..4j+3; files of the
 *                 first format version store zero-1 (zero_offset = 1)
 *         g_idx   [K] group of each row when quantised in activation order;
 *                 perm = stable argsort(g_idx) makes the groups contiguous
 *   AWQ   qweight [K, N/8] int32, qzeros [G, N/8] int32; column 8c+j in nibble
 *         {0,4,1,5,2,6,3,7}[j] of word c; zero_offset = 0
 */
typedef enum ks_int4_source_t {
  KS_INT4_SOURCE_GPTQ = 0,
  KS_INT4_SOURCE_AWQ = 1
} ks_int4_source_t;

typedef enum ks_int4_packing_t {
  KS_INT4_PACKING_BYTES = 0, /* uint8 [K/2, N], what ks_gemm_w4a16 reads     */
  KS_INT4_PACKING_WORDS = 1  /* int32 [K/8, N], what ks_dequantize_int4 reads */
} ks_int4_packing_t;

/*
 * Writes the codes of a checkpoint's qweight in one of the two packings of
 * this library. `perm` as in ks_repack_int4 (NULL: rows keep their order).
 * size_k and size_n multiples of 8; both pointers 16-byte aligned.
 */
KS_API ks_status_t ks_int4_import_weight(void* out, const void* qweight,
                                         const int32_t* perm, int64_t size_k,
                                         int64_t size_n,
                                         ks_int4_source_t source,
                                         ks_int4_packing_t packing,
                                         ks_stream_t stream);

/*
 * zeros[g, n] = code(qzeros, g, n) + zero_offset, as `out_dtype` (f32 / f16 /
 * bf16): the [G, N] zero-points that ks_gemm_w4a16 and ks_dequantize_int4
 * read. zero_offset 0 or 1; size_n a multiple of 8.
 */
KS_API ks_status_t ks_int4_import_zeros(void* zeros, const void* qzeros,
                                        int64_t groups, int64_t size_n,
                                        ks_int4_source_t source,
                                        int zero_offset, ks_dtype_t out_dtype,
                                        ks_stream_t stream);

/*
 * out[r, j] = input[r, perm[j]]: the activations of a layer whose weight rows
 * were reordered with the same perm. perm int32 [cols]; an entry outside
 * 0..cols-1 yields 0. out must not alias input.
 */
KS_API ks_status_t ks_gather_columns(void* out, const void* input,
                                     const int32_t* perm, int64_t rows,
                                     int64_t cols, ks_dtype_t dtype,
                                     ks_stream_t stream);

KS_END_EXTERN_C

#endif /* KERNEL_SET_QUANT_H_ */
