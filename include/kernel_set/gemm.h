/*
 * Quantized GEMM entry points: FP8 with fine-grained fp32 scales, and int4
 * weight-only with 16-bit activations.
 *
 * Replaces the quantized entries of include/kernel_set/gemm.h of the
 * reference project (ks_gemm_w8a8 at :39-49, ks_gemm_w4a16 at :51-59,
 * ks_gemm_fp8 at :60-77, ks_gemm_fp8_blockwise at :79-98). The dense, batched
 * and nvfp4 GEMMs of that header are a different code path and are exported
 * only as NOT_IMPLEMENTED stubs.
 *
 * All matrices are row-major and dense (row stride = number of columns). All
 * pointers are device pointers. Calls enqueue work on `stream` and return
 * without synchronising.
 */
#ifndef KERNEL_SET_GEMM_H_
#define KERNEL_SET_GEMM_H_

#include "kernel_set/types.h"

KS_BEGIN_EXTERN_C

/*
 * C[M,N] = A[M,K] . W[K,N] + bias,  W[k,n] = (q[k,n] - zero[g,n]) * scale[g,n],
 * g = k / group_size.
 *
 *   a         [M,K]      f16 or bf16 (`dtype`)
 *   b_packed  [K/2,N]    uint8; low nibble holds the code of the even k, high
 *                        nibble the code of the odd k; codes are 0..15
 *   scales    [K/gs,N]   `dtype`
 *   zeros     [K/gs,N]   `dtype`, in code units (8.0 for a symmetric grid);
 *                        NULL means zero-point 0
 *   bias      [N]        `dtype` or NULL
 *   group_size <= 0 means one group spanning all of K.
 *
 * K must be even and group_size must divide K (UNSUPPORTED_SHAPE otherwise);
 * dtype other than f16/bf16 is UNSUPPORTED_DTYPE.
 * Same contract as the reference: gemm.h:51-59, gemm_w4a16.cu:6-19,151-182.
 */
KS_API ks_status_t ks_gemm_w4a16(void* c, const void* a, const void* b_packed,
                                 const void* scales, const void* zeros,
                                 const void* bias, int64_t m, int64_t n,
                                 int64_t k, int group_size, ks_dtype_t dtype,
                                 ks_stream_t stream);

/*
 * ks_gemm_w4a16 for callers that are not allowed to allocate. It has no
 * counterpart in the reference project.
 *
 * The fast kernel behind ks_gemm_w4a16 splits K between thread blocks and
 * needs a few MiB of device scratch for the partial sums; ks_gemm_w4a16
 * obtains it from the stream-ordered CUDA allocator the first time a stream
 * is used. Some hosts cannot tolerate that: an inference server that hands
 * the whole GPU to its own pool at start-up (a later cudaMalloc inside a
 * plugin then fails or stalls), a latency-critical decode loop that bans
 * allocator calls once it is running, a sandbox that only lets a plugin
 * launch kernels and copy memory. This entry point performs the same
 * computation with the scratch in a fixed 16 MiB array that is part of the
 * library image (KS_W4A16_STATIC_SCRATCH_BYTES; every GPU that loads the
 * library carries it until the process exits) and calls neither cudaMalloc /
 * cudaFree nor any other allocating routine.
 *
 * Arguments, results and status codes are those of ks_gemm_w4a16, plus:
 *  - a shape whose scratch need exceeds the array (roughly: more than 128
 *    weight-column tiles x 32 token rows x 8 K-splits) is refused with
 *    KS_ERROR_UNSUPPORTED_SHAPE and a message naming both sizes;
 *  - the first call on each device resolves the array's device address; make
 *    that call before starting any stream capture;
 *  - all calls on a device share the one array, so two calls whose kernels
 *    may overlap on the GPU (different streams, no ordering between them)
 *    race on it. Calls on one stream, or ordered by events, are safe.
 */
#define KS_W4A16_STATIC_SCRATCH_BYTES (16u << 20)
KS_API ks_status_t ks_gemm_w4a16_static_scratch(void* c, const void* a,
                                                const void* b_packed,
                                                const void* scales,
                                                const void* zeros,
                                                const void* bias, int64_t m,
                                                int64_t n, int64_t k,
                                                int group_size,
                                                ks_dtype_t dtype,
                                                ks_stream_t stream);

/*
 * 8-bit GEMMs with one scale per row of A and one per column of B:
 *   C = (a_scale (x) b_scale) * (A @ B) [+ bias]
 *   a        [M,K]  fp8 (e4m3 / e5m2, `fp8_dtype`) resp. int8
 *   b        [K,N]  same type, row-major (the transposed, quantized weight)
 *   a_scale  [M] with KS_QUANT_PER_TOKEN, [1] with KS_QUANT_PER_TENSOR   (fp32)
 *   b_scale  [N] with KS_QUANT_PER_CHANNEL, [1] with KS_QUANT_PER_TENSOR (fp32)
 *   bias     [N] in `out_dtype` or NULL (ks_gemm_w8a8 only)
 *   out / c  [M,N]  f32 / f16 / bf16
 * The products are accumulated in fp32 (fp8) resp. exactly in int32 (int8); the
 * result is (acc * a_scale) * b_scale [+ bias], rounded once. Other modes are
 * INVALID_ARGUMENT. K and N multiples of 16 with 16-byte aligned operands take
 * the tcgen05 kernel (kind::f8f6f4 / kind::i8, the whole K range accumulated
 * in tensor memory); everything else a slower general kernel.
 * Same contracts as the reference: gemm.h:60-77 with gemm_fp8.cu:147-153, and
 * gemm.h:39-49 with gemm_w8a8.cu:134-141, 160-190.
 */
KS_API ks_status_t ks_gemm_fp8(void* out, const void* a_fp8, const void* b_fp8,
                               const float* a_scale, const float* b_scale,
                               int64_t m, int64_t n, int64_t k,
                               ks_quant_mode_t a_mode, ks_quant_mode_t b_mode,
                               ks_dtype_t fp8_dtype, ks_dtype_t out_dtype,
                               ks_stream_t stream);

KS_API ks_status_t ks_gemm_w8a8(void* c, const void* a_i8, const void* b_i8,
                                const float* a_scale, const float* b_scale,
                                const void* bias, int64_t m, int64_t n,
                                int64_t k, ks_quant_mode_t a_mode,
                                ks_quant_mode_t b_mode, ks_dtype_t out_dtype,
                                ks_stream_t stream);

/*
 * out[m,n] = sum over K-blocks kb of
 *            a_scale[m,kb] * b_scale[kb, n/block_n] * sum_{k in kb} A8[m,k]*B8[k,n]
 * with the inner sum and the outer sum both kept in fp32.
 *
 *   a_fp8    [M,K]                         e4m3 or e5m2 (`fp8_dtype`)
 *   b_fp8    [K,N]                         same fp8 type
 *   a_scale  [M, ceil(K/block_k)]          fp32, one per 1 x block_k strip
 *   b_scale  [ceil(K/block_k), ceil(N/block_n)]  fp32, one per weight block
 *   out      [M,N]                         f32 / f16 / bf16 (`out_dtype`)
 *
 * M, N, K need not be multiples of the block sizes. block_n = block_k = 128
 * with K and N multiples of 16 takes the tcgen05 kernel; every other legal
 * combination takes a slower general kernel with the same results.
 * Same contract as the reference: gemm.h:79-98, gemm_fp8_blockwise.cu:218-302.
 */
KS_API ks_status_t ks_gemm_fp8_blockwise(void* out, const void* a_fp8,
                                         const void* b_fp8,
                                         const float* a_scale,
                                         const float* b_scale, int64_t m,
                                         int64_t n, int64_t k, int block_n,
                                         int block_k, ks_dtype_t fp8_dtype,
                                         ks_dtype_t out_dtype,
                                         ks_stream_t stream);

/*
 * Same product with the weight stored the way checkpoints hold it:
 *   b_fp8    [N,K]                               (one row per output column)
 *   b_scale  [ceil(N/block_n), ceil(K/block_k)]
 * Everything else as ks_gemm_fp8_blockwise. The reference has no C entry for
 * this layout; its Python router reaches it through an external provider
 * (bindings/python/kernel_set/backends/_registry.py:416-424), so this symbol
 * is an addition, not a replacement.
 */
KS_API ks_status_t ks_gemm_fp8_blockwise_nt(void* out, const void* a_fp8,
                                            const void* b_fp8,
                                            const float* a_scale,
                                            const float* b_scale, int64_t m,
                                            int64_t n, int64_t k, int block_n,
                                            int block_k, ks_dtype_t fp8_dtype,
                                            ks_dtype_t out_dtype,
                                            ks_stream_t stream);

/*
 * The block-scaled GEMM (128 x 128 weight blocks, 1 x 128 activation groups)
 * with the activation scales stored column-major, as
 * ks_quantize_fp8_group_colscale writes them:
 *   a_scale_t[kb * a_scale_ld + m]
 * b_layout 0: b_fp8 [K,N], b_scale [ceil(K/128), ceil(N/128)];
 * b_layout 1: b_fp8 [N,K], b_scale [ceil(N/128), ceil(K/128)].
 * The epilogue's scale loads of a warp then touch one 128-byte line per
 * K-block instead of 32. Only the tcgen05 kernel serves this entry (K, and N
 * for [K,N], multiples of 16; UNSUPPORTED_SHAPE otherwise). No counterpart in
 * the reference.
 */
KS_API ks_status_t ks_gemm_fp8_blockwise_colscale(void* out, const void* a_fp8,
                                                  const void* b_fp8,
                                                  const float* a_scale_t,
                                                  int64_t a_scale_ld,
                                                  const float* b_scale,
                                                  int64_t m, int64_t n,
                                                  int64_t k, int b_layout,
                                                  ks_dtype_t fp8_dtype,
                                                  ks_dtype_t out_dtype,
                                                  ks_stream_t stream);

/*
 * The block-scaled GEMM with a scattered output, for a row-parallel (K-split)
 * layer: rows [b * rows_per_part, (b + 1) * rows_per_part) of this call's product
 * are written to out_parts[b], a [rows_per_part, n] matrix of `out_dtype` that may
 * live in another GPU's memory (a peer-mapped address, e.g. rank b's buffer of a
 * symmetric allocation, offset to the slot of the calling rank). The finished
 * tiles leave by TMA stores, so the transfer over NVLink runs under the tiles
 * still being computed; ks_sum_parts on the owning rank then adds the ranks'
 * slots. `out_parts` is a HOST array of num_parts (1..8) device pointers.
 * rows_per_part a multiple of 128, m = num_parts * rows_per_part, rows 16-byte
 * aligned. Only the tcgen05 kernel serves this entry. No counterpart in the
 * reference, which has no multi-GPU path.
 */
KS_API ks_status_t ks_gemm_fp8_blockwise_scatter(void* const* out_parts,
                                                 int num_parts,
                                                 int64_t rows_per_part,
                                                 const void* a_fp8,
                                                 const void* b_fp8,
                                                 const float* a_scale,
                                                 const float* b_scale,
                                                 int64_t m, int64_t n,
                                                 int64_t k, int b_layout,
                                                 ks_dtype_t fp8_dtype,
                                                 ks_dtype_t out_dtype,
                                                 ks_stream_t stream);

/*
 * out = sum over q of parts[q], parts [num_parts, rows, n] of `part_dtype`
 * (f32 / f16 / bf16), added in part order in fp32 and rounded once to
 * `out_dtype`; the result is written to every one of the num_dsts (1..8)
 * pointers of the HOST array `dsts` (this GPU's copy and, for an all-gather by
 * peer stores, other GPUs'). rows * n a multiple of 8; 16-byte aligned
 * pointers. No counterpart in the reference.
 */
KS_API ks_status_t ks_sum_parts(void* const* dsts, int num_dsts,
                                const void* parts, int num_parts,
                                int64_t rows, int64_t n,
                                ks_dtype_t part_dtype, ks_dtype_t out_dtype,
                                ks_stream_t stream);

KS_END_EXTERN_C

#endif /* KERNEL_SET_GEMM_H_ */
