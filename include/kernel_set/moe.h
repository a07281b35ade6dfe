/*
 * Mixture-of-experts layer: softmax top-k gate, the permutation that sorts
 * (token, slot) pairs by expert, row gather / weighted scatter, and the
 * grouped (per-expert) GEMMs over rows sorted by expert.
 *
 * Replaces ks_moe_gate_softmax_topk, ks_moe_compute_permutation,
 * ks_moe_permute, ks_moe_unpermute and ks_moe_grouped_gemm of
 * include/kernel_set/moe.h:14-65 of the reference project, and adds the FP8
 * forms (block-scaled grouped GEMM, gather fused with the 1 x 128 quantizer)
 * that the reference only reaches through external providers. The sigmoid
 * group-limited gate of that header (moe.h:25-31) is not exported here.
 */
#ifndef KERNEL_SET_MOE_H_
#define KERNEL_SET_MOE_H_

#include "kernel_set/types.h"

KS_BEGIN_EXTERN_C

/*
 * Softmax over the experts, then the top_k largest probabilities.
 *   logits       [num_tokens, num_experts]  f32 / f16 / bf16 (`dtype`)
 *   out_weights  [num_tokens, top_k]  fp32, descending; divided by their sum
 *                                     when `renormalize` is non-zero
 *   out_indices  [num_tokens, top_k]  int32 expert ids; among equal
 *                                     probabilities the lowest id comes first
 * At most 1024 experts and top_k 32 (UNSUPPORTED_SHAPE beyond), as the
 * reference. Same contract as the reference: moe.h:14-23, moe_gate.cu:43-119.
 */
KS_API ks_status_t ks_moe_gate_softmax_topk(float* out_weights,
                                            int32_t* out_indices,
                                            const void* logits,
                                            int64_t num_tokens,
                                            int num_experts, int top_k,
                                            int renormalize, ks_dtype_t dtype,
                                            ks_stream_t stream);

/*
 * Counting sort of the routed pairs by expert.
 *   topk_indices      [num_tokens, top_k]  int32
 *   sorted_token_ids  [num_tokens*top_k]   int32: pair ids (token*top_k + slot)
 *                                          grouped by expert
 *   expert_offsets    [num_experts+1]      int32 group boundaries
 * The sort is stable (pairs of one expert keep their order), where the
 * reference leaves the order inside a group unspecified; pairs whose expert id
 * is out of range are dropped and the unused tail of sorted_token_ids is
 * filled with -1. One launch, no allocation, no synchronisation (the
 * reference does all three per call, moe_permute.cu:205-242).
 * Same contract otherwise: moe.h:33-40.
 */
KS_API ks_status_t ks_moe_compute_permutation(int32_t* sorted_token_ids,
                                              int32_t* expert_offsets,
                                              const int32_t* topk_indices,
                                              int64_t num_tokens,
                                              int num_experts, int top_k,
                                              ks_stream_t stream);

/*
 * permuted[r, :] = input[sorted_token_ids[r] / top_k, :]; rows whose id is
 * negative or out of range are zero-filled.
 *   input [num_tokens, hidden], permuted [num_tokens*top_k, hidden], any of
 *   f32 / f16 / bf16 / e4m3 / e5m2.
 * Same contract as the reference: moe.h:42-47, moe_permute.cu:107-127.
 */
KS_API ks_status_t ks_moe_permute(void* permuted, const void* input,
                                  const int32_t* sorted_token_ids,
                                  int64_t num_tokens, int top_k,
                                  int64_t hidden, ks_dtype_t dtype,
                                  ks_stream_t stream);

/*
 * ks_moe_permute fused with ks_quantize_fp8_group(group_size = 128): row r of
 * the output holds the fp8 codes and the 1 x 128 scales of input row
 * sorted_token_ids[r] / top_k, bit-identical to running the two calls one
 * after the other, without the 16-bit intermediate.
 *   out_fp8 [num_tokens*top_k, hidden], out_scale [num_tokens*top_k, hidden/128]
 * hidden must be a multiple of 128. No counterpart in the reference.
 */
KS_API ks_status_t ks_moe_permute_quant_fp8(void* out_fp8, float* out_scale,
                                            const void* input,
                                            const int32_t* sorted_token_ids,
                                            int64_t num_tokens, int top_k,
                                            int64_t hidden,
                                            ks_dtype_t in_dtype,
                                            ks_dtype_t fp8_dtype,
                                            ks_stream_t stream);

/*
 * out[t, :] = sum over slots k of routing_weights[t, k] * permuted[row of
 * pair (t, k), :], slots added in order in fp32, one rounding at the end.
 *   permuted [num_tokens*top_k, hidden], out [num_tokens, hidden], f32/f16/bf16
 *   routing_weights [num_tokens, top_k] fp32
 * The inverse permutation lives in a library-owned, stream-ordered buffer
 * (first use of a stream allocates it; do that before any stream capture); the
 * reference allocates, synchronises and frees per call
 * (moe_permute.cu:317-375). Same contract otherwise: moe.h:49-56.
 */
KS_API ks_status_t ks_moe_unpermute(void* out, const void* permuted,
                                    const int32_t* sorted_token_ids,
                                    const float* routing_weights,
                                    int64_t num_tokens, int top_k,
                                    int64_t hidden, ks_dtype_t dtype,
                                    ks_stream_t stream);

/*
 * For every expert e: C[off_e : off_{e+1}, :] = A[off_e : off_{e+1}, :] . B[e]
 *
 *   a               [total_rows, K]  `dtype`
 *   b               [E, K, N]        `dtype`
 *   expert_offsets  [E+1]            int32, non-decreasing, off_0 = 0
 *   c               [total_rows, N]  `dtype`
 * dtype: f32 / f16 / bf16 / e4m3 / e5m2, fp32 accumulation, no scales (fp8
 * operands are multiplied as the raw values they encode and C is written in
 * the same fp8 type). total_rows == 0 returns success without a launch.
 * Unlike the reference (moe_grouped_gemm.cu:162-192) the call neither
 * allocates nor synchronises.
 */
KS_API ks_status_t ks_moe_grouped_gemm(void* c, const void* a, const void* b,
                                       const int32_t* expert_offsets,
                                       int num_experts, int64_t total_rows,
                                       int64_t n, int64_t k, ks_dtype_t dtype,
                                       ks_stream_t stream);

/*
 * Per expert e the block-scaled product of ks_gemm_fp8_blockwise:
 *   out[r,n] = sum_kb a_scale[r,kb] * b_scale[e,..] * sum_{k in kb} A8[r,k] * B8[e][..]
 *
 *   a_fp8    [total_rows, K]            fp8
 *   a_scale  [total_rows, ceil(K/bk)]   fp32
 *   b_layout 0: b_fp8 [E, K, N], b_scale [E, ceil(K/bk), ceil(N/bn)]
 *   b_layout 1: b_fp8 [E, N, K], b_scale [E, ceil(N/bn), ceil(K/bk)]
 *   out      [total_rows, N]            f32 / f16 / bf16
 * No counterpart in the reference's C ABI: its ks_moe_grouped_gemm carries no
 * scale arguments, and its router passes a_scale/b_scale only to external
 * providers (backends/_registry.py:1677-1700).
 */
KS_API ks_status_t ks_moe_grouped_gemm_fp8_blockwise(
    void* out, const void* a_fp8, const void* b_fp8, const float* a_scale,
    const float* b_scale, const int32_t* expert_offsets, int num_experts,
    int64_t total_rows, int64_t n, int64_t k, int block_n, int block_k,
    int b_layout, ks_dtype_t fp8_dtype, ks_dtype_t out_dtype,
    ks_stream_t stream);

/*
 * The same product over the masked layout that CUDA-graph decode uses: every
 * expert owns a fixed slab of max_m rows and computes only its first
 * masked_m[e] of them, so the launch does not depend on the routing.
 *   a_fp8    [E, max_m, K]            a_scale [E, max_m, ceil(K/bk)]
 *   masked_m [E] int32 on the device  (values are clamped to [0, max_m])
 *   out      [E, max_m, N]; rows at or beyond masked_m[e] are left untouched
 *   b_fp8 / b_scale / b_layout as above.
 * Needs block_n = block_k = 128 (UNSUPPORTED_SHAPE otherwise). The reference
 * reaches this layout only through an external provider
 * (backends/_registry.py:1686-1689); it has no C entry for it.
 */
KS_API ks_status_t ks_moe_grouped_gemm_fp8_blockwise_masked(
    void* out, const void* a_fp8, const void* b_fp8, const float* a_scale,
    const float* b_scale, const int32_t* masked_m, int num_experts,
    int64_t max_m, int64_t n, int64_t k, int block_n, int block_k,
    int b_layout, ks_dtype_t fp8_dtype, ks_dtype_t out_dtype,
    ks_stream_t stream);

/*
 * Expert-parallel dispatch and combine through peer memory (no counterpart in the
 * reference, which has no multi-GPU path). Experts are split contiguously over the
 * ranks, `experts_per_rank` each (the last rank may own fewer). `counts` is the
 * all-gathered matrix int32 [world, world * experts_per_rank]: counts[s][e] = rows
 * rank s routes to expert e (0 for padding experts).
 *
 * ks_moe_dispatch_plan (one small kernel) derives, for the calling rank:
 *   dst_base      [world * experts_per_rank]   row at which this rank's rows of expert e
 *                                              start in the receive buffer of rank
 *                                              e / experts_per_rank
 *   local_offsets [experts_per_rank + 1]       expert offsets of the rows this rank receives
 *                                              (expert-major, inside an expert by source)
 *   seg_start     [experts_per_rank * world + 1]  first received row of (expert, source)
 *   ret_base      [experts_per_rank * world]   position of that segment's first row in
 *                                              the source rank's sorted order
 */
KS_API ks_status_t ks_moe_dispatch_plan(int32_t* dst_base, int32_t* local_offsets,
                                        int32_t* seg_start, int32_t* ret_base,
                                        const int32_t* counts, int world, int rank,
                                        int experts_per_rank, ks_stream_t stream);

/*
 * ks_moe_permute_quant_fp8 with every output row written to its destination rank:
 * sorted row r of expert e goes to row dst_base[e] + r - expert_offsets[e] of
 * dst_fp8[e / experts_per_rank] ([capacity_rows, hidden] fp8) and its scales to the
 * same row of dst_scale[...] ([capacity_rows, hidden / 128] f32). `dst_fp8` and
 * `dst_scale` are HOST arrays of `world` device pointers (peer-mapped addresses; the
 * entry of the calling rank is its own buffer). Rows outside [0, capacity_rows) are
 * dropped. Codes and scales are those of ks_quantize_fp8_group(group_size = 128).
 * The caller places a cross-rank barrier between this call and the use of the buffers.
 */
KS_API ks_status_t ks_moe_permute_quant_fp8_scatter(
    void* const* dst_fp8, float* const* dst_scale, int world, int64_t capacity_rows,
    const int32_t* dst_base, const int32_t* expert_offsets, int num_experts,
    int experts_per_rank, const void* input, const int32_t* sorted_token_ids,
    int64_t num_tokens, int top_k, int64_t hidden, ks_dtype_t in_dtype,
    ks_dtype_t fp8_dtype, ks_stream_t stream);

/*
 * The way back: received row i (i < seg_start[segments], read on the device) of `src`
 * ([capacity_rows, hidden] `dtype`) lies in segment j (seg_start[j] <= i) and is copied
 * to row ret_base[j] + i - seg_start[j] of dst[j % world] ([dst_rows, hidden]).
 * `dst` is a HOST array of `world` device pointers. segments = experts of this rank x world.
 */
KS_API ks_status_t ks_moe_scatter_rows(void* const* dst, int world, int64_t dst_rows,
                                       const void* src, int64_t capacity_rows,
                                       const int32_t* seg_start, const int32_t* ret_base,
                                       int segments, int64_t hidden, ks_dtype_t dtype,
                                       ks_stream_t stream);

KS_END_EXTERN_C

#endif /* KERNEL_SET_MOE_H_ */
