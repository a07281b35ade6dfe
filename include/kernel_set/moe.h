/*
 * Grouped (per-expert) GEMM over rows already sorted by expert.
 *
 * Replaces ks_moe_grouped_gemm of include/kernel_set/moe.h:57-65 of the
 * reference project and adds the FP8 block-scaled form that the reference
 * only reaches through external providers. Gating and permutation kernels of
 * that header are not exported here.
 */
#ifndef KERNEL_SET_MOE_H_
#define KERNEL_SET_MOE_H_

#include "kernel_set/types.h"

KS_BEGIN_EXTERN_C

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

KS_END_EXTERN_C

#endif /* KERNEL_SET_MOE_H_ */
