/*
 * RMSNorm, the usual producer of the activations that the 1 x 128 FP8 quantizer
 * and the block-scaled GEMM consume, alone and fused with that quantizer.
 *
 * Replaces ks_rms_norm of include/kernel_set/norm.h:16-19 of the reference
 * project (kernels/src/norm/rms_norm.cu:19-42) and adds the fused form. The
 * other normalisations of that header are a different code path and are
 * exported only as NOT_IMPLEMENTED stubs.
 */
#ifndef KERNEL_SET_NORM_H_
#define KERNEL_SET_NORM_H_

#include "kernel_set/types.h"

KS_BEGIN_EXTERN_C

/* out[r,:] = round(input[r,:] * rsqrt(mean(input[r,:]^2) + eps)) * weight:
 * the normalised value is rounded to `dtype` (f32 / f16 / bf16), multiplied by
 * the weight and rounded again, as the reference's torch statement of the op
 * does (benchmarks/bench.py:877-879). input, out [rows, cols]; weight [cols].
 * Same contract as the reference: norm.h:16-19. */
KS_API ks_status_t ks_rms_norm(void* out, const void* input, const void* weight,
                               int64_t rows, int64_t cols, float eps,
                               ks_dtype_t dtype, ks_stream_t stream);

/* ks_rms_norm fused with ks_quantize_fp8_group(group_size = 128): the
 * normalised row is rounded to the input type (f16 / bf16) and quantized,
 * giving codes and scales bit-identical to the two calls run one after the
 * other; the row is read once and the 16-bit intermediate is never written.
 *   out_fp8 [rows, cols], out_scale [rows, cols/128]; cols % 128 == 0,
 *   cols <= 8192. No counterpart in the reference. */
KS_API ks_status_t ks_rms_norm_quant_fp8(void* out_fp8, float* out_scale,
                                         const void* input, const void* weight,
                                         int64_t rows, int64_t cols, float eps,
                                         ks_dtype_t in_dtype,
                                         ks_dtype_t fp8_dtype,
                                         ks_stream_t stream);

KS_END_EXTERN_C

#endif /* KERNEL_SET_NORM_H_ */
