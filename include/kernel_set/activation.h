/*
 * SwiGLU, the activation between the two expert GEMMs of a gated MLP.
 *
 * Replaces ks_swiglu and ks_swiglu_packed of include/kernel_set/activation.h:
 * 26-35 of the reference project (kernels/src/activation/gated_mlp.cu) and adds
 * the form fused with the 1 x 128 FP8 quantizer. The other activations of that
 * header are a different code path and are not exported by this library.
 */
#ifndef KERNEL_SET_ACTIVATION_H_
#define KERNEL_SET_ACTIVATION_H_

#include "kernel_set/types.h"

KS_BEGIN_EXTERN_C

/* out[r,c] = silu(gate[r,c]) * up[r,c], silu(x) = x / (1 + exp(-x)) in fp32,
 * one rounding to `dtype` (f32 / f16 / bf16). gate, up, out: [rows, inter].
 * Same contract as the reference: activation.h:26-29. */
KS_API ks_status_t ks_swiglu(void* out, const void* gate, const void* up,
                             int64_t rows, int64_t inter, ks_dtype_t dtype,
                             ks_stream_t stream);

/* Packed form: input [rows, 2*inter] with gate = input[:, :inter] and
 * up = input[:, inter:]; out [rows, inter].
 * Same contract as the reference: activation.h:31-35. */
KS_API ks_status_t ks_swiglu_packed(void* out, const void* input, int64_t rows,
                                    int64_t inter, ks_dtype_t dtype,
                                    ks_stream_t stream);

/* ks_swiglu_packed fused with ks_quantize_fp8_group(group_size = 128): the
 * activation is rounded to the input type (f16 / bf16) and quantized, giving
 * codes and scales bit-identical to the two calls run one after the other.
 *   out_fp8 [rows, inter], out_scale [rows, inter/128]; inter % 128 == 0.
 * No counterpart in the reference. */
KS_API ks_status_t ks_swiglu_packed_quant_fp8(void* out_fp8, float* out_scale,
                                              const void* input, int64_t rows,
                                              int64_t inter,
                                              ks_dtype_t in_dtype,
                                              ks_dtype_t fp8_dtype,
                                              ks_stream_t stream);

KS_END_EXTERN_C

#endif /* KERNEL_SET_ACTIVATION_H_ */
