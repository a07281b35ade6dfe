// Entry points of the reference project's C ABI that lie outside the quantized-GEMM path
// this library implements. They are exported so that bindings which resolve every symbol
// of the reference's headers when they load (cgo, a Rust build script, an eager dlsym
// loop) still link against this library; each returns KS_ERROR_NOT_IMPLEMENTED ("declared
// but no backend yet", include/kernel_set/types.h:30 of the reference) and records its
// name in the thread's error string. The reference's own link stub does the same for
// every symbol (bindings/verify/stub_kernel_set.c).
//
// The stubs take no parameters: with C linkage the name is all a binder resolves, and the
// platform's C calling convention lets a callee ignore the arguments it was given. The
// list below is the set difference between the reference's headers
// (include/kernel_set/*.h, 89 functions) and this library's own.
#include "common.cuh"
#include "kernel_set/export.h"

#define KSB_NOT_IMPLEMENTED(name)                                                        \
  extern "C" KS_API ks_status_t name(void) {                                             \
    ::ksb::set_last_error(#name ": not part of this library (quantized-GEMM path only)"); \
    return KS_ERROR_NOT_IMPLEMENTED;                                                     \
  }


// activation.h
KSB_NOT_IMPLEMENTED(ks_geglu)
KSB_NOT_IMPLEMENTED(ks_gelu)
KSB_NOT_IMPLEMENTED(ks_relu)
KSB_NOT_IMPLEMENTED(ks_silu)
KSB_NOT_IMPLEMENTED(ks_swiglu_backward)

// attention.h
KSB_NOT_IMPLEMENTED(ks_attention_state_merge)
KSB_NOT_IMPLEMENTED(ks_dsa_topk_select)
KSB_NOT_IMPLEMENTED(ks_flash_attn)
KSB_NOT_IMPLEMENTED(ks_flash_attn_backward)
KSB_NOT_IMPLEMENTED(ks_flash_attn_varlen)
KSB_NOT_IMPLEMENTED(ks_mla_decode)
KSB_NOT_IMPLEMENTED(ks_mla_decode_split_k)
KSB_NOT_IMPLEMENTED(ks_paged_attn_decode)
KSB_NOT_IMPLEMENTED(ks_paged_attn_decode_split_k)
KSB_NOT_IMPLEMENTED(ks_reshape_and_cache)

// elementwise.h
KSB_NOT_IMPLEMENTED(ks_add)
KSB_NOT_IMPLEMENTED(ks_add_residual)
KSB_NOT_IMPLEMENTED(ks_axpby)
KSB_NOT_IMPLEMENTED(ks_cast)
KSB_NOT_IMPLEMENTED(ks_mul)
KSB_NOT_IMPLEMENTED(ks_scale)

// embedding.h
KSB_NOT_IMPLEMENTED(ks_embedding_backward)
KSB_NOT_IMPLEMENTED(ks_embedding_lookup)

// gemm.h
KSB_NOT_IMPLEMENTED(ks_gemm)
KSB_NOT_IMPLEMENTED(ks_gemm_batched)
KSB_NOT_IMPLEMENTED(ks_gemm_bias_act)
KSB_NOT_IMPLEMENTED(ks_gemm_nvfp4)

// linear_attn.h
KSB_NOT_IMPLEMENTED(ks_gated_delta_rule)
KSB_NOT_IMPLEMENTED(ks_gated_linear_attn)
KSB_NOT_IMPLEMENTED(ks_rwkv_wkv7)

// loss.h
KSB_NOT_IMPLEMENTED(ks_cross_entropy)
KSB_NOT_IMPLEMENTED(ks_fused_linear_cross_entropy)

// moe.h
KSB_NOT_IMPLEMENTED(ks_moe_gate_sigmoid_group_topk)

// norm.h
KSB_NOT_IMPLEMENTED(ks_fused_rmsnorm_gated)
KSB_NOT_IMPLEMENTED(ks_layer_norm)
KSB_NOT_IMPLEMENTED(ks_layer_norm_backward)
KSB_NOT_IMPLEMENTED(ks_rms_norm_backward)
KSB_NOT_IMPLEMENTED(ks_rms_norm_residual)

// optimizer.h
KSB_NOT_IMPLEMENTED(ks_adamw)
KSB_NOT_IMPLEMENTED(ks_global_grad_norm)
KSB_NOT_IMPLEMENTED(ks_sgd_momentum)

// quant.h
KSB_NOT_IMPLEMENTED(ks_dequantize_fp8)
KSB_NOT_IMPLEMENTED(ks_dequantize_int8)
KSB_NOT_IMPLEMENTED(ks_quantize_fp8)
KSB_NOT_IMPLEMENTED(ks_quantize_int8)
KSB_NOT_IMPLEMENTED(ks_quantize_nvfp4)

// rope.h
KSB_NOT_IMPLEMENTED(ks_rope)
KSB_NOT_IMPLEMENTED(ks_rope_backward)
KSB_NOT_IMPLEMENTED(ks_rope_gather)
KSB_NOT_IMPLEMENTED(ks_rope_inplace)

// sampling.h
KSB_NOT_IMPLEMENTED(ks_argmax)
KSB_NOT_IMPLEMENTED(ks_log_softmax)
KSB_NOT_IMPLEMENTED(ks_sample)
KSB_NOT_IMPLEMENTED(ks_softmax)

// ssm.h
KSB_NOT_IMPLEMENTED(ks_causal_conv1d)
KSB_NOT_IMPLEMENTED(ks_selective_scan)
KSB_NOT_IMPLEMENTED(ks_selective_scan_update)
