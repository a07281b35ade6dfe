// C ABI of the int4 weight-only GEMM: argument checks with the status codes
// of the reference (kernels/src/gemm/gemm_w4a16.cu:151-182), then the kernel
// choice.
#include "common.cuh"
#include "gemm_general.cuh"
#include "kernel_set/gemm.h"

extern "C" ks_status_t ks_gemm_w4a16(void* c, const void* a, const void* b_packed, const void* scales,
                                     const void* zeros, const void* bias, int64_t m, int64_t n, int64_t k,
                                     int group_size, ks_dtype_t dtype, ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_gemm_w4a16";
  KSB_REQUIRE_PTR(c);
  KSB_REQUIRE_PTR(a);
  KSB_REQUIRE_PTR(b_packed);
  KSB_REQUIRE_PTR(scales);
  if (m <= 0 || n <= 0 || k <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_gemm_w4a16: bad shape");
  if (k % 2 != 0) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gemm_w4a16: K must be even (two int4 per byte)");
  if (group_size <= 0 && k > INT32_MAX)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gemm_w4a16: K too large for a single group");
  const int gs = group_size > 0 ? group_size : static_cast<int>(k);
  if (k % gs != 0) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gemm_w4a16: group_size must divide K");
  if (dtype != KS_DTYPE_F16 && dtype != KS_DTYPE_BF16)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_gemm_w4a16: unsupported dtype");
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  st = poll_kernel_fault(where);
  if (st != KS_SUCCESS) return st;
  const int64_t tiles_m = (m + general::kTM - 1) / general::kTM;
  const int64_t tiles_n = (n + general::kTN - 1) / general::kTN;
  if (tiles_m > 2147483647LL || tiles_n > 65535LL)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gemm_w4a16: tile grid exceeds CUDA grid limits");
  cudaStream_t s = as_stream(stream);
  dim3 grid(static_cast<unsigned>(tiles_m), static_cast<unsigned>(tiles_n));
  if (dtype == KS_DTYPE_F16) {
    general::w4a16_kernel<__half><<<grid, general::kThreads, 0, s>>>(
        static_cast<__half*>(c), static_cast<const __half*>(a), static_cast<const uint8_t*>(b_packed),
        static_cast<const __half*>(scales), static_cast<const __half*>(zeros), static_cast<const __half*>(bias), m,
        n, k, gs);
  } else {
    general::w4a16_kernel<__nv_bfloat16><<<grid, general::kThreads, 0, s>>>(
        static_cast<__nv_bfloat16*>(c), static_cast<const __nv_bfloat16*>(a),
        static_cast<const uint8_t*>(b_packed), static_cast<const __nv_bfloat16*>(scales),
        static_cast<const __nv_bfloat16*>(zeros), static_cast<const __nv_bfloat16*>(bias), m, n, k, gs);
  }
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}
