// C ABI of the int4 weight-only GEMM: argument checks with the status codes
// of the reference (kernels/src/gemm/gemm_w4a16.cu:151-182), then the kernel
// choice.
#include "common.cuh"
#include "gemm_general.cuh"
#include <cstdlib>

#include "kernel_set/gemm.h"
#include "sm100_w4a16.cuh"

namespace {
// KS_B200_W4A16_OPERAND=smem|tmem pins how decode shapes pass the dequantised weights to
// the tensor core (tests and profiling only).
int env_operand_path() {
  const char* v = std::getenv("KS_B200_W4A16_OPERAND");
  if (v == nullptr) return 0;
  return v[0] == 's' ? 1 : (v[0] == 't' ? 2 : 0);
}
}  // namespace

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
  cudaStream_t s = as_stream(stream);
  {
    // KS_B200_W4A16_PATH=general pins the general kernel, =tcgen05 refuses to
    // fall back; unset means "choose" (tests and profiling only).
    const char* env = std::getenv("KS_B200_W4A16_PATH");
    const int path = env == nullptr ? 0 : (env[0] == 'g' ? 1 : (env[0] == 't' ? 2 : 0));
    sm100::W4A16Args args;
    args.c = c; args.a = a; args.b_packed = b_packed; args.scales = scales; args.zeros = zeros; args.bias = bias;
    args.m = m; args.n = n; args.k = k; args.group_size = gs; args.dtype = dtype;
    args.operand_path = env_operand_path();
    if (path != 1 && sm100::w4a16_eligible(args)) return sm100::launch_w4a16(args, s);
    if (path == 2) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gemm_w4a16: shape not eligible for the tcgen05 kernel");
  }
  const int64_t tiles_m = (m + general::kTM - 1) / general::kTM;
  const int64_t tiles_n = (n + general::kTN - 1) / general::kTN;
  if (tiles_m > 2147483647LL || tiles_n > 65535LL)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gemm_w4a16: tile grid exceeds CUDA grid limits");
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

// Allocation-free variant: same checks, same kernels, but the tcgen05 kernel's
// split-K scratch comes from a fixed array inside the library (see
// sm100_w4a16.cu). Shapes the tcgen05 kernel declines run on the general
// kernel, which needs no scratch at all.
extern "C" ks_status_t ks_gemm_w4a16_static_scratch(void* c, const void* a, const void* b_packed,
                                                    const void* scales, const void* zeros, const void* bias,
                                                    int64_t m, int64_t n, int64_t k, int group_size,
                                                    ks_dtype_t dtype, ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_gemm_w4a16_static_scratch";
  KSB_REQUIRE_PTR(c);
  KSB_REQUIRE_PTR(a);
  KSB_REQUIRE_PTR(b_packed);
  KSB_REQUIRE_PTR(scales);
  if (m <= 0 || n <= 0 || k <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_gemm_w4a16_static_scratch: bad shape");
  if (k % 2 != 0)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gemm_w4a16_static_scratch: K must be even (two int4 per byte)");
  if (group_size <= 0 && k > INT32_MAX)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gemm_w4a16_static_scratch: K too large for a single group");
  const int gs = group_size > 0 ? group_size : static_cast<int>(k);
  if (k % gs != 0) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gemm_w4a16_static_scratch: group_size must divide K");
  if (dtype != KS_DTYPE_F16 && dtype != KS_DTYPE_BF16)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_gemm_w4a16_static_scratch: unsupported dtype");
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  st = poll_kernel_fault(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  sm100::W4A16Args args;
  args.c = c; args.a = a; args.b_packed = b_packed; args.scales = scales; args.zeros = zeros; args.bias = bias;
  args.m = m; args.n = n; args.k = k; args.group_size = gs; args.dtype = dtype;
    args.operand_path = env_operand_path();
  if (sm100::w4a16_eligible(args)) return sm100::launch_w4a16_static(args, s);
  const int64_t tiles_m = (m + general::kTM - 1) / general::kTM;
  const int64_t tiles_n = (n + general::kTN - 1) / general::kTN;
  if (tiles_m > 2147483647LL || tiles_n > 65535LL)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gemm_w4a16_static_scratch: tile grid exceeds CUDA grid limits");
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
