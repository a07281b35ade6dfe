// C ABI of the int4 weight-only GEMM: argument checks with the status codes
// of the reference (kernels/src/gemm/gemm_w4a16.cu:151-182), then the kernel
// choice.
#include "common.cuh"
#include "gemm_general.cuh"
#include <cstdlib>
#include <string>

#include "kernel_set/gemm.h"
#include "sm100_w4a16.cuh"

namespace {

// Environment switches for tests and profiling, read once per process:
//   KS_B200_W4A16_PATH=general|tcgen05|decode  pins the kernel (tcgen05 / decode refuse
//                                              shapes they cannot take instead of falling back)
//   KS_B200_W4A16_OPERAND=smem|tmem            how the tcgen05 kernel passes the weights on
// KS_B200_ENV_RELOAD=1 makes every call read them again (the test-suite flips them).
struct EnvChoice {
  int path = 0;      // 0 choose, 1 general, 2 tcgen05, 3 decode
  int operand = 0;   // 0 choose, 1 shared memory, 2 tensor memory
};
EnvChoice read_env() {
  EnvChoice c;
  if (const char* v = std::getenv("KS_B200_W4A16_PATH"))
    c.path = v[0] == 'g' ? 1 : (v[0] == 't' ? 2 : (v[0] == 'd' ? 3 : 0));
  if (const char* v = std::getenv("KS_B200_W4A16_OPERAND")) c.operand = v[0] == 's' ? 1 : (v[0] == 't' ? 2 : 0);
  return c;
}
EnvChoice env_choice() {
  static const bool reload = std::getenv("KS_B200_ENV_RELOAD") != nullptr;
  static const EnvChoice cached = read_env();
  return reload ? read_env() : cached;
}

// Shared body of ks_gemm_w4a16 and ks_gemm_w4a16_static_scratch; `static_scratch`
// selects where the fast kernels' split-K workspace comes from.
ks_status_t gemm_w4a16_impl(const char* where, bool static_scratch, void* c, const void* a, const void* b_packed,
                            const void* scales, const void* zeros, const void* bias, int64_t m, int64_t n,
                            int64_t k, int group_size, ks_dtype_t dtype, ks_stream_t stream) {
  using namespace ksb;
  const std::string w(where);
  KSB_REQUIRE_PTR(c);
  KSB_REQUIRE_PTR(a);
  KSB_REQUIRE_PTR(b_packed);
  KSB_REQUIRE_PTR(scales);
  if (m <= 0 || n <= 0 || k <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, w + ": bad shape");
  if (k % 2 != 0) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, w + ": K must be even (two int4 per byte)");
  if (group_size <= 0 && k > INT32_MAX) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, w + ": K too large for a single group");
  const int gs = group_size > 0 ? group_size : static_cast<int>(k);
  if (k % gs != 0) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, w + ": group_size must divide K");
  if (dtype != KS_DTYPE_F16 && dtype != KS_DTYPE_BF16) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, w + ": unsupported dtype");
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  st = poll_kernel_fault(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  {
    const EnvChoice env = env_choice();
    sm100::W4A16Args args;
    args.c = c; args.a = a; args.b_packed = b_packed; args.scales = scales; args.zeros = zeros; args.bias = bias;
    args.m = m; args.n = n; args.k = k; args.group_size = gs; args.dtype = dtype;
    args.operand_path = env.operand;
    args.kernel = env.path == 2 ? 1 : (env.path == 3 ? 2 : 0);
    if (env.path == 3 && !sm100::decode::eligible(args))
      KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, w + ": shape not eligible for the decode kernel");
    if (env.path != 1 && (sm100::w4a16_eligible(args) || (args.kernel != 1 && sm100::decode::eligible(args))))
      return static_scratch ? sm100::launch_w4a16_static(args, s) : sm100::launch_w4a16(args, s);
    if (env.path == 2) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, w + ": shape not eligible for the tcgen05 kernel");
  }
  // general kernel: any shape, no workspace
  const int64_t tiles_m = (m + general::kTM - 1) / general::kTM;
  const int64_t tiles_n = (n + general::kTN - 1) / general::kTN;
  if (tiles_m > 2147483647LL || tiles_n > 65535LL)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, w + ": tile grid exceeds CUDA grid limits");
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

}  // namespace

extern "C" ks_status_t ks_gemm_w4a16(void* c, const void* a, const void* b_packed, const void* scales,
                                     const void* zeros, const void* bias, int64_t m, int64_t n, int64_t k,
                                     int group_size, ks_dtype_t dtype, ks_stream_t stream) {
  return gemm_w4a16_impl("ks_gemm_w4a16", false, c, a, b_packed, scales, zeros, bias, m, n, k, group_size, dtype,
                         stream);
}

// Allocation-free variant: same checks, same kernels, but the fast kernels'
// split-K scratch comes from a fixed array inside the library (see
// sm100_w4a16.cu). Shapes the fast kernels decline run on the general
// kernel, which needs no scratch at all.
extern "C" ks_status_t ks_gemm_w4a16_static_scratch(void* c, const void* a, const void* b_packed,
                                                    const void* scales, const void* zeros, const void* bias,
                                                    int64_t m, int64_t n, int64_t k, int group_size,
                                                    ks_dtype_t dtype, ks_stream_t stream) {
  return gemm_w4a16_impl("ks_gemm_w4a16_static_scratch", true, c, a, b_packed, scales, zeros, bias, m, n, k,
                         group_size, dtype, stream);
}
