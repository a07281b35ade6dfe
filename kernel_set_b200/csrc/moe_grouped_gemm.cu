// C ABI of the unscaled grouped GEMM (reference: kernels/src/moe/
// moe_grouped_gemm.cu:136-198). One launch, no allocation, no host sync: each
// block finds its (expert, row tile) from the offsets itself, where the
// reference builds a schedule with a one-thread kernel into a buffer it
// allocates and frees around a stream synchronisation.
#include "common.cuh"
#include "gemm_general.cuh"
#include "kernel_set/moe.h"

namespace ksb {
namespace {
template <typename T>
void launch(void* c, const void* a, const void* b, const int32_t* offs, int e, int64_t rows, int64_t n, int64_t k,
            cudaStream_t s) {
  dim3 grid(static_cast<unsigned>((rows + general::kTM - 1) / general::kTM + e),
            static_cast<unsigned>((n + general::kTN - 1) / general::kTN));
  general::grouped_plain_kernel<T><<<grid, general::kThreads, 0, s>>>(
      static_cast<T*>(c), static_cast<const T*>(a), static_cast<const T*>(b), offs, e, n, k);
}
}  // namespace
}  // namespace ksb

extern "C" ks_status_t ks_moe_grouped_gemm(void* c, const void* a, const void* b,
                                           const int32_t* expert_offsets, int num_experts, int64_t total_rows,
                                           int64_t n, int64_t k, ks_dtype_t dtype, ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_moe_grouped_gemm";
  KSB_REQUIRE_PTR(c);
  KSB_REQUIRE_PTR(a);
  KSB_REQUIRE_PTR(b);
  KSB_REQUIRE_PTR(expert_offsets);
  if (num_experts <= 0 || total_rows < 0 || n <= 0 || k <= 0)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_grouped_gemm: bad shape");
  if (total_rows == 0) return KS_SUCCESS;
  if (!is_float3(dtype) && !is_fp8(dtype))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_moe_grouped_gemm: unsupported dtype");
  if ((total_rows + general::kTM - 1) / general::kTM + num_experts > 2147483647LL ||
      (n + general::kTN - 1) / general::kTN > 65535LL)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_moe_grouped_gemm: tile grid exceeds CUDA grid limits");
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  switch (dtype) {
    case KS_DTYPE_F32: launch<float>(c, a, b, expert_offsets, num_experts, total_rows, n, k, s); break;
    case KS_DTYPE_F16: launch<__half>(c, a, b, expert_offsets, num_experts, total_rows, n, k, s); break;
    case KS_DTYPE_BF16: launch<__nv_bfloat16>(c, a, b, expert_offsets, num_experts, total_rows, n, k, s); break;
    case KS_DTYPE_F8E4M3: launch<__nv_fp8_e4m3>(c, a, b, expert_offsets, num_experts, total_rows, n, k, s); break;
    default: launch<__nv_fp8_e5m2>(c, a, b, expert_offsets, num_experts, total_rows, n, k, s); break;
  }
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}
