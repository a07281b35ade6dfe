// C ABI of the unscaled grouped GEMM (reference: kernels/src/moe/
// moe_grouped_gemm.cu:136-198). One launch, no allocation, no host sync: each
// block finds its (expert, row tile) from the offsets itself, where the
// reference builds a schedule with a one-thread kernel into a buffer it
// allocates and frees around a stream synchronisation.
//
// f16 / bf16 problems with 16-byte row pitches run on the tcgen05 mainloop of the FP8 GEMM
// (its 16-bit mode: kind::f16, the whole K range accumulated in tensor memory); the
// environment variable KS_B200_GROUPED_PATH=general pins the SIMT kernel (tests).
#include <cstdlib>

#include "common.cuh"
#include "gemm_general.cuh"
#include "kernel_set/moe.h"
#include "sm100_fp8_gemm.cuh"

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
  if (dtype == KS_DTYPE_F16 || dtype == KS_DTYPE_BF16) {
    static const bool reload = std::getenv("KS_B200_ENV_RELOAD") != nullptr;
    static const bool general_cached = [] { const char* v = std::getenv("KS_B200_GROUPED_PATH"); return v && v[0] == 'g'; }();
    bool pin_general = general_cached;
    if (reload) { const char* v = std::getenv("KS_B200_GROUPED_PATH"); pin_general = v && v[0] == 'g'; }
    sm100::Fp8GemmArgs g;
    g.where = where; g.out = c; g.a = a; g.b = b; g.offsets = expert_offsets; g.num_experts = num_experts;
    g.m = total_rows; g.n = n; g.k = k; g.nt = false; g.out_dtype = dtype; g.mode = 3;
    if (!pin_general && sm100::fp8_blockwise_eligible(g)) {
      st = poll_kernel_fault(where);
      if (st != KS_SUCCESS) return st;
      return sm100::launch_fp8_blockwise(g, s);
    }
  }
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
