// C ABI of the FP8 block-scaled GEMMs: argument checks in the order and with
// the status codes of the reference (kernels/src/gemm/gemm_fp8_blockwise.cu:
// 218-302), then a choice between the tcgen05 kernel and the general kernel.
#include <cstdlib>

#include "common.cuh"
#include "gemm_general.cuh"
#include "kernel_set/gemm.h"
#include "kernel_set/moe.h"
#include "sm100_fp8_gemm.cuh"

namespace ksb {
namespace {

// KS_B200_FP8_PATH=general pins the general kernel, =tcgen05 refuses to fall
// back (UNSUPPORTED_SHAPE instead); KS_B200_FP8_BN=128|256 pins the tile width;
// KS_B200_FP8_SPLIT=0 switches the K-split of the last partial round off.
// They exist for tests and profiling; unset means "choose". Read once per process
// unless KS_B200_ENV_RELOAD is set (the test-suite flips them between calls).
struct EnvChoice {
  int path = 0;   // 0 choose, 1 general, 2 tcgen05
  int bn = 0;
  int split = -1; // -1 choose, 0 off, 1 on
};
EnvChoice read_env() {
  EnvChoice c;
  if (const char* v = std::getenv("KS_B200_FP8_PATH")) c.path = v[0] == 'g' ? 1 : (v[0] == 't' ? 2 : 0);
  if (const char* v = std::getenv("KS_B200_FP8_BN")) c.bn = std::atoi(v);
  if (const char* v = std::getenv("KS_B200_FP8_SPLIT")) c.split = std::atoi(v) != 0 ? 1 : 0;
  return c;
}
EnvChoice env_choice() {
  static const bool reload = std::getenv("KS_B200_ENV_RELOAD") != nullptr;
  static const EnvChoice cached = read_env();
  return reload ? read_env() : cached;
}

template <typename F8, typename OutT, bool NT, bool GROUPED>
void launch_general(const sm100::Fp8GemmArgs& a, cudaStream_t s) {
  const int64_t nkb = (a.k + a.block_k - 1) / a.block_k;
  const int64_t nnb = (a.n + a.block_n - 1) / a.block_n;
  const int64_t tiles_m = (a.m + general::kTM - 1) / general::kTM + (GROUPED ? a.num_experts : 0);
  dim3 grid(static_cast<unsigned>(tiles_m), static_cast<unsigned>((a.n + general::kTN - 1) / general::kTN));
  general::fp8_blockwise_kernel<F8, OutT, NT, GROUPED><<<grid, general::kThreads, 0, s>>>(
      static_cast<OutT*>(a.out), static_cast<const F8*>(a.a), static_cast<const F8*>(a.b), a.a_scale, a.b_scale,
      a.offsets, a.num_experts, a.m, a.n, a.k, a.block_n, a.block_k, nkb, nnb);
}

template <typename F8, bool NT, bool GROUPED>
void launch_general_out(const sm100::Fp8GemmArgs& a, cudaStream_t s) {
  if (a.out_dtype == KS_DTYPE_F32) launch_general<F8, float, NT, GROUPED>(a, s);
  else if (a.out_dtype == KS_DTYPE_F16) launch_general<F8, __half, NT, GROUPED>(a, s);
  else launch_general<F8, __nv_bfloat16, NT, GROUPED>(a, s);
}

template <bool GROUPED>
void launch_general_any(const sm100::Fp8GemmArgs& a, cudaStream_t s) {
  if (a.e5m2) {
    if (a.nt) launch_general_out<__nv_fp8_e5m2, true, GROUPED>(a, s);
    else launch_general_out<__nv_fp8_e5m2, false, GROUPED>(a, s);
  } else {
    if (a.nt) launch_general_out<__nv_fp8_e4m3, true, GROUPED>(a, s);
    else launch_general_out<__nv_fp8_e4m3, false, GROUPED>(a, s);
  }
}

ks_status_t run(sm100::Fp8GemmArgs& a, ks_stream_t stream) {
  ks_status_t st = require_sm100(a.where);
  if (st != KS_SUCCESS) return st;
  st = poll_kernel_fault(a.where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const EnvChoice env = env_choice();
  const int path = env.path;
  a.force_bn = env.bn;
  a.force_split = env.split;
  if (path != 1 && sm100::fp8_blockwise_eligible(a)) return sm100::launch_fp8_blockwise(a, s);
  if (path == 2)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, std::string(a.where) + ": shape not eligible for the tcgen05 kernel");
  const int64_t tiles_m = (a.m + general::kTM - 1) / general::kTM + a.num_experts;
  const int64_t tiles_n = (a.n + general::kTN - 1) / general::kTN;
  if (tiles_m > 2147483647LL || tiles_n > 65535LL)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, std::string(a.where) + ": tile grid exceeds CUDA grid limits");
  if (a.offsets != nullptr) launch_general_any<true>(a, s);
  else launch_general_any<false>(a, s);
  return cuda_status(cudaGetLastError(), a.where);
}

ks_status_t check_common(const char* where, const void* out, const void* a, const void* b, const float* as,
                         const float* bs, int64_t m, int64_t n, int64_t k, int block_n, int block_k,
                         ks_dtype_t fp8_dtype, ks_dtype_t out_dtype, bool m_may_be_zero) {
  if (out == nullptr) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "null arg: out");
  if (a == nullptr) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "null arg: a_fp8");
  if (b == nullptr) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "null arg: b_fp8");
  if (as == nullptr) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "null arg: a_scale");
  if (bs == nullptr) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "null arg: b_scale");
  if ((m_may_be_zero ? m < 0 : m <= 0) || n <= 0 || k <= 0)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, std::string(where) + ": bad shape");
  if (block_n <= 0 || block_k <= 0)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, std::string(where) + ": block_n/block_k must be > 0");
  constexpr int64_t kMax = INT64_MAX;
  if ((m > 0 && (m > kMax / k || m > kMax / n)) || k > kMax / n)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, std::string(where) + ": M*K / K*N / M*N exceeds int64 range");
  if (!is_fp8(fp8_dtype))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, std::string(where) + ": fp8_dtype must be e4m3 or e5m2");
  if (!is_float3(out_dtype))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, std::string(where) + ": out_dtype must be f32/f16/bf16");
  return KS_SUCCESS;
}

}  // namespace
}  // namespace ksb

extern "C" {

ks_status_t ks_gemm_fp8_blockwise(void* out, const void* a_fp8, const void* b_fp8, const float* a_scale,
                                  const float* b_scale, int64_t m, int64_t n, int64_t k, int block_n,
                                  int block_k, ks_dtype_t fp8_dtype, ks_dtype_t out_dtype,
                                  ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_gemm_fp8_blockwise";
  ks_status_t st = check_common(where, out, a_fp8, b_fp8, a_scale, b_scale, m, n, k, block_n, block_k, fp8_dtype,
                                out_dtype, false);
  if (st != KS_SUCCESS) return st;
  sm100::Fp8GemmArgs a;
  a.where = where; a.out = out; a.a = a_fp8; a.b = b_fp8; a.a_scale = a_scale; a.b_scale = b_scale;
  a.m = m; a.n = n; a.k = k; a.block_n = block_n; a.block_k = block_k; a.nt = false;
  a.e5m2 = fp8_dtype == KS_DTYPE_F8E5M2; a.out_dtype = out_dtype;
  return run(a, stream);
}

ks_status_t ks_gemm_fp8_blockwise_nt(void* out, const void* a_fp8, const void* b_fp8, const float* a_scale,
                                     const float* b_scale, int64_t m, int64_t n, int64_t k, int block_n,
                                     int block_k, ks_dtype_t fp8_dtype, ks_dtype_t out_dtype,
                                     ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_gemm_fp8_blockwise_nt";
  ks_status_t st = check_common(where, out, a_fp8, b_fp8, a_scale, b_scale, m, n, k, block_n, block_k, fp8_dtype,
                                out_dtype, false);
  if (st != KS_SUCCESS) return st;
  sm100::Fp8GemmArgs a;
  a.where = where; a.out = out; a.a = a_fp8; a.b = b_fp8; a.a_scale = a_scale; a.b_scale = b_scale;
  a.m = m; a.n = n; a.k = k; a.block_n = block_n; a.block_k = block_k; a.nt = true;
  a.e5m2 = fp8_dtype == KS_DTYPE_F8E5M2; a.out_dtype = out_dtype;
  return run(a, stream);
}

ks_status_t ks_moe_grouped_gemm_fp8_blockwise(void* out, const void* a_fp8, const void* b_fp8,
                                              const float* a_scale, const float* b_scale,
                                              const int32_t* expert_offsets, int num_experts,
                                              int64_t total_rows, int64_t n, int64_t k, int block_n,
                                              int block_k, int b_layout, ks_dtype_t fp8_dtype,
                                              ks_dtype_t out_dtype, ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_moe_grouped_gemm_fp8_blockwise";
  if (expert_offsets == nullptr) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "null arg: expert_offsets");
  if (num_experts <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, std::string(where) + ": bad shape");
  if (b_layout != 0 && b_layout != 1)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, std::string(where) + ": b_layout must be 0 ([E,K,N]) or 1 ([E,N,K])");
  ks_status_t st = check_common(where, out, a_fp8, b_fp8, a_scale, b_scale, total_rows, n, k, block_n, block_k,
                                fp8_dtype, out_dtype, true);
  if (st != KS_SUCCESS) return st;
  if (total_rows == 0) return KS_SUCCESS;
  sm100::Fp8GemmArgs a;
  a.where = where; a.out = out; a.a = a_fp8; a.b = b_fp8; a.a_scale = a_scale; a.b_scale = b_scale;
  a.offsets = expert_offsets; a.num_experts = num_experts;
  a.m = total_rows; a.n = n; a.k = k; a.block_n = block_n; a.block_k = block_k; a.nt = b_layout == 1;
  a.e5m2 = fp8_dtype == KS_DTYPE_F8E5M2; a.out_dtype = out_dtype;
  return run(a, stream);
}

ks_status_t ks_moe_grouped_gemm_fp8_blockwise_masked(void* out, const void* a_fp8, const void* b_fp8,
                                                     const float* a_scale, const float* b_scale,
                                                     const int32_t* masked_m, int num_experts, int64_t max_m,
                                                     int64_t n, int64_t k, int block_n, int block_k, int b_layout,
                                                     ks_dtype_t fp8_dtype, ks_dtype_t out_dtype,
                                                     ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_moe_grouped_gemm_fp8_blockwise_masked";
  if (masked_m == nullptr) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "null arg: masked_m");
  if (num_experts <= 0 || max_m <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, std::string(where) + ": bad shape");
  if (b_layout != 0 && b_layout != 1)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, std::string(where) + ": b_layout must be 0 ([E,K,N]) or 1 ([E,N,K])");
  if (max_m > INT32_MAX / num_experts)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, std::string(where) + ": num_experts * max_m exceeds int32 range");
  ks_status_t st = check_common(where, out, a_fp8, b_fp8, a_scale, b_scale, max_m * num_experts, n, k, block_n,
                                block_k, fp8_dtype, out_dtype, false);
  if (st != KS_SUCCESS) return st;
  st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  st = poll_kernel_fault(where);
  if (st != KS_SUCCESS) return st;
  sm100::Fp8GemmArgs a;
  a.where = where; a.out = out; a.a = a_fp8; a.b = b_fp8; a.a_scale = a_scale; a.b_scale = b_scale;
  a.masked_m = masked_m; a.max_m = max_m; a.num_experts = num_experts;
  a.m = max_m * num_experts; a.n = n; a.k = k; a.block_n = block_n; a.block_k = block_k; a.nt = b_layout == 1;
  a.e5m2 = fp8_dtype == KS_DTYPE_F8E5M2; a.out_dtype = out_dtype;
  const EnvChoice env = env_choice();
  a.force_bn = env.bn;
  // the row counts live on the device (that is the point of the layout: the launch does not
  // depend on them), so only the tcgen05 kernel, which reads them itself, serves this entry
  if (!sm100::fp8_blockwise_eligible(a))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE,
             std::string(where) + ": needs 128 x 128 scale blocks, K (and N for [E,K,N]) multiples of 16, "
                                  "16-byte aligned operands and at most 1024 experts");
  return sm100::launch_fp8_blockwise(a, as_stream(stream));
}

ks_status_t ks_gemm_fp8_blockwise_colscale(void* out, const void* a_fp8, const void* b_fp8, const float* a_scale_t,
                                           int64_t a_scale_ld, const float* b_scale, int64_t m, int64_t n,
                                           int64_t k, int b_layout, ks_dtype_t fp8_dtype, ks_dtype_t out_dtype,
                                           ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_gemm_fp8_blockwise_colscale";
  if (b_layout != 0 && b_layout != 1)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, std::string(where) + ": b_layout must be 0 ([K,N]) or 1 ([N,K])");
  ks_status_t st = check_common(where, out, a_fp8, b_fp8, a_scale_t, b_scale, m, n, k, 128, 128, fp8_dtype, out_dtype,
                                false);
  if (st != KS_SUCCESS) return st;
  if (a_scale_ld < m) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, std::string(where) + ": a_scale_ld must be at least m");
  st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  st = poll_kernel_fault(where);
  if (st != KS_SUCCESS) return st;
  sm100::Fp8GemmArgs a;
  a.where = where; a.out = out; a.a = a_fp8; a.b = b_fp8; a.a_scale = a_scale_t; a.a_scale_ld = a_scale_ld;
  a.b_scale = b_scale; a.m = m; a.n = n; a.k = k; a.nt = b_layout == 1;
  a.e5m2 = fp8_dtype == KS_DTYPE_F8E5M2; a.out_dtype = out_dtype;
  const EnvChoice env = env_choice();
  a.force_bn = env.bn;
  a.force_split = env.split;
  if (!sm100::fp8_blockwise_eligible(a))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE,
             std::string(where) + ": needs K (and N for [K,N]) multiples of 16 and 16-byte aligned operands");
  return sm100::launch_fp8_blockwise(a, as_stream(stream));
}

ks_status_t ks_gemm_fp8_blockwise_scatter(void* const* out_parts, int num_parts, int64_t rows_per_part,
                                          const void* a_fp8, const void* b_fp8, const float* a_scale,
                                          const float* b_scale, int64_t m, int64_t n, int64_t k, int b_layout,
                                          ks_dtype_t fp8_dtype, ks_dtype_t out_dtype, ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_gemm_fp8_blockwise_scatter";
  KSB_REQUIRE_PTR(out_parts);
  if (num_parts < 1 || num_parts > 8)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, std::string(where) + ": between 1 and 8 output parts");
  for (int i = 0; i < num_parts; ++i)
    if (out_parts[i] == nullptr) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, std::string(where) + ": null output part");
  if (b_layout != 0 && b_layout != 1)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, std::string(where) + ": b_layout must be 0 ([K,N]) or 1 ([N,K])");
  ks_status_t st = check_common(where, out_parts[0], a_fp8, b_fp8, a_scale, b_scale, m, n, k, 128, 128, fp8_dtype,
                                out_dtype, false);
  if (st != KS_SUCCESS) return st;
  if (rows_per_part <= 0 || rows_per_part % 128 != 0 || rows_per_part * num_parts != m)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE,
             std::string(where) + ": rows_per_part must be a multiple of 128 and num_parts * rows_per_part = m");
  st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  st = poll_kernel_fault(where);
  if (st != KS_SUCCESS) return st;
  sm100::Fp8GemmArgs a;
  a.where = where; a.out = nullptr; a.a = a_fp8; a.b = b_fp8; a.a_scale = a_scale;
  a.b_scale = b_scale; a.m = m; a.n = n; a.k = k; a.nt = b_layout == 1;
  a.e5m2 = fp8_dtype == KS_DTYPE_F8E5M2; a.out_dtype = out_dtype;
  a.out_parts = out_parts; a.num_out_parts = num_parts; a.rows_per_part = rows_per_part;
  const EnvChoice env = env_choice();
  a.force_bn = env.bn;
  a.force_split = 0;
  if (!sm100::fp8_blockwise_eligible(a))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE,
             std::string(where) + ": needs K (and N for [K,N]) multiples of 16 and 16-byte aligned operands");
  return sm100::launch_fp8_blockwise(a, as_stream(stream));
}

}  // extern "C"
