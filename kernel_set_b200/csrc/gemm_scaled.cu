// C ABI of the two 8-bit GEMMs with one scale per row of A and one per column of B:
// ks_gemm_fp8 (reference: kernels/src/gemm/gemm_fp8.cu, include/kernel_set/gemm.h:60-77)
// and ks_gemm_w8a8 (kernels/src/gemm/gemm_w8a8.cu, gemm.h:39-49).
//
//   C = (a_scale (x) b_scale) * (A @ B) [+ bias],  A [M,K], B [K,N] row-major,
//   a_scale [M] (per token) or [1] (per tensor), b_scale [N] (per channel) or [1].
//
// Both run on the tcgen05 mainloop of sm100_fp8_gemm.cu with the whole K range accumulated in
// tensor memory (fp32 for kind::f8f6f4, int32 for kind::i8) and one epilogue per tile that
// computes (acc * a_scale) * b_scale [+ bias] in the reference's order and rounds once. Shapes
// that kernel declines (K or N not a multiple of 16, unaligned operands) take the SIMT kernels
// below, which accumulate exactly as the reference's do (fp32 in ascending k; int32).
#include <string>

#include "common.cuh"
#include "gemm_general.cuh"
#include "kernel_set/gemm.h"
#include "sm100_fp8_gemm.cuh"

namespace ksb {
namespace {

template <typename F8, typename OutT>
__global__ void __launch_bounds__(general::kThreads)
fp8_scaled_general_kernel(OutT* __restrict__ c, const F8* __restrict__ a, const F8* __restrict__ b,
                          const float* __restrict__ a_scale, const float* __restrict__ b_scale, int64_t m, int64_t n,
                          int64_t k, int a_per_row, int b_per_col) {
  using namespace general;
  __shared__ Tile tile;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * kTM, n0 = static_cast<int64_t>(blockIdx.y) * kTN;
  const int tr = threadIdx.x >> 4, tc = threadIdx.x & 15;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < k; k0 += kTK) {
    stage_a<F8>(tile, a, k, row0, m, k0, k);
    stage_b_kn<F8>(tile, b, n, k0, k, n0, n);
    __syncthreads();
    mac_chunk(tile, tr, tc, acc);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gr = row0 + tr * 4 + i;
    if (gr >= m) continue;
    const float as = a_per_row ? a_scale[gr] : a_scale[0];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t gn = n0 + tc * 4 + j;
      if (gn >= n) continue;
      const float bs = b_per_col ? b_scale[gn] : b_scale[0];
      c[gr * n + gn] = from_f32<OutT>(__fmul_rn(__fmul_rn(acc[i][j], as), bs));
    }
  }
}

// int8 x int8 with exact int32 accumulation: 32 x 32 output tile, one element per thread.
template <typename OutT>
__global__ void __launch_bounds__(1024)
w8a8_general_kernel(OutT* __restrict__ c, const int8_t* __restrict__ a, const int8_t* __restrict__ b,
                    const float* __restrict__ a_scale, const float* __restrict__ b_scale,
                    const OutT* __restrict__ bias, int64_t m, int64_t n, int64_t k, int a_per_row, int b_per_col) {
  __shared__ int8_t sa[32][33], sb[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 32 + ty, col = static_cast<int64_t>(blockIdx.y) * 32 + tx;
  int acc = 0;
  for (int64_t k0 = 0; k0 < k; k0 += 32) {
    sa[ty][tx] = (row < m && k0 + tx < k) ? a[row * k + k0 + tx] : 0;
    const int64_t brow = k0 + ty;
    sb[ty][tx] = (brow < k && col < n) ? b[brow * n + col] : 0;
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 32; ++kk) acc += static_cast<int>(sa[ty][kk]) * static_cast<int>(sb[kk][tx]);
    __syncthreads();
  }
  if (row < m && col < n) {
    float v = __fmul_rn(__fmul_rn(static_cast<float>(acc), a_per_row ? a_scale[row] : a_scale[0]),
                        b_per_col ? b_scale[col] : b_scale[0]);
    if (bias != nullptr) v = __fadd_rn(v, to_f32<OutT>(bias[col]));
    c[row * n + col] = from_f32<OutT>(v);
  }
}

ks_status_t check_modes(const std::string& w, ks_quant_mode_t a_mode, ks_quant_mode_t b_mode) {
  if (a_mode != KS_QUANT_PER_TENSOR && a_mode != KS_QUANT_PER_TOKEN)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, w + ": a_mode must be per-tensor or per-token");
  if (b_mode != KS_QUANT_PER_TENSOR && b_mode != KS_QUANT_PER_CHANNEL)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, w + ": b_mode must be per-tensor or per-channel");
  return KS_SUCCESS;
}

}  // namespace
}  // namespace ksb

using namespace ksb;

extern "C" ks_status_t ks_gemm_fp8(void* out, const void* a_fp8, const void* b_fp8, const float* a_scale,
                                   const float* b_scale, int64_t m, int64_t n, int64_t k, ks_quant_mode_t a_mode,
                                   ks_quant_mode_t b_mode, ks_dtype_t fp8_dtype, ks_dtype_t out_dtype,
                                   ks_stream_t stream) {
  const char* where = "ks_gemm_fp8";
  KSB_REQUIRE_PTR(out);
  KSB_REQUIRE_PTR(a_fp8);
  KSB_REQUIRE_PTR(b_fp8);
  KSB_REQUIRE_PTR(a_scale);
  KSB_REQUIRE_PTR(b_scale);
  if (m <= 0 || n <= 0 || k <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_gemm_fp8: bad shape");
  ks_status_t st = check_modes(where, a_mode, b_mode);
  if (st != KS_SUCCESS) return st;
  if (!is_fp8(fp8_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_gemm_fp8: fp8_dtype must be e4m3 or e5m2");
  if (!is_float3(out_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_gemm_fp8: out_dtype must be f32/f16/bf16");
  st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  st = poll_kernel_fault(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const int apr = a_mode == KS_QUANT_PER_TOKEN, bpc = b_mode == KS_QUANT_PER_CHANNEL;
  sm100::Fp8GemmArgs g;
  g.where = where; g.out = out; g.a = a_fp8; g.b = b_fp8; g.a_scale = a_scale; g.b_scale = b_scale;
  g.m = m; g.n = n; g.k = k; g.nt = false; g.e5m2 = fp8_dtype == KS_DTYPE_F8E5M2; g.out_dtype = out_dtype;
  g.mode = 1; g.a_per_row = apr; g.b_per_col = bpc;
  if (sm100::fp8_blockwise_eligible(g)) return sm100::launch_fp8_blockwise(g, s);
  const int64_t tm = (m + general::kTM - 1) / general::kTM, tn = (n + general::kTN - 1) / general::kTN;
  if (tm > 2147483647LL || tn > 65535LL) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gemm_fp8: tile grid exceeds CUDA grid limits");
  dim3 grid(static_cast<unsigned>(tm), static_cast<unsigned>(tn));
#define KSB_F8(F8, OutT)                                                                                     \
  fp8_scaled_general_kernel<F8, OutT><<<grid, general::kThreads, 0, s>>>(                                   \
      static_cast<OutT*>(out), static_cast<const F8*>(a_fp8), static_cast<const F8*>(b_fp8), a_scale, b_scale, m, n, \
      k, apr, bpc)
  if (g.e5m2) {
    if (out_dtype == KS_DTYPE_F32) KSB_F8(__nv_fp8_e5m2, float);
    else if (out_dtype == KS_DTYPE_F16) KSB_F8(__nv_fp8_e5m2, __half);
    else KSB_F8(__nv_fp8_e5m2, __nv_bfloat16);
  } else {
    if (out_dtype == KS_DTYPE_F32) KSB_F8(__nv_fp8_e4m3, float);
    else if (out_dtype == KS_DTYPE_F16) KSB_F8(__nv_fp8_e4m3, __half);
    else KSB_F8(__nv_fp8_e4m3, __nv_bfloat16);
  }
#undef KSB_F8
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}

extern "C" ks_status_t ks_gemm_w8a8(void* c, const void* a_i8, const void* b_i8, const float* a_scale,
                                    const float* b_scale, const void* bias, int64_t m, int64_t n, int64_t k,
                                    ks_quant_mode_t a_mode, ks_quant_mode_t b_mode, ks_dtype_t out_dtype,
                                    ks_stream_t stream) {
  const char* where = "ks_gemm_w8a8";
  KSB_REQUIRE_PTR(c);
  KSB_REQUIRE_PTR(a_i8);
  KSB_REQUIRE_PTR(b_i8);
  KSB_REQUIRE_PTR(a_scale);
  KSB_REQUIRE_PTR(b_scale);
  if (m <= 0 || n <= 0 || k <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_gemm_w8a8: bad shape");
  ks_status_t st = check_modes(where, a_mode, b_mode);
  if (st != KS_SUCCESS) return st;
  if (!is_float3(out_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_gemm_w8a8: out_dtype must be f32/f16/bf16");
  st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  st = poll_kernel_fault(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const int apr = a_mode == KS_QUANT_PER_TOKEN, bpc = b_mode == KS_QUANT_PER_CHANNEL;
  sm100::Fp8GemmArgs g;
  g.where = where; g.out = c; g.a = a_i8; g.b = b_i8; g.a_scale = a_scale; g.b_scale = b_scale; g.bias = bias;
  g.m = m; g.n = n; g.k = k; g.nt = false; g.out_dtype = out_dtype;
  g.mode = 2; g.a_per_row = apr; g.b_per_col = bpc;
  if (sm100::fp8_blockwise_eligible(g)) return sm100::launch_fp8_blockwise(g, s);
  const int64_t tm = (m + 31) / 32, tn = (n + 31) / 32;
  if (tm > 2147483647LL || tn > 65535LL) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gemm_w8a8: tile grid exceeds CUDA grid limits");
  dim3 grid(static_cast<unsigned>(tm), static_cast<unsigned>(tn));
#define KSB_I8(OutT)                                                                                               \
  w8a8_general_kernel<OutT><<<grid, 1024, 0, s>>>(static_cast<OutT*>(c), static_cast<const int8_t*>(a_i8),         \
                                                  static_cast<const int8_t*>(b_i8), a_scale, b_scale,              \
                                                  static_cast<const OutT*>(bias), m, n, k, apr, bpc)
  if (out_dtype == KS_DTYPE_F32) KSB_I8(float);
  else if (out_dtype == KS_DTYPE_F16) KSB_I8(__half);
  else KSB_I8(__nv_bfloat16);
#undef KSB_I8
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}
