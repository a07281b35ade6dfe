// RMSNorm, alone and fused with the 1 x 128 FP8 group quantizer that usually follows it in
// front of a block-scaled GEMM.
//
// Reference: ks_rms_norm (include/kernel_set/norm.h:16-19, kernels/src/norm/rms_norm.cu:19-42).
// The arithmetic follows the reference's torch statement of the op (benchmarks/bench.py:
// 877-879): the normalised value x * rsqrt(mean(x^2) + eps) is rounded to the storage type,
// then multiplied by the weight and rounded again (the reference kernel keeps the product in
// fp32 and rounds once; the two differ by at most one unit in the last place). The
// fused form rounds the normalised row to the input type exactly as the plain kernel writes
// it and quantizes those values exactly as ks_quantize_fp8_group reads them, so its codes and
// scales are bit-identical to the two calls run one after the other, without the 16-bit
// intermediate ever reaching memory (the row is read once and kept in registers).
//
// One CTA of 128 threads per row; a thread owns the 16-element segments t, t + 128, ... of the
// row (up to four: rows of at most 8192 elements), so eight consecutive lanes hold the eight
// segments of a quantisation group, the arrangement quant_segment_codes expects.
#include <string>

#include "common.cuh"
#include "kernel_set/norm.h"
#include "quant_math.cuh"

namespace ksb {
namespace {

using namespace quantmath;

constexpr int kNormThreads = 128;
constexpr int kMaxSegsPerThread = 4;

__device__ __forceinline__ float block_sum_128(float v) {
  __shared__ float red[kNormThreads / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return (red[0] + red[1]) + (red[2] + red[3]);
}

// QUANT == false: out is T [rows, cols]. QUANT == true: out is fp8 [rows, cols], scale [rows, cols / 128].
template <typename T, bool QUANT, bool E5M2>
__global__ void __launch_bounds__(kNormThreads)
rms_norm_rows_kernel(void* __restrict__ out, float* __restrict__ scale, const T* __restrict__ in,
                     const T* __restrict__ weight, int64_t cols, float eps, float qmax) {
  const int64_t row = blockIdx.x;
  const int segs = static_cast<int>(cols / 16);
  const T* x = in + row * cols;
  Raw16<T> raw[kMaxSegsPerThread];
  float sumsq = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxSegsPerThread; ++i) {
    const int seg = threadIdx.x + i * kNormThreads;
    if (seg < segs) {
      raw[i] = Raw16<T>::load(x + seg * 16);
      float v[16];
      raw[i].unpack(v);
#pragma unroll
      for (int j = 0; j < 16; ++j) sumsq = fmaf(v[j], v[j], sumsq);
    } else {
      raw[i] = Raw16<T>::zero();
    }
  }
  sumsq = block_sum_128(sumsq);
  const float inv_rms = rsqrtf(sumsq / static_cast<float>(cols) + eps);
#pragma unroll
  for (int i = 0; i < kMaxSegsPerThread; ++i) {
    if (i * kNormThreads >= segs) break;   // uniform over the CTA
    const int seg = threadIdx.x + i * kNormThreads;
    const bool live = seg < segs;
    float v[16], w[16];
    raw[i].unpack(v);
    if (live) {
      Raw16<T>::load(weight + seg * 16).unpack(w);
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) w[j] = 0.f;
    }
    T y[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) y[j] = from_f32<T>(to_f32<T>(from_f32<T>(v[j] * inv_rms)) * w[j]);
    if constexpr (QUANT) {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = to_f32<T>(y[j]);
      float sc;
      const uint4 codes = quant_segment_codes<E5M2>(v, qmax, &sc);
      if (live) {
        if ((threadIdx.x & 7) == 0) scale[row * (cols / 128) + (seg >> 3)] = sc;
        __stcs(reinterpret_cast<uint4*>(static_cast<uint8_t*>(out) + row * cols + seg * 16), codes);
      }
    } else if (live) {
      uint4* dst = reinterpret_cast<uint4*>(static_cast<T*>(out) + row * cols + seg * 16);
      const uint4* src = reinterpret_cast<const uint4*>(y);
#pragma unroll
      for (int q = 0; q < static_cast<int>(sizeof(T)) * 16 / 16; ++q) dst[q] = src[q];
    }
  }
}

// Any width / alignment: one CTA per row, the row read twice.
template <typename T>
__global__ void __launch_bounds__(kNormThreads)
rms_norm_any_kernel(T* __restrict__ out, const T* __restrict__ in, const T* __restrict__ weight, int64_t cols,
                    float eps) {
  const int64_t row = blockIdx.x;
  const T* x = in + row * cols;
  float sumsq = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += kNormThreads) {
    const float v = to_f32<T>(x[c]);
    sumsq = fmaf(v, v, sumsq);
  }
  sumsq = block_sum_128(sumsq);
  const float inv_rms = rsqrtf(sumsq / static_cast<float>(cols) + eps);
  for (int64_t c = threadIdx.x; c < cols; c += kNormThreads)
    out[row * cols + c] = from_f32<T>(to_f32<T>(from_f32<T>(to_f32<T>(x[c]) * inv_rms)) * to_f32<T>(weight[c]));
}

bool rows_kernel_fits(int64_t cols, const void* a, const void* b, const void* c) {
  return cols % 128 == 0 && cols <= 16 * kNormThreads * kMaxSegsPerThread && aligned16(a) && aligned16(b) &&
         aligned16(c);
}

}  // namespace
}  // namespace ksb

using namespace ksb;

extern "C" ks_status_t ks_rms_norm(void* out, const void* input, const void* weight, int64_t rows, int64_t cols,
                                   float eps, ks_dtype_t dtype, ks_stream_t stream) {
  const char* where = "ks_rms_norm";
  KSB_REQUIRE_PTR(out);
  KSB_REQUIRE_PTR(input);
  KSB_REQUIRE_PTR(weight);
  if (rows < 0 || cols <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_rms_norm: bad shape");
  if (!is_float3(dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_rms_norm: unsupported dtype");
  if (rows == 0) return KS_SUCCESS;
  if (rows > 2147483647LL) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_rms_norm: grid exceeds CUDA grid limits");
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const unsigned grid = static_cast<unsigned>(rows);
  const bool fast = rows_kernel_fits(cols, out, input, weight);
#define KSB_RN(T)                                                                                               \
  do {                                                                                                          \
    if (fast) rms_norm_rows_kernel<T, false, false><<<grid, kNormThreads, 0, s>>>(                              \
        out, nullptr, static_cast<const T*>(input), static_cast<const T*>(weight), cols, eps, 0.f);             \
    else rms_norm_any_kernel<T><<<grid, kNormThreads, 0, s>>>(static_cast<T*>(out), static_cast<const T*>(input), \
                                                              static_cast<const T*>(weight), cols, eps);        \
  } while (0)
  if (dtype == KS_DTYPE_F32) KSB_RN(float);
  else if (dtype == KS_DTYPE_F16) KSB_RN(__half);
  else KSB_RN(__nv_bfloat16);
#undef KSB_RN
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}

extern "C" ks_status_t ks_rms_norm_quant_fp8(void* out_fp8, float* out_scale, const void* input, const void* weight,
                                             int64_t rows, int64_t cols, float eps, ks_dtype_t in_dtype,
                                             ks_dtype_t fp8_dtype, ks_stream_t stream) {
  const char* where = "ks_rms_norm_quant_fp8";
  KSB_REQUIRE_PTR(out_fp8);
  KSB_REQUIRE_PTR(out_scale);
  KSB_REQUIRE_PTR(input);
  KSB_REQUIRE_PTR(weight);
  if (rows < 0 || cols <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_rms_norm_quant_fp8: bad shape");
  if (!rows_kernel_fits(cols, out_fp8, input, weight))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE,
             "ks_rms_norm_quant_fp8: cols must be a multiple of 128, at most 8192, and the buffers 16-byte aligned");
  if (!is_fp8(fp8_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_rms_norm_quant_fp8: fp8_dtype must be e4m3 or e5m2");
  if (in_dtype != KS_DTYPE_F16 && in_dtype != KS_DTYPE_BF16)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_rms_norm_quant_fp8: input must be f16 or bf16");
  if (rows == 0) return KS_SUCCESS;
  if (rows > 2147483647LL) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_rms_norm_quant_fp8: grid exceeds CUDA grid limits");
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const unsigned grid = static_cast<unsigned>(rows);
  const bool e5 = fp8_dtype == KS_DTYPE_F8E5M2;
#define KSB_RQ(T)                                                                                                 \
  do {                                                                                                            \
    if (e5) rms_norm_rows_kernel<T, true, true><<<grid, kNormThreads, 0, s>>>(                                    \
        out_fp8, out_scale, static_cast<const T*>(input), static_cast<const T*>(weight), cols, eps, 57344.0f);    \
    else rms_norm_rows_kernel<T, true, false><<<grid, kNormThreads, 0, s>>>(                                      \
        out_fp8, out_scale, static_cast<const T*>(input), static_cast<const T*>(weight), cols, eps, 448.0f);      \
  } while (0)
  if (in_dtype == KS_DTYPE_F16) KSB_RQ(__half);
  else KSB_RQ(__nv_bfloat16);
#undef KSB_RQ
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}
