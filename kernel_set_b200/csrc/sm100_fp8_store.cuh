// Row-segment stores shared by the FP8 GEMM kernels: 16 consecutive outputs of
// one row, rounded once from fp32 to the output type.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace ksb {
namespace sm100 {

template <typename OutT>
__device__ __forceinline__ void store_16(OutT* dst, const float* v, bool vec, int valid_cols);

// Stores 16 consecutive outputs of one row; `valid_cols` of them exist.
template <>
__device__ __forceinline__ void store_16<float>(float* dst, const float* v, bool vec, int valid_cols) {
  if (vec && valid_cols >= 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < valid_cols) dst[i] = v[i];
  }
}
template <>
__device__ __forceinline__ void store_16<__nv_bfloat16>(__nv_bfloat16* dst, const float* v, bool vec,
                                                        int valid_cols) {
  if (vec && valid_cols >= 16) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < valid_cols) dst[i] = __float2bfloat16_rn(v[i]);
  }
}
template <>
__device__ __forceinline__ void store_16<__half>(__half* dst, const float* v, bool vec, int valid_cols) {
  if (vec && valid_cols >= 16) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < valid_cols) dst[i] = __float2half_rn(v[i]);
  }
}

// Packs the 16 bytes that follow output column `c` (a multiple of 16 / sizeof(OutT))
// of a row held as float2 pairs: 8 outputs of a 2-byte type, 4 floats.
template <typename OutT>
__device__ __forceinline__ uint4 pack_16_bytes(const float2* acc, int c);
template <>
__device__ __forceinline__ uint4 pack_16_bytes<float>(const float2* acc, int c) {
  const float2 a = acc[c / 2], b = acc[c / 2 + 1];
  return make_uint4(__float_as_uint(a.x), __float_as_uint(a.y), __float_as_uint(b.x), __float_as_uint(b.y));
}
template <>
__device__ __forceinline__ uint4 pack_16_bytes<__nv_bfloat16>(const float2* acc, int c) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(acc[c / 2 + i].x, acc[c / 2 + i].y);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ uint4 pack_16_bytes<__half>(const float2* acc, int c) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(acc[c / 2 + i].x, acc[c / 2 + i].y);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

}  // namespace sm100
}  // namespace ksb
