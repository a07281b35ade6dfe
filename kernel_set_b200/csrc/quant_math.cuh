// Arithmetic of the 1 x 128 FP8 group quantizer, shared by the plain quantizer and the
// kernels that fuse it into their producer (row gather, SwiGLU): 16-element loads as
// fp32, the group maximum over an 8-lane segment, the scale, and exact quotients.
// Every user produces bit-identical codes and scales for identical inputs.
//
// Reference arithmetic: kernels/src/quant/quant_fp8_group.cu:38-107 with the
// division of the reference's torch statement (benchmarks/bench.py:1444-1457).
#pragma once

#include "common.cuh"

namespace ksb {
namespace quantmath {

constexpr float kScaleFloor = 1e-12f;

template <typename T> struct Vec16;  // 16 elements of T as fp32

template <> struct Vec16<__nv_bfloat16> {
  __device__ static void load(const __nv_bfloat16* p, float (&v)[16]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
template <> struct Vec16<__half> {
  __device__ static void load(const __half* p, float (&v)[16]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};
template <> struct Vec16<float> {
  __device__ static void load(const float* p, float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(p) + i);
      v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
    }
  }
};

// The same 16 elements as raw 16-byte words, so that a load can be issued long before its
// conversion: Raw16<T>::load now, Raw16<T>::unpack later.
template <typename T> struct Raw16 {
  uint4 a, b;
  __device__ static Raw16 load(const T* p) {
    Raw16 r;
    r.a = __ldg(reinterpret_cast<const uint4*>(p));
    r.b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    return r;
  }
  __device__ static Raw16 zero() {
    Raw16 r;
    r.a = make_uint4(0u, 0u, 0u, 0u);
    r.b = r.a;
    return r;
  }
  __device__ void unpack(float (&v)[16]) const {
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if constexpr (sizeof(T) == 2 && !__is_same(T, __half)) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
      }
    }
  }
};
template <> struct Raw16<float> {
  float4 q[4];
  __device__ static Raw16 load(const float* p) {
    Raw16 r;
#pragma unroll
    for (int i = 0; i < 4; ++i) r.q[i] = __ldg(reinterpret_cast<const float4*>(p) + i);
    return r;
  }
  __device__ static Raw16 zero() {
    Raw16 r;
#pragma unroll
    for (int i = 0; i < 4; ++i) r.q[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    return r;
  }
  __device__ void unpack(float (&v)[16]) const {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[4 * i] = q[i].x; v[4 * i + 1] = q[i].y; v[4 * i + 2] = q[i].z; v[4 * i + 3] = q[i].w;
    }
  }
};

// Two fp32 -> two fp8 codes (low byte = first value), RNE, saturating.
template <bool E5M2>
__device__ __forceinline__ uint32_t cvt_pair(float lo, float hi) {
  return __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
}
template <bool E5M2>
__device__ __forceinline__ uint8_t cvt_one(float v) {
  return __nv_cvt_float_to_fp8(v, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
}

// Codes and scale of one 16-element segment of a 128-element group held by 8 consecutive
// lanes (all 32 lanes of the warp call this together; a lane without data passes zeros).
template <bool E5M2>
__device__ __forceinline__ uint4 quant_segment_codes(const float (&v)[16], float qmax, float* sc_out) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  const float sc = fmaxf(__fdiv_rn(amax, qmax), kScaleFloor);
  *sc_out = sc;
  // x / sc, correctly rounded, without sixteen IEEE divisions: with r = RN(1/sc) and
  // q0 = RN(x*r) (within one ulp of the quotient), the residual e = x - q0*sc is exact in
  // an FMA and RN(q0 + e*r) is the correctly rounded quotient (Markstein's correction
  // step, the tail of the division routine itself). Valid while nothing overflows or
  // goes subnormal on the way; scales outside [1e-30, 1e30] take the division.
  float q[16];
  if (sc > 1e-30f && sc < 1e30f) {
    const float r = __frcp_rn(sc);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float q0 = __fmul_rn(v[i], r);
      const float e = __fmaf_rn(-q0, sc, v[i]);
      q[i] = __fmaf_rn(e, r, q0);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = __fdiv_rn(v[i], sc);
  }
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t p0 = cvt_pair<E5M2>(q[4 * i], q[4 * i + 1]);
    const uint32_t p1 = cvt_pair<E5M2>(q[4 * i + 2], q[4 * i + 3]);
    w[i] = (p0 & 0xffffu) | (p1 << 16);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// One 16-element segment of a dense [rows, cols] matrix (cols % 128 == 0): segment `seg`
// covers elements [16 seg, 16 seg + 16); its group's scale goes to scale[seg / 8].
template <typename T, bool E5M2>
__device__ __forceinline__ void quant_segment(uint8_t* __restrict__ out, float* __restrict__ scale, const float (&v)[16],
                                              int64_t seg, bool live, float qmax) {
  float sc;
  const uint4 codes = quant_segment_codes<E5M2>(v, qmax, &sc);
  if (!live) return;
  if ((threadIdx.x & 7) == 0) scale[seg >> 3] = sc;
  __stcs(reinterpret_cast<uint4*>(out + seg * 16), codes);
}

}  // namespace quantmath
}  // namespace ksb
