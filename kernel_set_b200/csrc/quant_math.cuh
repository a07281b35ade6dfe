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

// Two-wide fp32 arithmetic (one instruction, two IEEE round-to-nearest results).
struct F2 {
  uint64_t bits;
};
__device__ __forceinline__ F2 pack2(float lo, float hi) {
  F2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r.bits) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(F2 v, float* lo, float* hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(*lo), "=f"(*hi) : "l"(v.bits));
}
__device__ __forceinline__ F2 mul2(F2 a, F2 b) {
  F2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.bits) : "l"(a.bits), "l"(b.bits));
  return r;
}
__device__ __forceinline__ F2 fma2(F2 a, F2 b, F2 c) {
  F2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.bits) : "l"(a.bits), "l"(b.bits), "l"(c.bits));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Codes and scale of one 16-element segment of a 128-element group held by 8 consecutive
// lanes (all 32 lanes of the warp call this together; a lane without data passes zeros).
//
// Both divisions of the op are replaced by their correctly rounded equivalents:
// * amax / qmax: qmax is 1.75 * 2^8 or 1.75 * 2^15. With r = RN(1/qmax), q0 = RN(amax * r),
//   e = amax - q0 * qmax (exact in an FMA), RN(q0 + e * r) equals the IEEE quotient for every
//   finite amax whose quotient is not subnormal (checked over all 2^31 positive floats for
//   both constants); subnormal quotients are below the 1e-12 floor that replaces them anyway.
// * x / scale for the 16 elements: the same correction step with r = RN(1/scale) (Markstein:
//   q0 within one ulp, exact residual, one more rounding), two elements per instruction.
//   Valid while nothing overflows or goes subnormal on the way: groups with amax of 4.48e32
//   or more (scale >= 1e30), or infinite, take IEEE divisions.
template <bool E5M2>
__device__ __forceinline__ uint4 quant_segment_codes(const float (&v)[16], float qmax, float* sc_out) {
  float amax = max3(fabsf(v[0]), fabsf(v[1]), 0.f);
#pragma unroll
  for (int i = 2; i < 16; i += 2) amax = max3(amax, fabsf(v[i]), fabsf(v[i + 1]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  float q[16];
  float sc;
  if (amax < 4.48e32f) {
    const float rq = E5M2 ? (1.0f / 57344.0f) : (1.0f / 448.0f);   // RN(1/qmax), folded at compile time
    const float s0 = __fmul_rn(amax, rq);
    const float se = __fmaf_rn(-s0, qmax, amax);
    sc = fmaxf(__fmaf_rn(se, rq, s0), kScaleFloor);
    const float r = __frcp_rn(sc);
    // Written so that a zero keeps its sign, as x / sc does: with e' = q0 * sc - x the last
    // step q0 + e' * (-r) adds two zeros of x's sign when x is +-0 (x - q0 * sc would give
    // +0 for both, and -0.0 would lose its sign bit in the code).
    const F2 r2 = pack2(r, r);
    const F2 nr2 = pack2(-r, -r);
    const F2 sc2 = pack2(sc, sc);
    const F2 neg1 = pack2(-1.f, -1.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const F2 x2 = pack2(v[2 * i], v[2 * i + 1]);
      const F2 nx2 = mul2(x2, neg1);
      const F2 q0 = mul2(x2, r2);
      const F2 e = fma2(q0, sc2, nx2);     // q0 * sc - x, exact
      unpack2(fma2(e, nr2, q0), &q[2 * i], &q[2 * i + 1]);
    }
  } else {
    sc = fmaxf(__fdiv_rn(amax, qmax), kScaleFloor);
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = __fdiv_rn(v[i], sc);
  }
  *sc_out = sc;
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t p0 = cvt_pair<E5M2>(q[4 * i], q[4 * i + 1]);
    const uint32_t p1 = cvt_pair<E5M2>(q[4 * i + 2], q[4 * i + 3]);
    w[i] = __byte_perm(p0, p1, 0x5410);
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
