// Per-token-group dynamic FP8 quantizer: 1 x group_size strips of a row-major
// matrix share one fp32 scale.
//
// Reference: ks_quantize_fp8_group, kernels/src/quant/quant_fp8_group.cu:133-214
// (kernels :38-107, constants quant_common.cuh:25-33). The arithmetic follows
// the reference's torch statement of the op (benchmarks/bench.py:1444-1457 and
// 2339-2344): scale = max(amax / qmax, 1e-12) and out = fp8(x / scale), both
// with IEEE fp32 division. (The reference CUDA kernel multiplies by 1/scale
// instead, which differs from its own torch statement in about one code in
// two thousand.)
//
// Layout of the fast kernel (group_size == 128, cols % 128 == 0, 16-byte
// aligned buffers): a lane owns 16 consecutive elements (two 16-byte loads for
// 16-bit inputs), 8 lanes own one group, a warp owns 4 groups. The group
// maximum is a 3-step xor shuffle inside the 8-lane segment; the 16 fp8 codes
// leave as one 16-byte streaming store. Algorithmic bytes per element: in_bytes + 1,
// plus 4/128 for the scale.
#include "common.cuh"
#include "kernel_set/quant.h"

#ifndef KSB_QUANT_SEGS
#define KSB_QUANT_SEGS 1
#endif

namespace ksb {
namespace {

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

// Two fp32 -> two fp8 codes (low byte = first value), RNE, saturating.
template <bool E5M2>
__device__ __forceinline__ uint32_t cvt_pair(float lo, float hi) {
  return __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
}
template <bool E5M2>
__device__ __forceinline__ uint8_t cvt_one(float v) {
  return __nv_cvt_float_to_fp8(v, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
}

// One 16-element segment of a group: maximum over the 8-lane segment, scale, codes.
template <typename T, bool E5M2>
__device__ __forceinline__ void quant_segment(uint8_t* __restrict__ out, float* __restrict__ scale, const float (&v)[16],
                                              int64_t seg, bool live, float qmax) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  // All 32 lanes take part in the shuffles; a dead tail segment carries 0.
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  if (!live) return;
  const float sc = fmaxf(__fdiv_rn(amax, qmax), kScaleFloor);
  if ((threadIdx.x & 7) == 0) scale[seg >> 3] = sc;
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
  __stcs(reinterpret_cast<uint4*>(out + seg * 16), make_uint4(w[0], w[1], w[2], w[3]));
}

// A thread owns kSegs segments, all loaded before the first is used. Measured on B200 for
// [4096, 7168] bf16: 22 us with one segment per thread, 25 us with two, 35 us with four
// (fewer resident threads cost more than the extra loads in flight gain), so one it is.
template <typename T, bool E5M2, int kSegs>
__global__ void __launch_bounds__(256)
quant_group128_kernel(uint8_t* __restrict__ out, float* __restrict__ scale,
                      const T* __restrict__ in, int64_t total_groups, float qmax) {
  // a block owns kSegs consecutive runs of 256 segments (contiguous in memory)
  const int64_t stride = blockDim.x;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.x * kSegs + threadIdx.x;
  float v[kSegs][16];
  bool live[kSegs];
#pragma unroll
  for (int s = 0; s < kSegs; ++s) {
    const int64_t seg = first + s * stride;
    live[s] = (seg >> 3) < total_groups;
    if (live[s]) {
      Vec16<T>::load(in + seg * 16, v[s]);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[s][i] = 0.f;
    }
  }
#pragma unroll
  for (int s = 0; s < kSegs; ++s) quant_segment<T, E5M2>(out, scale, v[s], first + s * stride, live[s], qmax);
}

// Any group size, any width, any alignment: one warp per (row, group).
template <typename T, bool E5M2>
__global__ void __launch_bounds__(256)
quant_group_any_kernel(uint8_t* __restrict__ out, float* __restrict__ scale,
                       const T* __restrict__ in, int64_t rows, int64_t cols, int group_size,
                       int64_t groups_per_row, float qmax) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (warp >= rows * groups_per_row) return;  // whole warp leaves together
  const int64_t row = warp / groups_per_row;
  const int64_t grp = warp - row * groups_per_row;
  const int64_t c0 = grp * group_size;
  const int64_t c1 = (c0 + group_size < cols) ? (c0 + group_size) : cols;
  const T* x = in + row * cols;
  uint8_t* y = out + row * cols;
  float amax = 0.f;
  for (int64_t c = c0 + lane; c < c1; c += 32) amax = fmaxf(amax, fabsf(to_f32<T>(x[c])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float sc = fmaxf(__fdiv_rn(amax, qmax), kScaleFloor);
  if (lane == 0) scale[warp] = sc;
  for (int64_t c = c0 + lane; c < c1; c += 32) y[c] = cvt_one<E5M2>(__fdiv_rn(to_f32<T>(x[c]), sc));
}

template <typename T, bool E5M2>
void launch(uint8_t* out, float* scale, const T* in, int64_t rows, int64_t cols, int gs,
            cudaStream_t s) {
  const float qmax = E5M2 ? 57344.0f : 448.0f;
  const int64_t groups_per_row = (cols + gs - 1) / gs;
  if (gs == 128 && cols % 128 == 0 && aligned16(in) && aligned16(out)) {
    const int64_t total_groups = rows * groups_per_row;
    constexpr int kSegs = KSB_QUANT_SEGS;
    const int64_t blocks = (total_groups * 8 + 256 * kSegs - 1) / (256 * kSegs);
    quant_group128_kernel<T, E5M2, kSegs><<<static_cast<unsigned>(blocks), 256, 0, s>>>(out, scale, in, total_groups, qmax);
  } else {
    const int64_t warps = rows * groups_per_row;
    const int64_t blocks = (warps + 7) / 8;
    quant_group_any_kernel<T, E5M2><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        out, scale, in, rows, cols, gs, groups_per_row, qmax);
  }
}

}  // namespace
}  // namespace ksb

extern "C" ks_status_t ks_quantize_fp8_group(void* out, float* scale, const void* input,
                                             int64_t rows, int64_t cols, int group_size,
                                             ks_dtype_t in_dtype, ks_dtype_t fp8_dtype,
                                             ks_stream_t stream) {
  using namespace ksb;
  KSB_REQUIRE_PTR(out);
  KSB_REQUIRE_PTR(scale);
  KSB_REQUIRE_PTR(input);
  if (rows <= 0 || cols <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_quantize_fp8_group: bad shape");
  if (group_size <= 0)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_quantize_fp8_group: group_size must be > 0");
  if (!is_fp8(fp8_dtype))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_quantize_fp8_group: fp8_dtype must be e4m3 or e5m2");
  if (!is_float3(in_dtype))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_quantize_fp8_group: unsupported dtype");
  const int64_t groups_per_row = (cols + group_size - 1) / group_size;
  // One warp (general kernel) or 8 lanes (fast kernel) per group must fit a 1-D grid.
  if (rows > (INT64_C(1) << 31) / groups_per_row * 4)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_quantize_fp8_group: grid exceeds CUDA grid limits");
  ks_status_t st = require_sm100("ks_quantize_fp8_group");
  if (st != KS_SUCCESS) return st;

  cudaStream_t s = as_stream(stream);
  uint8_t* o = static_cast<uint8_t*>(out);
  const bool e5 = fp8_dtype == KS_DTYPE_F8E5M2;
#define KSB_Q(T)                                                                        \
  do {                                                                                  \
    if (e5) launch<T, true>(o, scale, static_cast<const T*>(input), rows, cols, group_size, s); \
    else launch<T, false>(o, scale, static_cast<const T*>(input), rows, cols, group_size, s);   \
  } while (0)
  if (in_dtype == KS_DTYPE_F32) KSB_Q(float);
  else if (in_dtype == KS_DTYPE_F16) KSB_Q(__half);
  else KSB_Q(__nv_bfloat16);
#undef KSB_Q
  KSB_CHECK_LAUNCH("ks_quantize_fp8_group");
  return KS_SUCCESS;
}
