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
#include <cstdlib>

#include "common.cuh"
#include "kernel_set/quant.h"
#include "quant_math.cuh"

#ifndef KSB_QUANT_SEGS
#define KSB_QUANT_SEGS 1
#endif

namespace ksb {
namespace {

using namespace quantmath;

// A thread owns kSegs segments, all loaded before the first is used. Measured on B200 for
// [4096, 7168] bf16: 22 us with one segment per thread, 25 us with two, 35 us with four
// (fewer resident threads cost more than the extra loads in flight gain), so one it is.
// Column-major scales: scale_t[g * ld + row] instead of scale[row * groups + g], so that the
// 128 rows of a GEMM tile find their scales of one K-block in 512 contiguous bytes.
template <typename T, bool E5M2>
__global__ void __launch_bounds__(256)
quant_group128_colscale_kernel(uint8_t* __restrict__ out, float* __restrict__ scale_t, int64_t ld,
                               const T* __restrict__ in, int64_t total_groups, int groups_per_row, float qmax) {
  const int64_t seg = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool live = (seg >> 3) < total_groups;
  float v[16];
  if (live) {
    Vec16<T>::load(in + seg * 16, v);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
  }
  float sc;
  const uint4 codes = quant_segment_codes<E5M2>(v, qmax, &sc);
  if (!live) return;
  if ((threadIdx.x & 7) == 0) {
    const int64_t grp = seg >> 3;
    const int64_t row = grp / groups_per_row;
    scale_t[(grp - row * groups_per_row) * ld + row] = sc;
  }
  __stcs(reinterpret_cast<uint4*>(out + seg * 16), codes);
}

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
    // (Measured and not kept: a grid-stride form with the next segment's loads in flight during
    // the arithmetic, 22-24 us; persistent blocks fed by 8 KB bulk copies through a 12-stage
    // shared-memory ring, ~190 KB in flight per SM: 5.4 TB/s on [16384, 7168] where this kernel
    // reaches 5.6, and slower on [4096, 7168]. At that size a fixed ~5 us of launch, ramp and
    // tail is what separates the kernel from its steady-state rate.)
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

extern "C" ks_status_t ks_quantize_fp8_group_colscale(void* out, float* scale_t, int64_t scale_ld, const void* input,
                                                      int64_t rows, int64_t cols, ks_dtype_t in_dtype,
                                                      ks_dtype_t fp8_dtype, ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_quantize_fp8_group_colscale";
  KSB_REQUIRE_PTR(out);
  KSB_REQUIRE_PTR(scale_t);
  KSB_REQUIRE_PTR(input);
  if (rows <= 0 || cols <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_quantize_fp8_group_colscale: bad shape");
  if (scale_ld < rows) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_quantize_fp8_group_colscale: scale_ld must be at least rows");
  if (cols % 128 != 0 || !aligned16(input) || !aligned16(out))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE,
             "ks_quantize_fp8_group_colscale: cols must be a multiple of 128 and the buffers 16-byte aligned");
  if (!is_fp8(fp8_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_quantize_fp8_group_colscale: fp8_dtype must be e4m3 or e5m2");
  if (!is_float3(in_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_quantize_fp8_group_colscale: unsupported dtype");
  const int64_t groups_per_row = cols / 128;
  if (rows > (INT64_C(1) << 31) / groups_per_row * 4)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_quantize_fp8_group_colscale: grid exceeds CUDA grid limits");
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const int64_t total_groups = rows * groups_per_row;
  const unsigned blocks = static_cast<unsigned>((total_groups * 8 + 255) / 256);
  uint8_t* o = static_cast<uint8_t*>(out);
  const bool e5 = fp8_dtype == KS_DTYPE_F8E5M2;
#define KSB_QC(T)                                                                                                   \
  do {                                                                                                              \
    if (e5) quant_group128_colscale_kernel<T, true><<<blocks, 256, 0, s>>>(o, scale_t, scale_ld, static_cast<const T*>(input), \
                                                                           total_groups, static_cast<int>(groups_per_row), 57344.0f); \
    else quant_group128_colscale_kernel<T, false><<<blocks, 256, 0, s>>>(o, scale_t, scale_ld, static_cast<const T*>(input),  \
                                                                         total_groups, static_cast<int>(groups_per_row), 448.0f);  \
  } while (0)
  if (in_dtype == KS_DTYPE_F32) KSB_QC(float);
  else if (in_dtype == KS_DTYPE_F16) KSB_QC(__half);
  else KSB_QC(__nv_bfloat16);
#undef KSB_QC
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}
