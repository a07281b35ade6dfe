// int4 weight format helpers: dense dequantisation of the int32-word packing
// and its re-layout into the byte packing the W4A16 GEMM reads.
//
// Reference: ks_dequantize_int4 (kernels/src/quant/dequant_int4.cu:78-112,
// kernel :36-60) and ks_repack_int4 (kernels/src/quant/repack_int4.cu:43-70,
// kernel :10-34).
//
// Word packing: qweight[K/8, N] int32, the code of k = 8*row + j is bits
// 4j..4j+3. Byte packing: out[K/2, N] uint8, code of even k in the low nibble.
// Byte i of a word therefore IS the output byte of row 4*word_row + i: the
// re-layout is a byte transpose with no nibble arithmetic.
//
// Both kernels are HBM-bound. A thread owns V adjacent columns of one word
// row: one V*4-byte load, then 8 (dequant) or 4 (repack) row stores of V
// elements, each coalesced across the warp. Algorithmic bytes per weight:
// dequant 0.5 + sizeof(out) (+ scales/zeros, 2*sizeof(out)/group_size);
// repack 0.5 + 0.5.
#include "common.cuh"
#include "kernel_set/quant.h"

namespace ksb {
namespace {

template <typename T, int V>
__global__ void __launch_bounds__(256)
dequant_int4_kernel(T* __restrict__ out, const int32_t* __restrict__ qw,
                    const T* __restrict__ scales, const T* __restrict__ zeros, int64_t k,
                    int64_t n, int group_size) {
  const int64_t nv = n / V;
  const int64_t total = (k >> 3) * nv;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t wr = idx / nv;
    const int64_t col = (idx - wr * nv) * V;
    uint32_t w[V];
    if constexpr (V == 4) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(qw + wr * n + col));
      w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w;
    } else {
      w[0] = static_cast<uint32_t>(__ldg(qw + wr * n + col));
    }
    int64_t g_prev = -1;
    float sc[V], zp[V];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t kk = wr * 8 + j;
      const int64_t g = kk / group_size;
      if (g != g_prev) {
#pragma unroll
        for (int v = 0; v < V; ++v) {
          sc[v] = to_f32<T>(scales[g * n + col + v]);
          zp[v] = to_f32<T>(zeros[g * n + col + v]);
        }
        g_prev = g;
      }
      T r[V];
#pragma unroll
      for (int v = 0; v < V; ++v) {
        const float q = static_cast<float>((w[v] >> (4 * j)) & 0xFu);
        r[v] = from_f32<T>(__fmul_rn(__fsub_rn(q, zp[v]), sc[v]));
      }
      T* dst = out + kk * n + col;
      if constexpr (V == 4 && sizeof(T) == 2) {
        *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(r);
      } else if constexpr (V == 4 && sizeof(T) == 4) {
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(r);
      } else {
#pragma unroll
        for (int v = 0; v < V; ++v) dst[v] = r[v];
      }
    }
  }
}

template <int V>
__global__ void __launch_bounds__(256)
repack_int4_kernel(uint8_t* __restrict__ out, const int32_t* __restrict__ in, int64_t rows_out,
                   int64_t n) {
  const int64_t nv = n / V;
  const int64_t word_rows = (rows_out + 3) >> 2;
  const int64_t total = word_rows * nv;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t wr = idx / nv;
    const int64_t col = (idx - wr * nv) * V;
    uint32_t w[V];
    if constexpr (V == 4) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(in + wr * n + col));
      w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w;
    } else {
      w[0] = static_cast<uint32_t>(__ldg(in + wr * n + col));
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t r = wr * 4 + i;
      if (r >= rows_out) break;
      uint8_t* dst = out + r * n + col;
      if constexpr (V == 4) {
        const uint32_t packed = ((w[0] >> (8 * i)) & 0xFFu) | (((w[1] >> (8 * i)) & 0xFFu) << 8) |
                                (((w[2] >> (8 * i)) & 0xFFu) << 16) | (((w[3] >> (8 * i)) & 0xFFu) << 24);
        *reinterpret_cast<uint32_t*>(dst) = packed;
      } else {
        dst[0] = static_cast<uint8_t>((w[0] >> (8 * i)) & 0xFFu);
      }
    }
  }
}

inline unsigned grid_for(int64_t work_items) {
  int64_t b = (work_items + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;  // grid-stride beyond this
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<unsigned>(b);
}

template <typename T>
void launch_dequant(void* out, const void* qw, const void* scales, const void* zeros, int64_t k,
                    int64_t n, int gs, cudaStream_t s) {
  const bool vec = (n % 4 == 0) && aligned16(qw) && aligned16(out);
  if (vec) {
    dequant_int4_kernel<T, 4><<<grid_for((k >> 3) * (n / 4)), 256, 0, s>>>(
        static_cast<T*>(out), static_cast<const int32_t*>(qw), static_cast<const T*>(scales),
        static_cast<const T*>(zeros), k, n, gs);
  } else {
    dequant_int4_kernel<T, 1><<<grid_for((k >> 3) * n), 256, 0, s>>>(
        static_cast<T*>(out), static_cast<const int32_t*>(qw), static_cast<const T*>(scales),
        static_cast<const T*>(zeros), k, n, gs);
  }
}

}  // namespace
}  // namespace ksb

extern "C" {

ks_status_t ks_dequantize_int4(void* out, const void* qweight_packed, const void* scales,
                               const void* zeros, int64_t k, int64_t n, int group_size,
                               ks_dtype_t out_dtype, ks_stream_t stream) {
  using namespace ksb;
  KSB_REQUIRE_PTR(out);
  KSB_REQUIRE_PTR(qweight_packed);
  KSB_REQUIRE_PTR(scales);
  KSB_REQUIRE_PTR(zeros);
  if (k <= 0 || n <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_dequantize_int4: bad shape");
  if (group_size <= 0)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_dequantize_int4: group_size must be > 0");
  if (k % 8 != 0)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_dequantize_int4: K must be a multiple of 8 (8 codes/word)");
  if (k % group_size != 0)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_dequantize_int4: K must be a multiple of group_size");
  if (!is_float3(out_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_dequantize_int4: unsupported dtype");
  ks_status_t st = require_sm100("ks_dequantize_int4");
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  if (out_dtype == KS_DTYPE_F32) launch_dequant<float>(out, qweight_packed, scales, zeros, k, n, group_size, s);
  else if (out_dtype == KS_DTYPE_F16) launch_dequant<__half>(out, qweight_packed, scales, zeros, k, n, group_size, s);
  else launch_dequant<__nv_bfloat16>(out, qweight_packed, scales, zeros, k, n, group_size, s);
  KSB_CHECK_LAUNCH("ks_dequantize_int4");
  return KS_SUCCESS;
}

ks_status_t ks_repack_int4(void* out_packed, const void* qweight, const void* perm, int64_t size_k,
                           int64_t size_n, int num_bits, ks_stream_t stream) {
  using namespace ksb;
  KSB_REQUIRE_PTR(out_packed);
  KSB_REQUIRE_PTR(qweight);
  if (size_k <= 0 || size_n <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_repack_int4: bad shape");
  if (num_bits != 4) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_repack_int4: only 4-bit supported");
  if (perm != nullptr)
    KSB_FAIL(KS_ERROR_NOT_IMPLEMENTED, "ks_repack_int4: act-order perm not yet supported");
  ks_status_t st = require_sm100("ks_repack_int4");
  if (st != KS_SUCCESS) return st;
  const int64_t rows_out = size_k / 2;
  if (rows_out == 0) return KS_SUCCESS;
  cudaStream_t s = as_stream(stream);
  const bool vec = (size_n % 4 == 0) && aligned16(qweight) && ((reinterpret_cast<uintptr_t>(out_packed) & 3u) == 0);
  const int64_t word_rows = (rows_out + 3) / 4;
  if (vec) {
    repack_int4_kernel<4><<<grid_for(word_rows * (size_n / 4)), 256, 0, s>>>(
        static_cast<uint8_t*>(out_packed), static_cast<const int32_t*>(qweight), rows_out, size_n);
  } else {
    repack_int4_kernel<1><<<grid_for(word_rows * size_n), 256, 0, s>>>(
        static_cast<uint8_t*>(out_packed), static_cast<const int32_t*>(qweight), rows_out, size_n);
  }
  KSB_CHECK_LAUNCH("ks_repack_int4");
  return KS_SUCCESS;
}

}  // extern "C"
