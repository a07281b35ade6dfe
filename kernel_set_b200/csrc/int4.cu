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
// Checkpoint formats (the import entries at the end of this file):
//   GPTQ  qweight [K/8, N] int32 = the word packing above; qzeros [G, N/8]
//         int32, column 8c+j in bits 4j..4j+3, holding zero-1 in files of the
//         first format version; g_idx [K] names the group of each row when the
//         rows were quantised in activation order.
//   AWQ   qweight [K, N/8] and qzeros [G, N/8] int32, column 8c+j in nibble
//         {0,4,1,5,2,6,3,7}[j] of word c (the packer fills nibble i with column
//         8c + {0,2,4,6,1,3,5,7}[i]).
// An import thread owns eight adjacent columns: it brings the codes of its
// source rows into "natural" words (column j in nibble j) and then emits the
// byte rows or the code words of the target packing.
//
// Both kernels are HBM-bound. A thread owns V adjacent columns of one word
// row: one V*4-byte load, then 8 (dequant) or 4 (repack) row stores of V
// elements, each coalesced across the warp. Algorithmic bytes per weight:
// dequant 0.5 + sizeof(out) (+ scales/zeros, 2*sizeof(out)/group_size);
// repack 0.5 + 0.5.
#include <algorithm>

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

// ---- checkpoint import ------------------------------------------------------

// nibble of an AWQ word that holds column j of its eight
__device__ __forceinline__ uint32_t awq_to_natural(uint32_t w) {
  // natural nibble j = source nibble {0,4,1,5,2,6,3,7}[j]
  return (w & 0xFu) | (((w >> 16) & 0xFu) << 4) | (((w >> 4) & 0xFu) << 8) |
         (((w >> 20) & 0xFu) << 12) | (((w >> 8) & 0xFu) << 16) | (((w >> 24) & 0xFu) << 20) |
         (((w >> 12) & 0xFu) << 24) | (((w >> 28) & 0xFu) << 28);
}

// codes of row `kk`, columns 8c..8c+7, column j in nibble j; 0 for a row outside the matrix
template <int SOURCE>
__device__ __forceinline__ uint32_t natural_row(const int32_t* __restrict__ qw, int64_t kk, int64_t c,
                                                int64_t k, int64_t n) {
  if (kk < 0 || kk >= k) return 0u;
  if constexpr (SOURCE == 1) {
    return awq_to_natural(static_cast<uint32_t>(__ldg(qw + kk * (n >> 3) + c)));
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(qw + (kk >> 3) * n + c * 8);
    const uint4 lo = __ldg(src), hi = __ldg(src + 1);
    const int sh = static_cast<int>(kk & 7) * 4;
    return ((lo.x >> sh) & 0xFu) | (((lo.y >> sh) & 0xFu) << 4) | (((lo.z >> sh) & 0xFu) << 8) |
           (((lo.w >> sh) & 0xFu) << 12) | (((hi.x >> sh) & 0xFu) << 16) |
           (((hi.y >> sh) & 0xFu) << 20) | (((hi.z >> sh) & 0xFu) << 24) |
           (((hi.w >> sh) & 0xFu) << 28);
  }
}

// ROWS = 2: one byte row of the [K/2, N] packing; ROWS = 8: one word row of [K/8, N].
template <int SOURCE, int ROWS>
__global__ void __launch_bounds__(256)
import_weight_kernel(void* __restrict__ out, const int32_t* __restrict__ qw,
                     const int32_t* __restrict__ perm, int64_t k, int64_t n) {
  const int64_t nc = n >> 3;
  const int64_t out_rows = (k + ROWS - 1) / ROWS;
  const int64_t total = out_rows * nc;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / nc;
    const int64_t c = idx - r * nc;
    uint32_t nat[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      int64_t kk = r * ROWS + i;
      if (kk < k && perm != nullptr) kk = __ldg(perm + kk);
      nat[i] = (r * ROWS + i < k) ? natural_row<SOURCE>(qw, kk, c, k, n) : 0u;
    }
    if constexpr (ROWS == 2) {
      uint32_t b[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t v = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int sh = (h * 4 + j) * 4;
          v |= (((nat[0] >> sh) & 0xFu) | (((nat[1] >> sh) & 0xFu) << 4)) << (8 * j);
        }
        b[h] = v;
      }
      *reinterpret_cast<uint2*>(static_cast<uint8_t*>(out) + r * n + c * 8) = make_uint2(b[0], b[1]);
    } else {
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t v = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) v |= ((nat[i] >> (4 * j)) & 0xFu) << (4 * i);
        w[j] = v;
      }
      uint4* dst = reinterpret_cast<uint4*>(static_cast<int32_t*>(out) + r * n + c * 8);
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
import_zeros_kernel(T* __restrict__ out, const int32_t* __restrict__ qz, int64_t groups, int64_t n,
                    int source, int zero_offset) {
  const int64_t nc = n >> 3;
  const int64_t total = groups * nc;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    uint32_t w = static_cast<uint32_t>(__ldg(qz + idx));
    if (source == 1) w = awq_to_natural(w);
    T* dst = out + idx * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      dst[j] = from_f32<T>(static_cast<float>(static_cast<int>((w >> (4 * j)) & 0xFu) + zero_offset));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
gather_columns_kernel(T* __restrict__ out, const T* __restrict__ in, const int32_t* __restrict__ perm,
                      int64_t cols) {
  const int64_t row = blockIdx.y;
  for (int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < cols;
       j += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t src = __ldg(perm + j);
    out[row * cols + j] = (src >= 0 && src < cols) ? in[row * cols + src] : from_f32<T>(0.0f);
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
  if (perm != nullptr && (size_k % 8 != 0 || size_n % 8 != 0 || !aligned16(qweight) ||
                          (reinterpret_cast<uintptr_t>(out_packed) & 7u) != 0))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE,
             "ks_repack_int4: with perm, K and N must be multiples of 8, qweight 16-byte and out 8-byte aligned");
  ks_status_t st = require_sm100("ks_repack_int4");
  if (st != KS_SUCCESS) return st;
  const int64_t rows_out = size_k / 2;
  if (rows_out == 0) return KS_SUCCESS;
  cudaStream_t s = as_stream(stream);
  if (perm != nullptr) {
    // row k' of the result is row perm[k'] of the source
    import_weight_kernel<0, 2><<<grid_for(rows_out * (size_n / 8)), 256, 0, s>>>(
        out_packed, static_cast<const int32_t*>(qweight), static_cast<const int32_t*>(perm), size_k, size_n);
    KSB_CHECK_LAUNCH("ks_repack_int4");
    return KS_SUCCESS;
  }
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

ks_status_t ks_int4_import_weight(void* out, const void* qweight, const int32_t* perm, int64_t size_k,
                                  int64_t size_n, ks_int4_source_t source, ks_int4_packing_t packing,
                                  ks_stream_t stream) {
  using namespace ksb;
  KSB_REQUIRE_PTR(out);
  KSB_REQUIRE_PTR(qweight);
  if (size_k <= 0 || size_n <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_int4_import_weight: bad shape");
  if (source != KS_INT4_SOURCE_GPTQ && source != KS_INT4_SOURCE_AWQ)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_int4_import_weight: unknown source format");
  if (packing != KS_INT4_PACKING_BYTES && packing != KS_INT4_PACKING_WORDS)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_int4_import_weight: unknown target packing");
  if (size_k % 8 != 0 || size_n % 8 != 0)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_int4_import_weight: K and N must be multiples of 8");
  if (!aligned16(out) || !aligned16(qweight))
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_int4_import_weight: pointers must be 16-byte aligned");
  ks_status_t st = require_sm100("ks_int4_import_weight");
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const int32_t* qw = static_cast<const int32_t*>(qweight);
  const int64_t nc = size_n / 8;
  if (packing == KS_INT4_PACKING_BYTES) {
    const unsigned g = grid_for((size_k / 2) * nc);
    if (source == KS_INT4_SOURCE_AWQ) import_weight_kernel<1, 2><<<g, 256, 0, s>>>(out, qw, perm, size_k, size_n);
    else import_weight_kernel<0, 2><<<g, 256, 0, s>>>(out, qw, perm, size_k, size_n);
  } else {
    const unsigned g = grid_for((size_k / 8) * nc);
    if (source == KS_INT4_SOURCE_AWQ) import_weight_kernel<1, 8><<<g, 256, 0, s>>>(out, qw, perm, size_k, size_n);
    else import_weight_kernel<0, 8><<<g, 256, 0, s>>>(out, qw, perm, size_k, size_n);
  }
  KSB_CHECK_LAUNCH("ks_int4_import_weight");
  return KS_SUCCESS;
}

ks_status_t ks_int4_import_zeros(void* zeros, const void* qzeros, int64_t groups, int64_t size_n,
                                 ks_int4_source_t source, int zero_offset, ks_dtype_t out_dtype,
                                 ks_stream_t stream) {
  using namespace ksb;
  KSB_REQUIRE_PTR(zeros);
  KSB_REQUIRE_PTR(qzeros);
  if (groups <= 0 || size_n <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_int4_import_zeros: bad shape");
  if (source != KS_INT4_SOURCE_GPTQ && source != KS_INT4_SOURCE_AWQ)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_int4_import_zeros: unknown source format");
  if (zero_offset < 0 || zero_offset > 1)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_int4_import_zeros: zero_offset must be 0 or 1");
  if (size_n % 8 != 0) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_int4_import_zeros: N must be a multiple of 8");
  if (!is_float3(out_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_int4_import_zeros: unsupported dtype");
  ks_status_t st = require_sm100("ks_int4_import_zeros");
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const unsigned g = grid_for(groups * (size_n / 8));
  const int32_t* qz = static_cast<const int32_t*>(qzeros);
  const int src = static_cast<int>(source);
  if (out_dtype == KS_DTYPE_F32)
    import_zeros_kernel<float><<<g, 256, 0, s>>>(static_cast<float*>(zeros), qz, groups, size_n, src, zero_offset);
  else if (out_dtype == KS_DTYPE_F16)
    import_zeros_kernel<__half><<<g, 256, 0, s>>>(static_cast<__half*>(zeros), qz, groups, size_n, src, zero_offset);
  else
    import_zeros_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(static_cast<__nv_bfloat16*>(zeros), qz, groups, size_n, src, zero_offset);
  KSB_CHECK_LAUNCH("ks_int4_import_zeros");
  return KS_SUCCESS;
}

ks_status_t ks_gather_columns(void* out, const void* input, const int32_t* perm, int64_t rows,
                              int64_t cols, ks_dtype_t dtype, ks_stream_t stream) {
  using namespace ksb;
  KSB_REQUIRE_PTR(out);
  KSB_REQUIRE_PTR(input);
  KSB_REQUIRE_PTR(perm);
  if (rows < 0 || cols <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_gather_columns: bad shape");
  if (out == input) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_gather_columns: out must not alias input");
  if (!is_float3(dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_gather_columns: unsupported dtype");
  if (rows > 65535) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_gather_columns: at most 65535 rows per call");
  ks_status_t st = require_sm100("ks_gather_columns");
  if (st != KS_SUCCESS) return st;
  if (rows == 0) return KS_SUCCESS;
  cudaStream_t s = as_stream(stream);
  const dim3 grid(static_cast<unsigned>(std::min<int64_t>((cols + 255) / 256, 64)), static_cast<unsigned>(rows));
  if (dtype == KS_DTYPE_F32)
    gather_columns_kernel<float><<<grid, 256, 0, s>>>(static_cast<float*>(out), static_cast<const float*>(input), perm, cols);
  else if (dtype == KS_DTYPE_F16)
    gather_columns_kernel<__half><<<grid, 256, 0, s>>>(static_cast<__half*>(out), static_cast<const __half*>(input), perm, cols);
  else
    gather_columns_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(input), perm, cols);
  KSB_CHECK_LAUNCH("ks_gather_columns");
  return KS_SUCCESS;
}

}  // extern "C"
