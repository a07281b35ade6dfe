// General (any shape, any block size, any supported dtype) kernels of the
// quantized GEMMs. They cover what the tcgen05 kernels decline: ragged or
// unaligned shapes, block sizes other than 128, e5m2 x f32-out corners, and
// they serve as the on-device cross-check of the fast kernels in the tests.
//
// One engine: 64 x 64 output tile, 256 threads, 4 x 4 register micro-tile,
// fp32 shared-memory staging in chunks of 16 along K, fp32 accumulation in
// ascending k. Operands are converted to fp32 while being staged, so the
// inner loop is shared by all three ops.
//
// The accumulation order (ascending k inside a K-block, then one fused
// multiply-add per K-block with the scale product) is the order of the
// reference kernels (gemm_fp8_blockwise.cu:107-150, gemm_w4a16.cu:74-114,
// moe_grouped_gemm.cu:72-127), so for fp32 outputs these kernels reproduce
// the reference kernels' bits.
#pragma once

#include "common.cuh"

namespace ksb {
namespace general {

constexpr int kTM = 64, kTN = 64, kTK = 16, kThreads = 256;

// Maps a block to (expert, first row, end row) when rows are grouped by
// expert: blockIdx.x counts 64-row tiles expert after expert. Returns false
// for the slack blocks past the last tile.
__device__ __forceinline__ bool locate_group_tile(const int32_t* __restrict__ offsets, int num_experts,
                                                  int tile, int* expert, int64_t* row0, int64_t* row_end) {
  __shared__ int s_e;
  __shared__ int64_t s_r0, s_r1;
  if (threadIdx.x == 0) {
    int e_found = -1;
    int64_t r0 = 0, r1 = 0;
    int t = tile;
    for (int e = 0; e < num_experts; ++e) {
      const int64_t b = offsets[e], en = offsets[e + 1];
      const int64_t rows = en > b ? en - b : 0;
      const int tiles = static_cast<int>((rows + kTM - 1) / kTM);
      if (t < tiles) { e_found = e; r0 = b + static_cast<int64_t>(t) * kTM; r1 = en; break; }
      t -= tiles;
    }
    s_e = e_found; s_r0 = r0; s_r1 = r1;
  }
  __syncthreads();
  *expert = s_e; *row0 = s_r0; *row_end = s_r1;
  return s_e >= 0;
}

struct Tile {
  float a[kTK][kTM + 4];
  float b[kTK][kTN + 4];
};

__device__ __forceinline__ void mac_chunk(const Tile& t, int tr, int tc, float (&acc)[4][4]) {
#pragma unroll
  for (int kk = 0; kk < kTK; ++kk) {
    float av[4], bv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) av[i] = t.a[kk][tr * 4 + i];
#pragma unroll
    for (int j = 0; j < 4; ++j) bv[j] = t.b[kk][tc * 4 + j];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
  }
}

// Stage rows [row0, row0+64) x k [k0, k0+16) of a row-major [rows_total, K]
// matrix; anything at or beyond row_end / k_end becomes 0.
template <typename T>
__device__ __forceinline__ void stage_a(Tile& t, const T* __restrict__ a, int64_t lda, int64_t row0,
                                        int64_t row_end, int64_t k0, int64_t k_end) {
  const int r = threadIdx.x >> 2;
  const int kc = (threadIdx.x & 3) * 4;
  const int64_t gr = row0 + r;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int64_t gk = k0 + kc + u;
    t.a[kc + u][r] = (gr < row_end && gk < k_end) ? to_f32<T>(a[gr * lda + gk]) : 0.f;
  }
}

// B stored [K, N] (ldb = N): stage k [k0,k0+16) x n [n0,n0+64).
template <typename T>
__device__ __forceinline__ void stage_b_kn(Tile& t, const T* __restrict__ b, int64_t ldb, int64_t k0,
                                           int64_t k_end, int64_t n0, int64_t n_end) {
  const int kr = threadIdx.x >> 4;
  const int nc = (threadIdx.x & 15) * 4;
  const int64_t gk = k0 + kr;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int64_t gn = n0 + nc + u;
    t.b[kr][nc + u] = (gk < k_end && gn < n_end) ? to_f32<T>(b[gk * ldb + gn]) : 0.f;
  }
}

// B stored [N, K] (ldb = K).
template <typename T>
__device__ __forceinline__ void stage_b_nk(Tile& t, const T* __restrict__ b, int64_t ldb, int64_t k0,
                                           int64_t k_end, int64_t n0, int64_t n_end) {
  const int nr = threadIdx.x >> 2;
  const int kc = (threadIdx.x & 3) * 4;
  const int64_t gn = n0 + nr;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int64_t gk = k0 + kc + u;
    t.b[kc + u][nr] = (gn < n_end && gk < k_end) ? to_f32<T>(b[gn * ldb + gk]) : 0.f;
  }
}

// ---------------------------------------------------------------------------
// FP8 block-scaled GEMM, optionally grouped by expert.
//   NT == false: B [E][K,N], b_scale [E][nkb, nnb]
//   NT == true : B [E][N,K], b_scale [E][nnb, nkb]
// ---------------------------------------------------------------------------
template <typename F8, typename OutT, bool NT, bool GROUPED>
__global__ void __launch_bounds__(kThreads)
fp8_blockwise_kernel(OutT* __restrict__ c, const F8* __restrict__ a, const F8* __restrict__ b,
                     const float* __restrict__ a_scale, const float* __restrict__ b_scale,
                     const int32_t* __restrict__ offsets, int num_experts, int64_t m, int64_t n,
                     int64_t k, int block_n, int block_k, int64_t nkb, int64_t nnb) {
  __shared__ Tile tile;
  int expert = 0;
  int64_t row0 = static_cast<int64_t>(blockIdx.x) * kTM, row_end = m;
  if constexpr (GROUPED) {
    if (!locate_group_tile(offsets, num_experts, blockIdx.x, &expert, &row0, &row_end)) return;
    b += static_cast<int64_t>(expert) * k * n;
    b_scale += static_cast<int64_t>(expert) * nkb * nnb;
  }
  const int64_t n0 = static_cast<int64_t>(blockIdx.y) * kTN;
  const int tr = threadIdx.x >> 4, tc = threadIdx.x & 15;

  float total[4][4] = {};
  for (int64_t kb = 0; kb < nkb; ++kb) {
    const int64_t kb0 = kb * block_k;
    const int64_t kb1 = (kb0 + block_k < k) ? kb0 + block_k : k;
    float part[4][4] = {};
    for (int64_t k0 = kb0; k0 < kb1; k0 += kTK) {
      stage_a<F8>(tile, a, k, row0, row_end, k0, kb1);
      if constexpr (NT) stage_b_nk<F8>(tile, b, k, k0, kb1, n0, n);
      else stage_b_kn<F8>(tile, b, n, k0, kb1, n0, n);
      __syncthreads();
      mac_chunk(tile, tr, tc, part);
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t gr = row0 + tr * 4 + i;
      if (gr >= row_end) continue;
      const float as = a_scale[gr * nkb + kb];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int64_t gn = n0 + tc * 4 + j;
        if (gn >= n) continue;
        const int64_t nb = gn / block_n;
        const float bs = NT ? b_scale[nb * nkb + kb] : b_scale[kb * nnb + nb];
        total[i][j] = fmaf(part[i][j], as * bs, total[i][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gr = row0 + tr * 4 + i;
    if (gr >= row_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t gn = n0 + tc * 4 + j;
      if (gn < n) c[gr * n + gn] = from_f32<OutT>(total[i][j]);
    }
  }
}

// ---------------------------------------------------------------------------
// Unscaled grouped GEMM: C[rows of e] = A[rows of e] . B[e], B [E][K,N].
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
grouped_plain_kernel(T* __restrict__ c, const T* __restrict__ a, const T* __restrict__ b,
                     const int32_t* __restrict__ offsets, int num_experts, int64_t n, int64_t k) {
  __shared__ Tile tile;
  int expert;
  int64_t row0, row_end;
  if (!locate_group_tile(offsets, num_experts, blockIdx.x, &expert, &row0, &row_end)) return;
  b += static_cast<int64_t>(expert) * k * n;
  const int64_t n0 = static_cast<int64_t>(blockIdx.y) * kTN;
  const int tr = threadIdx.x >> 4, tc = threadIdx.x & 15;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < k; k0 += kTK) {
    stage_a<T>(tile, a, k, row0, row_end, k0, k);
    stage_b_kn<T>(tile, b, n, k0, k, n0, n);
    __syncthreads();
    mac_chunk(tile, tr, tc, acc);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gr = row0 + tr * 4 + i;
    if (gr >= row_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t gn = n0 + tc * 4 + j;
      if (gn < n) c[gr * n + gn] = from_f32<T>(acc[i][j]);
    }
  }
}

// ---------------------------------------------------------------------------
// W4A16: weight (q - zero) * scale is rounded once to the activation type
// (as the reference's torch statement does, benchmarks/bench.py:1282-1284),
// then multiplied in fp32.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
w4a16_kernel(T* __restrict__ c, const T* __restrict__ a, const uint8_t* __restrict__ bq,
             const T* __restrict__ scales, const T* __restrict__ zeros, const T* __restrict__ bias,
             int64_t m, int64_t n, int64_t k, int group_size) {
  __shared__ Tile tile;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * kTM;
  const int64_t n0 = static_cast<int64_t>(blockIdx.y) * kTN;
  const int tr = threadIdx.x >> 4, tc = threadIdx.x & 15;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < k; k0 += kTK) {
    stage_a<T>(tile, a, k, row0, m, k0, k);
    {
      const int kr = threadIdx.x >> 4;
      const int nc = (threadIdx.x & 15) * 4;
      const int64_t gk = k0 + kr;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t gn = n0 + nc + u;
        float w = 0.f;
        if (gk < k && gn < n) {
          const uint8_t byte = bq[(gk >> 1) * n + gn];
          const float q = static_cast<float>((gk & 1) ? (byte >> 4) : (byte & 0xF));
          const int64_t g = gk / group_size;
          const float sc = to_f32<T>(scales[g * n + gn]);
          const float zp = zeros ? to_f32<T>(zeros[g * n + gn]) : 0.f;
          w = to_f32<T>(from_f32<T>(__fmul_rn(__fsub_rn(q, zp), sc)));
        }
        tile.b[kr][nc + u] = w;
      }
    }
    __syncthreads();
    mac_chunk(tile, tr, tc, acc);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gr = row0 + tr * 4 + i;
    if (gr >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t gn = n0 + tc * 4 + j;
      if (gn >= n) continue;
      float v = acc[i][j];
      if (bias) v += to_f32<T>(bias[gn]);
      c[gr * n + gn] = from_f32<T>(v);
    }
  }
}

}  // namespace general
}  // namespace ksb
