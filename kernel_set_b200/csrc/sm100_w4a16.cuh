// Host interface of the tcgen05 int4 weight-only GEMM.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "kernel_set/types.h"

namespace ksb {
namespace sm100 {

struct W4A16Args {
  void* c = nullptr;               // [m, n] dtype
  const void* a = nullptr;         // [m, k] dtype
  const void* b_packed = nullptr;  // [k/2, n] uint8, even k in the low nibble
  const void* scales = nullptr;    // [k/group_size, n] dtype
  const void* zeros = nullptr;     // same shape or NULL (zero-point 0)
  const void* bias = nullptr;      // [n] or NULL
  int64_t m = 0, n = 0, k = 0;
  int group_size = 128;            // already resolved (> 0, divides k)
  ks_dtype_t dtype = KS_DTYPE_BF16;
  // How the tcgen05 kernel hands the dequantised weights of decode shapes (at most 32
  // token rows) to the tensor core: 0 = choose (tensor memory), 1 = shared memory,
  // 2 = tensor memory.
  int operand_path = 0;
  // Which fast kernel: 0 = choose, 1 = tcgen05 (sm100_w4a16.cu), 2 = register-operand
  // decode kernel (w4a16_decode.cu).
  int kernel = 0;
};

// Stream-K split shared by both fast kernels: units (column tile * k_steps + K-step) are
// dealt to the CTAs in equal contiguous runs.
__host__ __device__ __forceinline__ long long run_start(long long units, int ctas, int c) {
  return (units * c) / ctas;
}
__host__ __device__ __forceinline__ int cta_of_unit(long long units, int ctas, long long u) {
  int c = static_cast<int>((u * ctas) / units);
  while (c + 1 < ctas && run_start(units, ctas, c + 1) <= u) ++c;
  while (c > 0 && run_start(units, ctas, c) > u) --c;
  return c;
}

// True when the tcgen05 kernel can take the problem: K and group_size multiples
// of 128, N a multiple of 16, 16-byte aligned operands, driver entry point found.
bool w4a16_eligible(const W4A16Args& a);

// Encodes the tensor maps, sizes the scratch memory and enqueues one launch.
ks_status_t launch_w4a16(const W4A16Args& a, cudaStream_t stream);

// Same launch with the scratch taken from a fixed array in the library image;
// performs no device or host allocation. Shapes whose scratch need exceeds
// w4a16_static_scratch_capacity() are refused with KS_ERROR_UNSUPPORTED_SHAPE.
ks_status_t launch_w4a16_static(const W4A16Args& a, cudaStream_t stream);
size_t w4a16_static_scratch_capacity();

// Register-operand kernel for the decode regime (w4a16_decode.cu): cp.async ring,
// ldmatrix, in-register dequantisation, mma.sync; split-K finished per warp.
namespace decode {
constexpr int kMaxTokens = 64;
struct Geometry {
  int mg = 1;      // token groups of 8 (1, 2, 4 or 8)
  int n_tiles = 0, k_steps = 0, grid = 0, max_parts = 0;
  size_t counter_bytes = 0, slot_bytes = 0;
};
// K and group_size multiples of 128, N a multiple of 16, at most kMaxTokens rows,
// 16-byte aligned operands.
bool eligible(const W4A16Args& a);
Geometry geometry_of(const W4A16Args& a);
// Enqueues one launch on scratch the caller owns: `counters` (all zero on entry; the
// kernel leaves them zero) and `slots`.
ks_status_t enqueue(const W4A16Args& a, const Geometry& g, unsigned int* counters, float* slots,
                    cudaStream_t stream);
}  // namespace decode

}  // namespace sm100
}  // namespace ksb
