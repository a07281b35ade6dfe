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
  // How decode shapes (at most 32 token rows) hand the dequantised weights to the tensor
  // core: 0 = choose (tensor memory), 1 = shared memory, 2 = tensor memory.
  int operand_path = 0;
};

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

}  // namespace sm100
}  // namespace ksb
