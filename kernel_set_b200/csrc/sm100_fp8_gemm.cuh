// Host interface of the tcgen05 FP8 block-scaled GEMM (dense and grouped).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "kernel_set/types.h"

namespace ksb {
namespace sm100 {

struct Fp8GemmArgs {
  const char* where = "";          // entry-point name for error messages
  void* out = nullptr;             // [m, n] out_dtype
  const void* a = nullptr;         // [m, k] fp8
  const void* b = nullptr;         // nt: [E][n, k]; else [E][k, n]
  const float* a_scale = nullptr;  // [m, ceil(k/128)]; or, with a_scale_ld > 0, stored column-major:
                                   // a_scale[kb * a_scale_ld + row]
  int64_t a_scale_ld = 0;
  const float* b_scale = nullptr;  // nt: [E][ceil(n/128), ceil(k/128)]; else transposed
  const int32_t* offsets = nullptr;  // [E+1] row boundaries; NULL = one dense problem
  int num_experts = 1;
  int64_t m = 0, n = 0, k = 0;     // m = all rows (all experts together)
  int block_n = 128, block_k = 128;
  bool nt = false;
  bool e5m2 = false;
  ks_dtype_t out_dtype = KS_DTYPE_BF16;
  int force_bn = 0;                // 128 / 256 pins the tile width (tests), 0 = choose
  int force_split = -1;            // K-split of the last partial round: -1 choose, 0 never, 1 whenever legal
  // Grouped, masked layout (a and out are [E, max_m, .]; expert e uses its first masked_m[e]
  // rows): set masked_m and max_m instead of offsets; m = E * max_m.
  const int32_t* masked_m = nullptr;
  int64_t max_m = 0;
  // mode 0: block scales as above. mode 1: fp8 operands, a_scale [m] or [1], b_scale [n] or
  // [1] (kernels/src/gemm/gemm_fp8.cu of the reference). mode 2: int8 operands, same scales,
  // optional bias [n] in the output type (gemm_w8a8.cu). mode 3: f16 / bf16 operands of type
  // out_dtype, a [m, k], b [E][k, n], no scales (kernels/src/moe/moe_grouped_gemm.cu), dense or grouped.
  int mode = 0;
  bool a_per_row = false, b_per_col = false;
  const void* bias = nullptr;
  // Scattered output (dense, mode 0): rows [b * rows_per_part, (b + 1) * rows_per_part) of the
  // product are written to out_parts[b] as a [rows_per_part, n] matrix; `out` is not used.
  // rows_per_part is a multiple of 128 and m = num_out_parts * rows_per_part. The parts may
  // live in other GPUs' memory (peer-mapped addresses): the tiles leave by TMA stores.
  void* const* out_parts = nullptr;
  int num_out_parts = 0;
  int64_t rows_per_part = 0;
};

// True when the tcgen05 kernel can take the problem (128 x 128 scale blocks,
// TMA-legal strides and alignment, driver entry point available).
bool fp8_blockwise_eligible(const Fp8GemmArgs& a);

// Encodes the tensor maps and enqueues one persistent launch on `stream`.
ks_status_t launch_fp8_blockwise(const Fp8GemmArgs& a, cudaStream_t stream);

}  // namespace sm100
}  // namespace ksb
