// The steps of a mixture-of-experts layer that sit between the router's logits and the
// two grouped expert GEMMs, and after them: gate (softmax + top-k), the permutation that
// sorts (token, slot) pairs by expert, the row gather (optionally fused with the 1 x 128
// FP8 quantizer), SwiGLU between the GEMMs (optionally fused with the re-quantisation),
// and the weighted sum that brings expert outputs back to token order.
//
// Reference: ks_moe_gate_softmax_topk (kernels/src/moe/moe_gate.cu:43-119),
// ks_moe_compute_permutation / ks_moe_permute / ks_moe_unpermute
// (kernels/src/moe/moe_permute.cu:60-170, 179-380), ks_swiglu / ks_swiglu_packed
// (kernels/src/activation/gated_mlp.cu:39-134). Differences, on purpose:
//   * nothing here allocates per call or synchronises the stream (the reference's
//     permutation and unpermute launchers cudaMalloc, cudaStreamSynchronize and cudaFree
//     on every call, moe_permute.cu:205-242, 317-375); the one piece of workspace, the
//     inverse permutation of ks_moe_unpermute, is a stream-ordered library buffer;
//   * the permutation is a STABLE counting sort (pairs of one expert keep their
//     token order), so results are reproducible; the reference scatters with atomics and
//     leaves the order inside an expert unspecified;
//   * the gate evaluates exp with expf (the reference's torch statement, benchmarks/
//     bench.py:1555-1557, is the parity target; the reference kernel uses __expf).
#include <cstdio>
#include <type_traits>

#include "common.cuh"
#include "kernel_set/activation.h"
#include "kernel_set/moe.h"
#include "quant_math.cuh"
#include "sm100_host.cuh"

namespace ksb {
namespace {

constexpr int kMaxExperts = 1024;   // as the reference (moe_gate.cu:33)
constexpr int kMaxTopK = 32;        // as the reference (moe_gate.cu:35)

// ---------------------------------------------------------------------------------
// gate: one warp per token
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
gate_softmax_topk_kernel(float* __restrict__ out_w, int32_t* __restrict__ out_i, const T* __restrict__ logits,
                         int64_t tokens, int experts, int top_k, int renorm) {
  extern __shared__ float gate_smem[];   // [warps][experts]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t token = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (token >= tokens) return;   // whole warp
  float* p = gate_smem + warp * experts;
  const T* row = logits + token * experts;
  float mx = -3.4028235e38f;
  for (int e = lane; e < experts; e += 32) {
    const float v = to_f32<T>(row[e]);
    p[e] = v;
    mx = fmaxf(mx, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int e = lane; e < experts; e += 32) {
    const float ex = expf(p[e] - mx);
    p[e] = ex;
    sum += ex;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  for (int e = lane; e < experts; e += 32) p[e] = __fdiv_rn(p[e], sum);
  __syncwarp();
  // top-k by repeated arg-max; among equal probabilities the lowest expert id wins
  float my_w = 0.f;
  int my_i = 0;
  float chosen_sum = 0.f;
  for (int k = 0; k < top_k; ++k) {
    float best = -1.f;
    int best_e = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = p[e];
      if (v > best) { best = v; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
    }
    if (lane == k) { my_w = best; my_i = best_e; }
    chosen_sum += best;
    if (lane == 0 && best_e < experts) p[best_e] = -2.f;   // not selectable again
    __syncwarp();
  }
  if (lane < top_k) {
    out_w[token * top_k + lane] = renorm ? __fdiv_rn(my_w, chosen_sum) : my_w;
    out_i[token * top_k + lane] = my_i;
  }
}

// ---------------------------------------------------------------------------------
// permutation: stable counting sort of the pairs by expert, one CTA, no workspace
// ---------------------------------------------------------------------------------
// Warp w owns a contiguous chunk of the pairs and walks it 32 pairs at a time.
// Pass 1 counts pairs per (warp, expert); a scan over warps and then over experts turns
// the counts into the first output position of every (warp, expert); pass 2 walks the
// chunks again and places every pair: position = running counter of (warp, expert) +
// number of lower lanes with the same expert in this step.
constexpr int kPermThreads = 1024;
constexpr int kPermWarps = kPermThreads / 32;

__global__ void __launch_bounds__(kPermThreads)
compute_permutation_kernel(int32_t* __restrict__ sorted_ids, int32_t* __restrict__ offsets,
                           const int32_t* __restrict__ topk_idx, int64_t pairs, int experts) {
  extern __shared__ int perm_smem[];       // [warps][experts] counters, then [experts] totals
  int* cnt = perm_smem;
  int* total = perm_smem + kPermWarps * experts;
  __shared__ int warp_sums[kPermWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kPermWarps * experts; i += kPermThreads) cnt[i] = 0;
  __syncthreads();
  const int64_t chunk = ((pairs + kPermWarps - 1) / kPermWarps + 31) & ~int64_t(31);
  const int64_t begin = warp * chunk;
  const int64_t end = begin + chunk < pairs ? begin + chunk : pairs;
  int* mine = cnt + warp * experts;
  for (int64_t base = begin; base < end; base += 32) {
    const int64_t i = base + lane;
    const int e = i < end ? topk_idx[i] : -1;
    const bool valid = e >= 0 && e < experts;
    const unsigned mask = __match_any_sync(0xffffffffu, valid ? e : experts + lane);
    if (valid && lane == __ffs(mask) - 1) mine[e] += __popc(mask);
    __syncwarp();
  }
  __syncthreads();
  // exclusive scan over warps for every expert
  for (int e = threadIdx.x; e < experts; e += kPermThreads) {
    int run = 0;
    for (int w = 0; w < kPermWarps; ++w) {
      const int c = cnt[w * experts + e];
      cnt[w * experts + e] = run;
      run += c;
    }
    total[e] = run;
  }
  __syncthreads();
  // exclusive scan of the totals over experts (experts <= 1024 = one element per thread)
  {
    const int v = threadIdx.x < experts ? total[threadIdx.x] : 0;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      const int ws = warp_sums[lane];
      int winc = ws;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += t;
      }
      warp_sums[lane] = winc - ws;
    }
    __syncthreads();
    const int excl = inc - v + warp_sums[warp];
    if (threadIdx.x < experts) {
      total[threadIdx.x] = excl;
      offsets[threadIdx.x] = excl;
      if (threadIdx.x == experts - 1) offsets[experts] = excl + v;
    }
  }
  __syncthreads();
  const int routed = offsets[experts];
  for (int i = threadIdx.x; i < kPermWarps * experts; i += kPermThreads) cnt[i] += total[i % experts];
  __syncthreads();
  for (int64_t base = begin; base < end; base += 32) {
    const int64_t i = base + lane;
    const int e = i < end ? topk_idx[i] : -1;
    const bool valid = e >= 0 && e < experts;
    const unsigned mask = __match_any_sync(0xffffffffu, valid ? e : experts + lane);
    if (valid) sorted_ids[mine[e] + __popc(mask & ((1u << lane) - 1u))] = static_cast<int32_t>(i);
    __syncwarp();
    if (valid && lane == __ffs(mask) - 1) mine[e] += __popc(mask);
    __syncwarp();
  }
  // pairs with an expert id out of range are dropped; their places at the end hold -1
  for (int64_t i = routed + threadIdx.x; i < pairs; i += kPermThreads) sorted_ids[i] = -1;
}

// ---------------------------------------------------------------------------------
// permute: gather token rows into expert order
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
permute_rows16_kernel(uint4* __restrict__ out, const uint4* __restrict__ in, const int32_t* __restrict__ ids,
                      int64_t pairs, int top_k, int64_t row_vec) {
  const int64_t total = pairs * row_vec;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = t / row_vec, c = t - r * row_vec;
    const int32_t pair = __ldg(ids + r);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (pair >= 0 && pair < pairs) v = __ldg(in + static_cast<int64_t>(pair / top_k) * row_vec + c);
    __stcs(out + t, v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
permute_rows_any_kernel(T* __restrict__ out, const T* __restrict__ in, const int32_t* __restrict__ ids,
                        int64_t pairs, int top_k, int64_t hidden) {
  const int64_t total = pairs * hidden;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = t / hidden, c = t - r * hidden;
    const int32_t pair = ids[r];
    out[t] = (pair >= 0 && pair < pairs) ? in[static_cast<int64_t>(pair / top_k) * hidden + c] : from_f32<T>(0.f);
  }
}

// Gather fused with the 1 x 128 quantizer: output row r holds the codes of token
// ids[r] / top_k; a lane owns 16 elements, 8 lanes a group (as quant_group128_kernel).
template <typename T, bool E5M2>
__global__ void __launch_bounds__(256)
permute_quant_kernel(uint8_t* __restrict__ out, float* __restrict__ scale, const T* __restrict__ in,
                     const int32_t* __restrict__ ids, int64_t pairs, int top_k, int64_t hidden, float qmax) {
  const int64_t segs_per_row = hidden / 16;
  const int64_t seg = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t r = seg / segs_per_row;
  const bool live = r < pairs;
  float v[16];
  bool have = false;
  if (live) {
    const int32_t pair = __ldg(ids + r);
    if (pair >= 0 && pair < pairs) {
      quantmath::Vec16<T>::load(in + static_cast<int64_t>(pair / top_k) * hidden + (seg - r * segs_per_row) * 16, v);
      have = true;
    }
  }
  if (!have) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
  }
  quantmath::quant_segment<T, E5M2>(out, scale, v, seg, live, qmax);
}

// ---------------------------------------------------------------------------------
// unpermute: out[token] = sum_k w[token, k] * permuted[row of pair (token, k)]
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
inverse_permutation_kernel(int32_t* __restrict__ inverse, const int32_t* __restrict__ ids, int64_t pairs) {
  const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= pairs) return;
  const int32_t pair = ids[r];
  if (pair >= 0 && pair < pairs) inverse[pair] = static_cast<int32_t>(r);
}

// A thread owns 8 consecutive columns (16 bytes of a 16-bit type) of one token; slots are
// added in slot order in fp32 and the row is written once.
template <typename T>
__global__ void __launch_bounds__(256)
unpermute_vec8_kernel(T* __restrict__ out, const T* __restrict__ permuted, const int32_t* __restrict__ inverse,
                      const float* __restrict__ weights, int64_t tokens, int top_k, int64_t hidden) {
  const int64_t row_vec = hidden / 8;
  const int64_t total = tokens * row_vec;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t token = t / row_vec, c = t - token * row_vec;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < top_k; ++k) {
      const int32_t prow = __ldg(inverse + token * top_k + k);
      if (prow < 0) continue;
      const float w = __ldg(weights + token * top_k + k);
      const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(permuted + static_cast<int64_t>(prow) * hidden) + c);
      const T* x = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(to_f32<T>(x[j]), w, acc[j]);
    }
    uint4 o;
    T* y = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = from_f32<T>(acc[j]);
    *(reinterpret_cast<uint4*>(out + token * hidden) + c) = o;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
unpermute_any_kernel(T* __restrict__ out, const T* __restrict__ permuted, const int32_t* __restrict__ inverse,
                     const float* __restrict__ weights, int64_t tokens, int top_k, int64_t hidden) {
  const int64_t total = tokens * hidden;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t token = t / hidden, c = t - token * hidden;
    float acc = 0.f;
    for (int k = 0; k < top_k; ++k) {
      const int32_t prow = inverse[token * top_k + k];
      if (prow < 0) continue;
      acc = fmaf(to_f32<T>(permuted[static_cast<int64_t>(prow) * hidden + c]), weights[token * top_k + k], acc);
    }
    out[t] = from_f32<T>(acc);
  }
}

// ---------------------------------------------------------------------------------
// SwiGLU
// ---------------------------------------------------------------------------------
__device__ __forceinline__ float silu(float x) { return __fdiv_rn(x, 1.0f + expf(-x)); }

// out[r, c] = silu(gate[r, c]) * up[r, c]; gate and up are rows of `in_stride` elements
// starting at gate0 / up0 (packed: gate0 = in, up0 = in + inter, stride 2 * inter).
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_kernel(T* __restrict__ out, const T* __restrict__ gate0, const T* __restrict__ up0, int64_t rows,
              int64_t inter, int64_t in_stride) {
  const int64_t total = rows * inter;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = t / inter, c = t - r * inter;
    out[t] = from_f32<T>(silu(to_f32<T>(gate0[r * in_stride + c])) * to_f32<T>(up0[r * in_stride + c]));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_vec16_kernel(T* __restrict__ out, const T* __restrict__ gate0, const T* __restrict__ up0, int64_t rows,
                    int64_t inter, int64_t in_stride) {
  const int64_t segs_per_row = inter / 16;
  const int64_t seg = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t r = seg / segs_per_row;
  if (r >= rows) return;
  const int64_t c = (seg - r * segs_per_row) * 16;
  float g[16], u[16];
  quantmath::Vec16<T>::load(gate0 + r * in_stride + c, g);
  quantmath::Vec16<T>::load(up0 + r * in_stride + c, u);
  T y[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) y[i] = from_f32<T>(silu(g[i]) * u[i]);
  uint4* dst = reinterpret_cast<uint4*>(out + r * inter + c);
  const uint4* src = reinterpret_cast<const uint4*>(y);
#pragma unroll
  for (int i = 0; i < static_cast<int>(sizeof(T)); ++i) dst[i] = src[i];
}

// Packed SwiGLU fused with the 1 x 128 quantizer: the activation is rounded to T exactly
// as the unfused kernel writes it, then quantized exactly as the quantizer reads it.
template <typename T, bool E5M2>
__global__ void __launch_bounds__(256)
swiglu_quant_kernel(uint8_t* __restrict__ out, float* __restrict__ scale, const T* __restrict__ in, int64_t rows,
                    int64_t inter, float qmax) {
  const int64_t segs_per_row = inter / 16;
  const int64_t seg = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t r = seg / segs_per_row;
  const bool live = r < rows;
  float v[16];
  if (live) {
    const int64_t c = (seg - r * segs_per_row) * 16;
    float g[16], u[16];
    quantmath::Vec16<T>::load(in + r * 2 * inter + c, g);
    quantmath::Vec16<T>::load(in + r * 2 * inter + inter + c, u);
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = to_f32<T>(from_f32<T>(silu(g[i]) * u[i]));
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
  }
  quantmath::quant_segment<T, E5M2>(out, scale, v, seg, live, qmax);
}

inline unsigned grid_for(int64_t work_items, int threads = 256) {
  const int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  return static_cast<unsigned>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

ks_status_t check_pairs(const char* where, int64_t tokens, int top_k, int64_t* pairs) {
  if (tokens > 0 && top_k > 0 && tokens > INT32_MAX / top_k)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, std::string(where) + ": num_tokens*top_k exceeds int32 limit");
  *pairs = tokens * static_cast<int64_t>(top_k);
  return KS_SUCCESS;
}

}  // namespace
}  // namespace ksb

using namespace ksb;

namespace {
template <typename T>
void launch_swiglu(void* out, const void* gate, const void* up, int64_t rows, int64_t inter, int64_t stride,
                   cudaStream_t s) {
  const bool vec = !std::is_same<T, float>::value && inter % 16 == 0 && stride % 8 == 0 && aligned16(out) &&
                   aligned16(gate) && aligned16(up);
  if (vec) {
    const int64_t segs = rows * (inter / 16);
    swiglu_vec16_kernel<T><<<static_cast<unsigned>((segs + 255) / 256), 256, 0, s>>>(
        static_cast<T*>(out), static_cast<const T*>(gate), static_cast<const T*>(up), rows, inter, stride);
  } else {
    swiglu_kernel<T><<<grid_for(rows * inter), 256, 0, s>>>(static_cast<T*>(out), static_cast<const T*>(gate),
                                                            static_cast<const T*>(up), rows, inter, stride);
  }
}

ks_status_t swiglu_common(const char* where, void* out, const void* gate, const void* up, int64_t rows,
                          int64_t inter, int64_t stride, ks_dtype_t dtype, ks_stream_t stream) {
  if (rows < 0 || inter <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, std::string(where) + ": bad shape");
  if (!is_float3(dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, std::string(where) + ": unsupported dtype");
  if (rows == 0) return KS_SUCCESS;
  if (rows * (inter / 16 + 1) / 256 > 2147483647LL)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, std::string(where) + ": grid exceeds CUDA grid limits");
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  if (dtype == KS_DTYPE_F32) launch_swiglu<float>(out, gate, up, rows, inter, stride, s);
  else if (dtype == KS_DTYPE_F16) launch_swiglu<__half>(out, gate, up, rows, inter, stride, s);
  else launch_swiglu<__nv_bfloat16>(out, gate, up, rows, inter, stride, s);
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}
}  // namespace

extern "C" {

ks_status_t ks_moe_gate_softmax_topk(float* out_weights, int32_t* out_indices, const void* logits,
                                     int64_t num_tokens, int num_experts, int top_k, int renormalize,
                                     ks_dtype_t dtype, ks_stream_t stream) {
  const char* where = "ks_moe_gate_softmax_topk";
  KSB_REQUIRE_PTR(out_weights);
  KSB_REQUIRE_PTR(out_indices);
  KSB_REQUIRE_PTR(logits);
  if (num_tokens < 0 || num_experts <= 0 || top_k <= 0 || top_k > num_experts)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_gate_softmax_topk: bad shape");
  if (num_experts > kMaxExperts || top_k > kMaxTopK)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_moe_gate_softmax_topk: at most 1024 experts and top_k 32");
  if (!is_float3(dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_moe_gate_softmax_topk: unsupported dtype");
  if (num_tokens == 0) return KS_SUCCESS;
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const int warps = num_experts <= 256 ? 8 : 2;   // 8 KB of shared memory per CTA either way
  const unsigned blocks = static_cast<unsigned>((num_tokens + warps - 1) / warps);
  const size_t smem = static_cast<size_t>(warps) * num_experts * sizeof(float);
#define KSB_GATE(T)                                                                                          \
  gate_softmax_topk_kernel<T><<<blocks, warps * 32, smem, s>>>(out_weights, out_indices,                     \
                                                               static_cast<const T*>(logits), num_tokens,   \
                                                               num_experts, top_k, renormalize)
  if (dtype == KS_DTYPE_F32) KSB_GATE(float);
  else if (dtype == KS_DTYPE_F16) KSB_GATE(__half);
  else KSB_GATE(__nv_bfloat16);
#undef KSB_GATE
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}

ks_status_t ks_moe_compute_permutation(int32_t* sorted_token_ids, int32_t* expert_offsets,
                                       const int32_t* topk_indices, int64_t num_tokens, int num_experts,
                                       int top_k, ks_stream_t stream) {
  const char* where = "ks_moe_compute_permutation";
  KSB_REQUIRE_PTR(sorted_token_ids);
  KSB_REQUIRE_PTR(expert_offsets);
  KSB_REQUIRE_PTR(topk_indices);
  if (num_tokens < 0 || num_experts <= 0 || top_k <= 0)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_compute_permutation: bad shape");
  if (num_experts > kMaxExperts)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_moe_compute_permutation: at most 1024 experts");
  int64_t pairs = 0;
  ks_status_t st = check_pairs(where, num_tokens, top_k, &pairs);
  if (st != KS_SUCCESS) return st;
  st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const size_t smem = (static_cast<size_t>(kPermWarps) + 1) * num_experts * sizeof(int);
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(compute_permutation_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>((kPermWarps + 1) * kMaxExperts * sizeof(int)));
    if (e != cudaSuccess) return cuda_status(e, where);
    attr_done[dev] = true;
  }
  compute_permutation_kernel<<<1, kPermThreads, smem, s>>>(sorted_token_ids, expert_offsets, topk_indices, pairs,
                                                           num_experts);
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}

ks_status_t ks_moe_permute(void* permuted, const void* input, const int32_t* sorted_token_ids, int64_t num_tokens,
                           int top_k, int64_t hidden, ks_dtype_t dtype, ks_stream_t stream) {
  const char* where = "ks_moe_permute";
  KSB_REQUIRE_PTR(permuted);
  KSB_REQUIRE_PTR(input);
  KSB_REQUIRE_PTR(sorted_token_ids);
  if (num_tokens < 0 || top_k <= 0 || hidden <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_permute: bad shape");
  if (!is_float3(dtype) && !is_fp8(dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_moe_permute: unsupported dtype");
  int64_t pairs = 0;
  ks_status_t st = check_pairs(where, num_tokens, top_k, &pairs);
  if (st != KS_SUCCESS) return st;
  if (pairs == 0) return KS_SUCCESS;
  st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const int64_t elt = dtype == KS_DTYPE_F32 ? 4 : (is_fp8(dtype) ? 1 : 2);
  const int64_t row_bytes = hidden * elt;
  if (row_bytes % 16 == 0 && aligned16(permuted) && aligned16(input)) {
    const int64_t row_vec = row_bytes / 16;
    permute_rows16_kernel<<<grid_for(pairs * row_vec), 256, 0, s>>>(
        static_cast<uint4*>(permuted), static_cast<const uint4*>(input), sorted_token_ids, pairs, top_k, row_vec);
  } else if (elt == 4) {
    permute_rows_any_kernel<float><<<grid_for(pairs * hidden), 256, 0, s>>>(
        static_cast<float*>(permuted), static_cast<const float*>(input), sorted_token_ids, pairs, top_k, hidden);
  } else if (elt == 2) {
    permute_rows_any_kernel<__half><<<grid_for(pairs * hidden), 256, 0, s>>>(
        static_cast<__half*>(permuted), static_cast<const __half*>(input), sorted_token_ids, pairs, top_k, hidden);
  } else {
    permute_rows_any_kernel<__nv_fp8_e4m3><<<grid_for(pairs * hidden), 256, 0, s>>>(
        static_cast<__nv_fp8_e4m3*>(permuted), static_cast<const __nv_fp8_e4m3*>(input), sorted_token_ids, pairs,
        top_k, hidden);
  }
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}

ks_status_t ks_moe_permute_quant_fp8(void* out_fp8, float* out_scale, const void* input,
                                     const int32_t* sorted_token_ids, int64_t num_tokens, int top_k,
                                     int64_t hidden, ks_dtype_t in_dtype, ks_dtype_t fp8_dtype,
                                     ks_stream_t stream) {
  const char* where = "ks_moe_permute_quant_fp8";
  KSB_REQUIRE_PTR(out_fp8);
  KSB_REQUIRE_PTR(out_scale);
  KSB_REQUIRE_PTR(input);
  KSB_REQUIRE_PTR(sorted_token_ids);
  if (num_tokens < 0 || top_k <= 0 || hidden <= 0)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_permute_quant_fp8: bad shape");
  if (hidden % 128 != 0 || !aligned16(out_fp8) || !aligned16(input))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE,
             "ks_moe_permute_quant_fp8: hidden must be a multiple of 128 and the buffers 16-byte aligned");
  if (!is_fp8(fp8_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_moe_permute_quant_fp8: fp8_dtype must be e4m3 or e5m2");
  if (!is_float3(in_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_moe_permute_quant_fp8: unsupported dtype");
  int64_t pairs = 0;
  ks_status_t st = check_pairs(where, num_tokens, top_k, &pairs);
  if (st != KS_SUCCESS) return st;
  if (pairs == 0) return KS_SUCCESS;
  st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const int64_t segs = pairs * (hidden / 16);
  if ((segs + 255) / 256 > 2147483647LL)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_moe_permute_quant_fp8: grid exceeds CUDA grid limits");
  const unsigned blocks = static_cast<unsigned>((segs + 255) / 256);
  const bool e5 = fp8_dtype == KS_DTYPE_F8E5M2;
  uint8_t* o = static_cast<uint8_t*>(out_fp8);
#define KSB_PQ(T)                                                                                               \
  do {                                                                                                          \
    if (e5) permute_quant_kernel<T, true><<<blocks, 256, 0, s>>>(o, out_scale, static_cast<const T*>(input),   \
                                                                 sorted_token_ids, pairs, top_k, hidden, 57344.0f); \
    else permute_quant_kernel<T, false><<<blocks, 256, 0, s>>>(o, out_scale, static_cast<const T*>(input),     \
                                                               sorted_token_ids, pairs, top_k, hidden, 448.0f); \
  } while (0)
  if (in_dtype == KS_DTYPE_F32) KSB_PQ(float);
  else if (in_dtype == KS_DTYPE_F16) KSB_PQ(__half);
  else KSB_PQ(__nv_bfloat16);
#undef KSB_PQ
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}

ks_status_t ks_moe_unpermute(void* out, const void* permuted, const int32_t* sorted_token_ids,
                             const float* routing_weights, int64_t num_tokens, int top_k, int64_t hidden,
                             ks_dtype_t dtype, ks_stream_t stream) {
  const char* where = "ks_moe_unpermute";
  KSB_REQUIRE_PTR(out);
  KSB_REQUIRE_PTR(permuted);
  KSB_REQUIRE_PTR(sorted_token_ids);
  KSB_REQUIRE_PTR(routing_weights);
  if (num_tokens < 0 || top_k <= 0 || hidden <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_unpermute: bad shape");
  if (!is_float3(dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_moe_unpermute: unsupported dtype");
  int64_t pairs = 0;
  ks_status_t st = check_pairs(where, num_tokens, top_k, &pairs);
  if (st != KS_SUCCESS) return st;
  if (pairs == 0) return KS_SUCCESS;
  st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  // inverse[pair] = row of the pair after the sort; -1 for dropped pairs. Stream-ordered
  // library workspace: allocated when the stream first needs it (or needs more), never freed
  // or synchronised per call.
  int32_t* inverse = static_cast<int32_t*>(sm100::stream_scratch(s, static_cast<size_t>(pairs) * sizeof(int32_t), 4));
  if (inverse == nullptr) KSB_FAIL(KS_ERROR_OUT_OF_MEMORY, "ks_moe_unpermute: workspace allocation failed");
  cudaError_t e = cudaMemsetAsync(inverse, 0xFF, static_cast<size_t>(pairs) * sizeof(int32_t), s);
  if (e != cudaSuccess) return cuda_status(e, where);
  inverse_permutation_kernel<<<static_cast<unsigned>((pairs + 255) / 256), 256, 0, s>>>(inverse, sorted_token_ids, pairs);
  const bool vec = dtype != KS_DTYPE_F32 && hidden % 8 == 0 && aligned16(out) && aligned16(permuted);
  if (dtype == KS_DTYPE_F32) {
    unpermute_any_kernel<float><<<grid_for(num_tokens * hidden), 256, 0, s>>>(
        static_cast<float*>(out), static_cast<const float*>(permuted), inverse, routing_weights, num_tokens, top_k, hidden);
  } else if (dtype == KS_DTYPE_F16) {
    if (vec) unpermute_vec8_kernel<__half><<<grid_for(num_tokens * (hidden / 8)), 256, 0, s>>>(
        static_cast<__half*>(out), static_cast<const __half*>(permuted), inverse, routing_weights, num_tokens, top_k, hidden);
    else unpermute_any_kernel<__half><<<grid_for(num_tokens * hidden), 256, 0, s>>>(
        static_cast<__half*>(out), static_cast<const __half*>(permuted), inverse, routing_weights, num_tokens, top_k, hidden);
  } else {
    if (vec) unpermute_vec8_kernel<__nv_bfloat16><<<grid_for(num_tokens * (hidden / 8)), 256, 0, s>>>(
        static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(permuted), inverse, routing_weights,
        num_tokens, top_k, hidden);
    else unpermute_any_kernel<__nv_bfloat16><<<grid_for(num_tokens * hidden), 256, 0, s>>>(
        static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(permuted), inverse, routing_weights,
        num_tokens, top_k, hidden);
  }
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}

ks_status_t ks_swiglu(void* out, const void* gate, const void* up, int64_t rows, int64_t inter, ks_dtype_t dtype,
                      ks_stream_t stream) {
  KSB_REQUIRE_PTR(out);
  KSB_REQUIRE_PTR(gate);
  KSB_REQUIRE_PTR(up);
  return swiglu_common("ks_swiglu", out, gate, up, rows, inter, inter, dtype, stream);
}

ks_status_t ks_swiglu_packed(void* out, const void* input, int64_t rows, int64_t inter, ks_dtype_t dtype,
                             ks_stream_t stream) {
  KSB_REQUIRE_PTR(out);
  KSB_REQUIRE_PTR(input);
  if (inter <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_swiglu_packed: bad shape");
  const int64_t elt = dtype == KS_DTYPE_F32 ? 4 : 2;
  const void* up = static_cast<const uint8_t*>(input) + inter * elt;
  return swiglu_common("ks_swiglu_packed", out, input, up, rows, inter, 2 * inter, dtype, stream);
}

ks_status_t ks_swiglu_packed_quant_fp8(void* out_fp8, float* out_scale, const void* input, int64_t rows,
                                       int64_t inter, ks_dtype_t in_dtype, ks_dtype_t fp8_dtype,
                                       ks_stream_t stream) {
  const char* where = "ks_swiglu_packed_quant_fp8";
  KSB_REQUIRE_PTR(out_fp8);
  KSB_REQUIRE_PTR(out_scale);
  KSB_REQUIRE_PTR(input);
  if (rows < 0 || inter <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_swiglu_packed_quant_fp8: bad shape");
  if (inter % 128 != 0 || !aligned16(out_fp8) || !aligned16(input))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE,
             "ks_swiglu_packed_quant_fp8: inter must be a multiple of 128 and the buffers 16-byte aligned");
  if (!is_fp8(fp8_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_swiglu_packed_quant_fp8: fp8_dtype must be e4m3 or e5m2");
  if (in_dtype != KS_DTYPE_F16 && in_dtype != KS_DTYPE_BF16)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_swiglu_packed_quant_fp8: input must be f16 or bf16");
  if (rows == 0) return KS_SUCCESS;
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const int64_t segs = rows * (inter / 16);
  if ((segs + 255) / 256 > 2147483647LL)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_swiglu_packed_quant_fp8: grid exceeds CUDA grid limits");
  const unsigned blocks = static_cast<unsigned>((segs + 255) / 256);
  const bool e5 = fp8_dtype == KS_DTYPE_F8E5M2;
  uint8_t* o = static_cast<uint8_t*>(out_fp8);
#define KSB_SQ(T)                                                                                                    \
  do {                                                                                                               \
    if (e5) swiglu_quant_kernel<T, true><<<blocks, 256, 0, s>>>(o, out_scale, static_cast<const T*>(input), rows,   \
                                                                inter, 57344.0f);                                    \
    else swiglu_quant_kernel<T, false><<<blocks, 256, 0, s>>>(o, out_scale, static_cast<const T*>(input), rows,     \
                                                              inter, 448.0f);                                        \
  } while (0)
  if (in_dtype == KS_DTYPE_F16) KSB_SQ(__half);
  else KSB_SQ(__nv_bfloat16);
#undef KSB_SQ
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}

}  // extern "C"
