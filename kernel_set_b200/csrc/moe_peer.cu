// Dispatch and combine of an expert-parallel MoE layer written straight into the other
// ranks' memory, instead of all-to-all collectives with a regrouping pass on either side.
//
// The reference project has no multi-GPU code; these steps stand where an expert-parallel
// layer calls all-to-all before the first and after the second expert GEMM.
//
// Experts are split contiguously over the ranks (expert e lives on rank e / per). Every rank
// knows the whole count matrix counts[s][e] (rows rank s routes to expert e, all-gathered on
// the device), so every rank can compute by itself where each of its rows lands:
//   * a receiving rank holds its rows expert-major, and inside an expert by source rank:
//     row of (expert el, source s, i-th row) = sum over el' < el of all sources' counts
//                                            + sum over s' < s of counts[s'][el] + i;
//   * the row goes back to position expert_offsets_s[e] + i of the source's sorted order.
// ks_moe_dispatch_plan turns the count matrix into those bases; ks_moe_permute_quant_fp8_scatter
// is the gather + 1 x 128 quantizer of ks_moe_permute_quant_fp8 with the row written to the
// destination rank's buffer at its final, expert-major position (peer stores of 16 bytes, the
// row's scales beside it), so the grouped GEMM runs on the received buffer as it is;
// ks_moe_scatter_rows sends the second GEMM's rows back to where the source's unpermute
// expects them. No kernel here waits on another GPU: the caller puts a cross-rank barrier
// between the stores and their use. All three are HBM / NVLink-bound row kernels:
// algorithmic bytes per row hidden * (in + 1) + hidden / 32 (dispatch), 2 * hidden * elt (combine).
#include "common.cuh"
#include "kernel_set/moe.h"
#include "quant_math.cuh"

namespace ksb {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxPlanExperts = 1024;

struct PeerPtrs {
  void* p[kMaxRanks];
};

// one CTA; counts [world, e_pad] with e_pad = world * per
__global__ void __launch_bounds__(256)
dispatch_plan_kernel(int32_t* __restrict__ dst_base, int32_t* __restrict__ local_offsets,
                     int32_t* __restrict__ seg_start, int32_t* __restrict__ ret_base,
                     const int32_t* __restrict__ counts, int world, int rank, int per) {
  __shared__ int32_t col_total[kMaxPlanExperts];   // rows of expert e over all sources
  const int e_pad = world * per;
  for (int e = threadIdx.x; e < e_pad; e += blockDim.x) {
    int32_t t = 0;
    for (int s = 0; s < world; ++s) t += max(counts[s * e_pad + e], 0);
    col_total[e] = t;
  }
  __syncthreads();
  // where my rows of expert e land on rank e / per
  for (int e = threadIdx.x; e < e_pad; e += blockDim.x) {
    const int d = e / per, el = e - d * per;
    int32_t base = 0;
    for (int j = 0; j < el; ++j) base += col_total[d * per + j];
    for (int s = 0; s < rank; ++s) base += max(counts[s * e_pad + e], 0);
    dst_base[e] = base;
  }
  // what I receive: expert offsets, the (expert, source) segments, and where they go back
  if (threadIdx.x == 0) {
    int32_t run = 0;
    for (int el = 0; el < per; ++el) {
      local_offsets[el] = run;
      for (int s = 0; s < world; ++s) {
        seg_start[el * world + s] = run;
        run += max(counts[s * e_pad + rank * per + el], 0);
      }
    }
    local_offsets[per] = run;
    seg_start[per * world] = run;
  }
  for (int j = threadIdx.x; j < per * world; j += blockDim.x) {
    const int el = j / world, s = j - el * world;
    const int e = rank * per + el;
    int32_t off = 0;   // expert_offsets of rank s at expert e
    for (int e2 = 0; e2 < e; ++e2) off += max(counts[s * e_pad + e2], 0);
    ret_base[j] = off;
  }
}

// last index i in [0, n) with a[i] <= v (a non-decreasing, a[0] <= v)
__device__ __forceinline__ int upper_index(const int32_t* __restrict__ a, int n, int32_t v) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (__ldg(a + mid) <= v) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Gather fused with the 1 x 128 quantizer (as permute_quant_kernel), the row written to the
// destination rank: sorted row r belongs to expert e (offsets[e] <= r < offsets[e+1]) and goes
// to row dst_base[e] + r - offsets[e] of rank e / per.
template <typename T, bool E5M2>
__global__ void __launch_bounds__(256)
permute_quant_scatter_kernel(const PeerPtrs dst_q, const PeerPtrs dst_s, const int32_t* __restrict__ dst_base,
                             const int32_t* __restrict__ offsets, int num_experts, int per,
                             const T* __restrict__ in, const int32_t* __restrict__ ids, int64_t pairs, int top_k,
                             int64_t hidden, int64_t capacity, float qmax) {
  const int64_t segs_per_row = hidden / 16;
  const int64_t seg = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t r = seg / segs_per_row;
  const bool live = r < pairs;
  float v[16];
  bool have = false;
  int64_t dst_row = 0;
  int d = 0;
  if (live) {
    const int32_t pair = __ldg(ids + r);
    if (pair >= 0 && pair < pairs) {
      quantmath::Vec16<T>::load(in + static_cast<int64_t>(pair / top_k) * hidden + (seg - r * segs_per_row) * 16, v);
      have = true;
    }
    const int e = upper_index(offsets, num_experts, static_cast<int32_t>(r));
    d = e / per;
    dst_row = static_cast<int64_t>(__ldg(dst_base + e)) + (r - __ldg(offsets + e));
  }
  if (!have) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
  }
  float sc;
  const uint4 codes = quantmath::quant_segment_codes<E5M2>(v, qmax, &sc);
  if (!live || dst_row < 0 || dst_row >= capacity) return;
  const int64_t in_row = seg - r * segs_per_row;
  uint8_t* q = static_cast<uint8_t*>(dst_q.p[d]) + dst_row * hidden + in_row * 16;
  *reinterpret_cast<uint4*>(q) = codes;
  if ((threadIdx.x & 7) == 0) static_cast<float*>(dst_s.p[d])[dst_row * (hidden / 128) + (in_row >> 3)] = sc;
}

// Row i of `src` (i < seg_start[segments]) lies in segment j = (expert el, source s = j % world)
// and goes to row ret_base[j] + i - seg_start[j] of rank s. A thread moves 16 bytes.
__global__ void __launch_bounds__(256)
scatter_rows_kernel(const PeerPtrs dst, const uint4* __restrict__ src, const int32_t* __restrict__ seg_start,
                    const int32_t* __restrict__ ret_base, int segments, int world, int64_t row_vec,
                    int64_t capacity_rows, int64_t dst_rows) {
  const int64_t total_rows = min(static_cast<int64_t>(__ldg(seg_start + segments)), capacity_rows);
  const int64_t total = total_rows * row_vec;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t i = t / row_vec, c = t - i * row_vec;
    const int j = upper_index(seg_start, segments, static_cast<int32_t>(i));
    const int s = j % world;
    const int64_t row = static_cast<int64_t>(__ldg(ret_base + j)) + (i - __ldg(seg_start + j));
    if (row < 0 || row >= dst_rows) continue;
    static_cast<uint4*>(dst.p[s])[row * row_vec + c] = __ldg(src + t);
  }
}

}  // namespace
}  // namespace ksb

extern "C" {

ks_status_t ks_moe_dispatch_plan(int32_t* dst_base, int32_t* local_offsets, int32_t* seg_start, int32_t* ret_base,
                                 const int32_t* counts, int world, int rank, int experts_per_rank,
                                 ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_moe_dispatch_plan";
  KSB_REQUIRE_PTR(dst_base);
  KSB_REQUIRE_PTR(local_offsets);
  KSB_REQUIRE_PTR(seg_start);
  KSB_REQUIRE_PTR(ret_base);
  KSB_REQUIRE_PTR(counts);
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || experts_per_rank < 1)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_dispatch_plan: 1..8 ranks, 0 <= rank < world, at least one expert per rank");
  if (world * experts_per_rank > kMaxPlanExperts)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_moe_dispatch_plan: at most 1024 experts");
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  dispatch_plan_kernel<<<1, 256, 0, as_stream(stream)>>>(dst_base, local_offsets, seg_start, ret_base, counts, world, rank,
                                                         experts_per_rank);
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}

ks_status_t ks_moe_permute_quant_fp8_scatter(void* const* dst_fp8, float* const* dst_scale, int world,
                                             int64_t capacity_rows, const int32_t* dst_base,
                                             const int32_t* expert_offsets, int num_experts, int experts_per_rank,
                                             const void* input, const int32_t* sorted_token_ids,
                                             int64_t num_tokens, int top_k, int64_t hidden, ks_dtype_t in_dtype,
                                             ks_dtype_t fp8_dtype, ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_moe_permute_quant_fp8_scatter";
  KSB_REQUIRE_PTR(dst_fp8);
  KSB_REQUIRE_PTR(dst_scale);
  KSB_REQUIRE_PTR(dst_base);
  KSB_REQUIRE_PTR(expert_offsets);
  KSB_REQUIRE_PTR(input);
  KSB_REQUIRE_PTR(sorted_token_ids);
  if (world < 1 || world > kMaxRanks || num_experts < 1 || experts_per_rank < 1 ||
      (num_experts + experts_per_rank - 1) / experts_per_rank > world)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_permute_quant_fp8_scatter: bad rank / expert counts");
  if (num_tokens < 0 || top_k <= 0 || hidden <= 0 || capacity_rows <= 0)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_permute_quant_fp8_scatter: bad shape");
  if (hidden % 128 != 0 || !aligned16(input))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_moe_permute_quant_fp8_scatter: hidden must be a multiple of 128 and the input 16-byte aligned");
  if (!is_fp8(fp8_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_moe_permute_quant_fp8_scatter: fp8_dtype must be e4m3 or e5m2");
  if (!is_float3(in_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_moe_permute_quant_fp8_scatter: unsupported dtype");
  PeerPtrs q, sc;
  for (int i = 0; i < kMaxRanks; ++i) { q.p[i] = nullptr; sc.p[i] = nullptr; }
  for (int i = 0; i < world; ++i) {
    if (dst_fp8[i] == nullptr || dst_scale[i] == nullptr || !aligned16(dst_fp8[i]))
      KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_permute_quant_fp8_scatter: destinations must be non-null and 16-byte aligned");
    q.p[i] = dst_fp8[i];
    sc.p[i] = dst_scale[i];
  }
  const int64_t pairs = num_tokens * top_k;
  if (pairs > 2147483647LL) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_moe_permute_quant_fp8_scatter: too many rows");
  if (pairs == 0) return KS_SUCCESS;
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  cudaStream_t s = as_stream(stream);
  const int64_t segs = pairs * (hidden / 16);
  if ((segs + 255) / 256 > 2147483647LL) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_moe_permute_quant_fp8_scatter: grid exceeds CUDA grid limits");
  const unsigned blocks = static_cast<unsigned>((segs + 255) / 256);
  const bool e5 = fp8_dtype == KS_DTYPE_F8E5M2;
#define KSB_PQS(T)                                                                                                   \
  do {                                                                                                               \
    if (e5) permute_quant_scatter_kernel<T, true><<<blocks, 256, 0, s>>>(q, sc, dst_base, expert_offsets, num_experts, \
        experts_per_rank, static_cast<const T*>(input), sorted_token_ids, pairs, top_k, hidden, capacity_rows, 57344.0f); \
    else permute_quant_scatter_kernel<T, false><<<blocks, 256, 0, s>>>(q, sc, dst_base, expert_offsets, num_experts,  \
        experts_per_rank, static_cast<const T*>(input), sorted_token_ids, pairs, top_k, hidden, capacity_rows, 448.0f);  \
  } while (0)
  if (in_dtype == KS_DTYPE_F32) KSB_PQS(float);
  else if (in_dtype == KS_DTYPE_F16) KSB_PQS(__half);
  else KSB_PQS(__nv_bfloat16);
#undef KSB_PQS
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}

ks_status_t ks_moe_scatter_rows(void* const* dst, int world, int64_t dst_rows, const void* src,
                                int64_t capacity_rows, const int32_t* seg_start, const int32_t* ret_base,
                                int segments, int64_t hidden, ks_dtype_t dtype, ks_stream_t stream) {
  using namespace ksb;
  const char* where = "ks_moe_scatter_rows";
  KSB_REQUIRE_PTR(dst);
  KSB_REQUIRE_PTR(src);
  KSB_REQUIRE_PTR(seg_start);
  KSB_REQUIRE_PTR(ret_base);
  if (world < 1 || world > kMaxRanks || segments < 1 || segments % world != 0)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_scatter_rows: segments must be (experts of this rank) x (1..8 ranks)");
  if (dst_rows < 0 || capacity_rows < 0 || hidden <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_scatter_rows: bad shape");
  if (!is_float3(dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_moe_scatter_rows: unsupported dtype");
  const int64_t row_bytes = hidden * (dtype == KS_DTYPE_F32 ? 4 : 2);
  if (row_bytes % 16 != 0 || !aligned16(src))
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_moe_scatter_rows: rows must be multiples of 16 bytes and 16-byte aligned");
  PeerPtrs d;
  for (int i = 0; i < kMaxRanks; ++i) d.p[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    if (dst[i] == nullptr || !aligned16(dst[i]))
      KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_moe_scatter_rows: destinations must be non-null and 16-byte aligned");
    d.p[i] = dst[i];
  }
  if (capacity_rows == 0) return KS_SUCCESS;
  ks_status_t st = require_sm100(where);
  if (st != KS_SUCCESS) return st;
  const int64_t row_vec = row_bytes / 16;
  int64_t blocks = (capacity_rows * row_vec + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;   // grid-stride beyond this
  if (blocks > cap) blocks = cap;
  scatter_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
      d, static_cast<const uint4*>(src), seg_start, ret_base, segments, world, row_vec, capacity_rows, dst_rows);
  KSB_CHECK_LAUNCH(where);
  return KS_SUCCESS;
}

}  // extern "C"
