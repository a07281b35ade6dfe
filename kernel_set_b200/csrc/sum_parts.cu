// Sum of the partial outputs of a K-split (row-parallel) GEMM, written to one or several
// destinations: the second half of a reduce-scatter / all-reduce that the GEMM kernel's
// scattered epilogue started (ks_gemm_fp8_blockwise_scatter writes every rank's partial of a
// row block into the memory of the rank that owns the block).
//
// The reference project has no multi-GPU code; this step stands where a row-parallel layer
// calls an all-reduce on the GEMM's output.
//
// parts [num_parts, rows, n] (fp32 / bf16 / f16) are added in part order in fp32 and rounded
// once to `out_dtype`; the result goes to every pointer of `dsts` (this GPU's copy and, for
// an all-gather by peer stores, the other GPUs'). HBM-bound on the reads when the
// destinations are local, NVLink-bound on the writes otherwise: algorithmic bytes
// num_parts * rows * n * sizeof(part) read, num_dsts * rows * n * sizeof(out) written.
#include "common.cuh"
#include "kernel_set/gemm.h"

namespace ksb {
namespace {

constexpr int kMaxDsts = 8;
struct Dsts {
  void* p[kMaxDsts];
};

template <typename PT> struct Load8;   // eight consecutive elements as fp32
template <> struct Load8<float> {
  __device__ static void run(const float* p, float (&v)[8]) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(p));
    const float4 b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct Load8<__nv_bfloat16> {
  __device__ static void run(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 a = __ldcs(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
template <> struct Load8<__half> {
  __device__ static void run(const __half* p, float (&v)[8]) {
    const uint4 a = __ldcs(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};

template <typename OT>
__device__ __forceinline__ void store8(OT* p, const float (&v)[8]) {
  if constexpr (sizeof(OT) == 4) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    OT o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = from_f32<OT>(v[i]);
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(o);
  }
}

template <typename PT, typename OT>
__global__ void __launch_bounds__(256)
sum_parts_kernel(const Dsts dsts, int num_dsts, const PT* __restrict__ parts, int num_parts, int64_t elems) {
  const int64_t chunks = elems >> 3;
  for (int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < chunks;
       c += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc[8];
    Load8<PT>::run(parts + c * 8, acc);
    for (int q = 1; q < num_parts; ++q) {
      float v[8];
      Load8<PT>::run(parts + static_cast<int64_t>(q) * elems + c * 8, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i];
    }
    for (int d = 0; d < num_dsts; ++d) store8<OT>(static_cast<OT*>(dsts.p[d]) + c * 8, acc);
  }
}

template <typename PT, typename OT>
void launch(const Dsts& dsts, int num_dsts, const void* parts, int num_parts, int64_t elems, cudaStream_t s) {
  int64_t blocks = ((elems >> 3) + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;   // grid-stride beyond this
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  sum_parts_kernel<PT, OT><<<static_cast<unsigned>(blocks), 256, 0, s>>>(dsts, num_dsts, static_cast<const PT*>(parts),
                                                                        num_parts, elems);
}

template <typename PT>
void launch_out(ks_dtype_t out_dtype, const Dsts& dsts, int num_dsts, const void* parts, int num_parts, int64_t elems,
                cudaStream_t s) {
  if (out_dtype == KS_DTYPE_F32) launch<PT, float>(dsts, num_dsts, parts, num_parts, elems, s);
  else if (out_dtype == KS_DTYPE_F16) launch<PT, __half>(dsts, num_dsts, parts, num_parts, elems, s);
  else launch<PT, __nv_bfloat16>(dsts, num_dsts, parts, num_parts, elems, s);
}

}  // namespace
}  // namespace ksb

extern "C" {

ks_status_t ks_sum_parts(void* const* dsts, int num_dsts, const void* parts, int num_parts, int64_t rows, int64_t n,
                         ks_dtype_t part_dtype, ks_dtype_t out_dtype, ks_stream_t stream) {
  using namespace ksb;
  KSB_REQUIRE_PTR(dsts);
  KSB_REQUIRE_PTR(parts);
  if (num_dsts < 1 || num_dsts > kMaxDsts || num_parts < 1)
    KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_sum_parts: between 1 and 8 destinations, at least one part");
  if (rows < 0 || n <= 0) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_sum_parts: bad shape");
  if (!is_float3(part_dtype) || !is_float3(out_dtype)) KSB_FAIL(KS_ERROR_UNSUPPORTED_DTYPE, "ks_sum_parts: unsupported dtype");
  if ((rows * n) % 8 != 0) KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, "ks_sum_parts: rows * n must be a multiple of 8");
  Dsts d;
  for (int i = 0; i < kMaxDsts; ++i) d.p[i] = nullptr;
  for (int i = 0; i < num_dsts; ++i) {
    if (dsts[i] == nullptr || !aligned16(dsts[i])) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_sum_parts: destinations must be non-null and 16-byte aligned");
    d.p[i] = dsts[i];
  }
  if (!aligned16(parts)) KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "ks_sum_parts: parts must be 16-byte aligned");
  ks_status_t st = require_sm100("ks_sum_parts");
  if (st != KS_SUCCESS) return st;
  if (rows == 0) return KS_SUCCESS;
  cudaStream_t s = as_stream(stream);
  const int64_t elems = rows * n;
  if (part_dtype == KS_DTYPE_F32) launch_out<float>(out_dtype, d, num_dsts, parts, num_parts, elems, s);
  else if (part_dtype == KS_DTYPE_F16) launch_out<__half>(out_dtype, d, num_dsts, parts, num_parts, elems, s);
  else launch_out<__nv_bfloat16>(out_dtype, d, num_dsts, parts, num_parts, elems, s);
  KSB_CHECK_LAUNCH("ks_sum_parts");
  return KS_SUCCESS;
}

}  // extern "C"
