// FP8 block-scaled GEMM on CTA pairs (tcgen05 cta_group::2), dense problems only.
//
// Same arithmetic as sm100_fp8_gemm.cu (reference algebra: kernels/src/gemm/
// gemm_fp8_blockwise.cu:107-150). Why a second kernel: a single CTA feeding
// M128 x N256 MMAs reads 48 KB of operands from its shared memory per K-block,
// and the tensor core's operand path delivers about 64 B per cycle — 750
// cycles for work the MMA does in 512. A pair of CTAs on neighbouring SMs
// computes a 256 x 256 tile with ONE instruction stream: each CTA holds its own
// 128 rows of A and only half (128 columns) of B, 32 KB per K-block, and the
// hardware lets both tensor cores see both halves of B.
//
//   cluster of 2 CTAs, persistent over 256 x BN tiles; rank 0 is the leader
//   warp 0 (both CTAs)   TMA producer for the CTA's own A rows and B half;
//                        completion bytes of BOTH CTAs are counted on the
//                        leader's `full` barrier
//   warp 1 (leader)      issues tcgen05.mma.cta_group::2 (M256, N=BN, K32);
//                        its commits arrive on `empty` / `tmem_full` in both CTAs
//   warps 4-11 (both)    epilogue for the CTA's own 128 accumulator rows, as in
//                        the single-CTA kernel; buffers are handed back on the
//                        leader's `tmem_empty` barrier (remote arrive)
// No load in this file names more than one destination CTA; the only
// cluster-wide signals are mbarrier arrivals.
//
// Status: numerically verified (tests force it with KS_B200_FP8_PAIR=1) but not
// selected by default; see fp8_blockwise_pair_eligible() for the measurements.
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "sm100_fp8_gemm.cuh"
#include "sm100_fp8_store.cuh"
#include "sm100_host.cuh"
#include "sm100_ptx.cuh"

namespace ksb {
namespace sm100 {
namespace {

constexpr int kBM = 128;   // rows per CTA (256 per pair)
constexpr int kBK = 128;

template <int BN>
struct PairCfg {
  static constexpr int kStages = 6;
  static constexpr int kABytes = kBM * kBK;
  static constexpr int kBBytes = (BN / 2) * kBK;       // this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiWarps = (BN / 128) * 4;
  static constexpr int kThreads = 128 + kEpiWarps * 32;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static constexpr int kRegsIssue = 40;
  static constexpr int kRegsEpi = 232;
};
static_assert(128 * PairCfg<256>::kRegsIssue + (PairCfg<256>::kThreads - 128) * PairCfg<256>::kRegsEpi <=
                  PairCfg<256>::kThreads * ((65536 / PairCfg<256>::kThreads) & ~7),
              "setmaxnreg budgets exceed the register pool the CTA is launched with");

struct PairParams {
  void* out;
  const float* a_scale;
  const float* b_scale;
  unsigned int* fault_word;
  int m, n, k;
  int nkb, nnb;
  int tiles_n, tiles_m2;   // tiles of 256 rows
  uint32_t idesc;
  int vec_store;
};

template <int BN, bool NT, typename OutT>
__global__ void __launch_bounds__(PairCfg<BN>::kThreads, 1)
fp8_blockwise_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                          const PairParams p) {
  using C = PairCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t ring = (raw_addr + 1023u) & ~1023u;
  uint8_t* ctrl = smem_raw + (ring - raw_addr) + C::kStages * C::kStageBytes;
  const uint32_t ctrl_addr = ring + C::kStages * C::kStageBytes;
  const uint32_t bar_full = ctrl_addr;                       // used in the leader only
  const uint32_t bar_empty = ctrl_addr + 8 * C::kStages;     // one per CTA
  const uint32_t bar_tfull = ctrl_addr + 16 * C::kStages;    // one per CTA
  const uint32_t bar_tempty = bar_tfull + 16;                // used in the leader only
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 16 * C::kStages + 32);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const WaitCtx wctx{abort_flag, p.fault_word};

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 2 * C::kEpiWarps);   // epilogue warps of both CTAs
    }
    *abort_flag = 0u;
    fence_barrier_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();   // barriers of both CTAs exist before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  const int total_tiles = p.tiles_m2 * p.tiles_n;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    setmaxnreg_dec<C::kRegsIssue>();
    uint32_t it = 0;
    bool ok = true;
    for (int t = cluster_id; ok && t < total_tiles; t += num_clusters) {
      const int mt = t / p.tiles_n;
      const int row0 = mt * 256 + static_cast<int>(rank) * kBM;
      const int n0 = (t - mt * p.tiles_n) * BN + static_cast<int>(rank) * (BN / 2);
      for (int kb = 0; kb < p.nkb; ++kb, ++it) {
        const uint32_t s = it % C::kStages;
        const uint32_t ph = (it / C::kStages) & 1u;
        if (!mbar_wait(wctx, bar_empty + 8 * s, ph ^ 1u, 0x1100u + s)) { ok = false; break; }
        const uint32_t full_leader = map_to_cta(bar_full + 8 * s, 0);
        const uint32_t a_dst = ring + s * C::kStageBytes;
        const uint32_t b_dst = a_dst + C::kABytes;
        // the leader announces the bytes of both CTAs; the peer's copies may land first
        if (leader) mbar_arrive_expect_tx_elect(bar_full + 8 * s, 2 * C::kStageBytes);
        tma_load_2d_pair_elect(a_dst, &tm_a, full_leader, kb * kBK, row0);
        if constexpr (NT) tma_load_3d_pair_elect(b_dst, &tm_b, full_leader, kb * kBK, n0, 0);
        else tma_load_3d_pair_elect(b_dst, &tm_b, full_leader, n0, kb * kBK, 0);
      }
    }
  } else if (warp == 1) {
    // --------------------------- MMA issuer (leader) ---------------------------
    setmaxnreg_dec<C::kRegsIssue>();
    if (leader) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = cluster_id; ok && t < total_tiles; t += num_clusters) {
        for (int kb = 0; kb < p.nkb; ++kb, ++it) {
          const uint32_t s = it % C::kStages;
          const uint32_t ph = (it / C::kStages) & 1u;
          const uint32_t buf = it & 1u;
          const uint32_t aph = (it >> 1) & 1u;
          if (!mbar_wait(wctx, bar_tempty + 8 * buf, aph ^ 1u, 0x1200u + buf)) { ok = false; break; }
          if (!mbar_wait(wctx, bar_full + 8 * s, ph, 0x1300u + s)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_src = ring + s * C::kStageBytes;
          const uint32_t b_src = a_src + C::kABytes;
          const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
          for (int kk = 0; kk < kBK / 32; ++kk) {
            // The same shared-memory offsets are read in both CTAs: A = each CTA's 128
            // rows (K-major), B = each CTA's BN/2 rows ([N,K], K-major) or its 128-column
            // atom ([K,N], MN-major).
            const uint64_t a_desc = umma_smem_desc_sw128(a_src + kk * 32, 16, 1024);
            const uint64_t b_desc = NT ? umma_smem_desc_sw128(b_src + kk * 32, 16, 1024)
                                       : umma_smem_desc_sw128(b_src + kk * 32 * 128, 128 * kBK, 1024);
            umma2_f8f6f4_elect(d_tmem, a_desc, b_desc, p.idesc, kk > 0 ? 1u : 0u);
          }
          tc_commit_pair_elect(bar_empty + 8 * s, 0x3);
          tc_commit_pair_elect(bar_tfull + 8 * buf, 0x3);
        }
      }
    }
  } else if (warp >= 4) {
    // -------------------------------- epilogue --------------------------------
    setmaxnreg_inc<C::kRegsEpi>();
    const int quarter = warp & 3;
    const int slice = (warp - 4) >> 2;
    constexpr int EC = 128;
    const int row_in_tile = quarter * 32 + lane;
    OutT* out = static_cast<OutT*>(p.out);
    uint32_t it = 0;
    bool ok = true;
    for (int t = cluster_id; ok && t < total_tiles; t += num_clusters) {
      const int mt = t / p.tiles_n;
      const int row = mt * 256 + static_cast<int>(rank) * kBM + row_in_tile;
      const bool row_ok = row < p.m;
      const int col0 = (t - mt * p.tiles_n) * BN + slice * EC;
      int nb = col0 >> 7;
      if (nb > p.nnb - 1) nb = p.nnb - 1;
      const float* as_ptr = p.a_scale + static_cast<size_t>(row_ok ? row : 0) * p.nkb;
      const float* bs_ptr = p.b_scale + (NT ? static_cast<size_t>(nb) * p.nkb : static_cast<size_t>(nb));
      const size_t bs_step = NT ? 1 : static_cast<size_t>(p.nnb);

      float2 acc[EC / 2];
#pragma unroll
      for (int i = 0; i < EC / 2; ++i) acc[i] = make_float2(0.f, 0.f);
      constexpr int G = 2;
      constexpr int CW = 16;
      float as_nxt[G], bs_nxt[G];
      auto fetch_scales = [&](int kb0) {
#pragma unroll
        for (int j = 0; j < G; ++j) {
          const int kb = kb0 + j;
          const bool in = kb < p.nkb;
          as_nxt[j] = (in && row_ok) ? __ldg(as_ptr + kb) : 0.f;
          bs_nxt[j] = in ? __ldg(bs_ptr + static_cast<size_t>(kb) * bs_step) : 0.f;
        }
      };
      fetch_scales(0);

      for (int kb0 = 0; kb0 < p.nkb && ok; kb0 += G) {
        float sc[G];
#pragma unroll
        for (int j = 0; j < G; ++j) sc[j] = as_nxt[j] * bs_nxt[j];
        fetch_scales(kb0 + G);
#pragma unroll
        for (int j4 = 0; j4 < G; ++j4) {
          if (kb0 + j4 >= p.nkb) break;
          const float2 scale2 = make_float2(sc[j4], sc[j4]);
          const uint32_t buf = it & 1u;
          const uint32_t aph = (it >> 1) & 1u;
          ++it;
          if (!mbar_wait(wctx, bar_tfull + 8 * buf, aph, 0x1400u + buf)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN + slice * EC;
          uint32_t r0[CW], r1[CW];
          tmem_ld(taddr, r0);
#pragma unroll
          for (int c = 0; c < EC / CW; ++c) {
            if (c & 1) tmem_wait_ld(r1);
            else tmem_wait_ld(r0);
            if (c < EC / CW - 1) {
              if (c & 1) tmem_ld(taddr + (c + 1) * CW, r0);
              else tmem_ld(taddr + (c + 1) * CW, r1);
            } else {
              // this warp's slice is in registers: hand the buffer back to the leader's MMA warp
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * buf, 0));
            }
#pragma unroll
            for (int j = 0; j < CW / 2; ++j) {
              const float lo = __uint_as_float((c & 1) ? r1[2 * j] : r0[2 * j]);
              const float hi = __uint_as_float((c & 1) ? r1[2 * j + 1] : r0[2 * j + 1]);
              ffma2(acc[c * (CW / 2) + j], lo, hi, scale2);
            }
          }
        }
      }
      if (ok && row_ok) {
        OutT* dst = out + static_cast<size_t>(row) * p.n + col0;
#pragma unroll
        for (int c = 0; c < EC / 16; ++c) {
          const int valid = p.n - (col0 + c * 16);
          float v[16];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[2 * j] = acc[c * 8 + j].x;
            v[2 * j + 1] = acc[c * 8 + j].y;
          }
          if (valid > 0) store_16<OutT>(dst + c * 16, v, p.vec_store != 0, valid);
        }
      }
    }
  } else {
    setmaxnreg_dec<C::kRegsIssue>();
  }

  // ------------------------------- teardown -------------------------------
  // Neither CTA may leave while the other can still signal its barriers, read
  // its shared memory through an MMA, or write its TMEM.
  tc_fence_before_sync();
  if (*abort_flag != 0u) {
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
}

template <int BN, bool NT, typename OutT>
ks_status_t launch_pair(const Fp8GemmArgs& a, const CUtensorMap& tm_a, const CUtensorMap& tm_b, PairParams p,
                        cudaStream_t stream) {
  using C = PairCfg<BN>;
  auto kernel = fp8_blockwise_pair_kernel<BN, NT, OutT>;
  static std::mutex mu;
  static int clusters_cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int max_clusters = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && clusters_cached[dev] == 0) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
      if (e != cudaSuccess) return cuda_status(e, a.where);
      cudaLaunchConfig_t probe = {};
      probe.gridDim = dim3(static_cast<unsigned>(sm_count() & ~1), 1, 1);
      probe.blockDim = dim3(C::kThreads, 1, 1);
      probe.dynamicSmemBytes = C::kSmemBytes;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
      probe.attrs = &attr;
      probe.numAttrs = 1;
      int n = 0;
      e = cudaOccupancyMaxActiveClusters(&n, kernel, &probe);
      if (e != cudaSuccess || n < 1) {
        cudaGetLastError();
        n = -1;  // pairs cannot be scheduled here
      }
      clusters_cached[dev] = n;
    }
    max_clusters = (dev >= 0 && dev < 64) ? clusters_cached[dev] : -1;
  }
  if (max_clusters < 1) KSB_FAIL(KS_ERROR_INTERNAL, std::string(a.where) + ": CTA pairs cannot be scheduled");
  const int tiles = p.tiles_m2 * p.tiles_n;
  int clusters = sm_count() / 2;
  if (clusters > max_clusters) clusters = max_clusters;
  if (clusters > tiles) clusters = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters), 1, 1);
  cfg.blockDim = dim3(C::kThreads, 1, 1);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cuda_status(cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, p), a.where);
}

template <int BN, bool NT>
ks_status_t launch_pair_out(const Fp8GemmArgs& a, const CUtensorMap& tm_a, const CUtensorMap& tm_b,
                            const PairParams& p, cudaStream_t stream) {
  switch (a.out_dtype) {
    case KS_DTYPE_F32: return launch_pair<BN, NT, float>(a, tm_a, tm_b, p, stream);
    case KS_DTYPE_F16: return launch_pair<BN, NT, __half>(a, tm_a, tm_b, p, stream);
    default: return launch_pair<BN, NT, __nv_bfloat16>(a, tm_a, tm_b, p, stream);
  }
}

}  // namespace

bool fp8_blockwise_pair_eligible(const Fp8GemmArgs& a) {
  if (a.offsets != nullptr) return false;           // grouped problems stay on single CTAs (128-row tiles)
  if (!fp8_blockwise_eligible(a)) return false;
  // Opt-in only (KS_B200_FP8_PAIR=1). Measured on B200 the pair kernel is slower
  // than the single-CTA one (400 us against 213 us on M=4096, N=K=7168): a hand-off
  // between the two CTAs of a cluster costs ~400 cycles each way (816 for the round
  // trip, against ~140 inside a CTA), and the per-K-block promotion needs two such
  // hand-offs (commit -> peer epilogue, peer epilogue -> leader's MMA warp) inside
  // a loop that only two TMEM buffers deep. The MMAs themselves run at full rate
  // (129 cycles per M256 x N256 x K32).
  const char* env = std::getenv("KS_B200_FP8_PAIR");
  return env != nullptr && env[0] == '1';
}

ks_status_t launch_fp8_blockwise_pair(const Fp8GemmArgs& a, cudaStream_t stream) {
  constexpr int BN = 256;
  CUtensorMap tm_a, tm_b;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.m)};
    const uint64_t str[1] = {static_cast<uint64_t>(a.k)};
    const uint32_t box[2] = {static_cast<uint32_t>(kBK), static_cast<uint32_t>(kBM)};
    if (!tma_encode(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      KSB_FAIL(KS_ERROR_INTERNAL, std::string(a.where) + ": tensor map for A rejected");
  }
  if (a.nt) {
    const uint64_t dims[3] = {static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.n), 1};
    const uint64_t str[2] = {static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.k) * static_cast<uint64_t>(a.n)};
    const uint32_t box[3] = {static_cast<uint32_t>(kBK), static_cast<uint32_t>(BN / 2), 1u};
    if (!tma_encode(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a.b, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      KSB_FAIL(KS_ERROR_INTERNAL, std::string(a.where) + ": tensor map for B rejected");
  } else {
    const uint64_t dims[3] = {static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.k), 1};
    const uint64_t str[2] = {static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.k) * static_cast<uint64_t>(a.n)};
    const uint32_t box[3] = {128u, static_cast<uint32_t>(kBK), 1u};
    if (!tma_encode(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a.b, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      KSB_FAIL(KS_ERROR_INTERNAL, std::string(a.where) + ": tensor map for B rejected");
  }
  PairParams p;
  p.out = a.out;
  p.a_scale = a.a_scale;
  p.b_scale = a.b_scale;
  p.fault_word = kernel_fault_word();
  p.m = static_cast<int>(a.m);
  p.n = static_cast<int>(a.n);
  p.k = static_cast<int>(a.k);
  p.nkb = static_cast<int>((a.k + kBK - 1) / kBK);
  p.nnb = static_cast<int>((a.n + 127) / 128);
  p.tiles_n = static_cast<int>((a.n + BN - 1) / BN);
  p.tiles_m2 = static_cast<int>((a.m + 255) / 256);
  const uint32_t fmt = a.e5m2 ? 1u : 0u;
  p.idesc = umma_instr_desc(fmt, fmt, 0u, a.nt ? 0u : 1u, 256u, static_cast<uint32_t>(BN));
  const size_t out_elt = a.out_dtype == KS_DTYPE_F32 ? 4 : 2;
  p.vec_store = (aligned16(a.out) && (static_cast<size_t>(a.n) * out_elt) % 16 == 0) ? 1 : 0;
  return a.nt ? launch_pair_out<BN, true>(a, tm_a, tm_b, p, stream)
              : launch_pair_out<BN, false>(a, tm_a, tm_b, p, stream);
}

}  // namespace sm100
}  // namespace ksb
