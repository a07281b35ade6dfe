// int4 weight-only GEMM for sm_100a, built for the decode regime (few
// activation rows, the packed weight read once from HBM).
//
// Computes what ks_gemm_w4a16 declares (reference: kernels/src/gemm/
// gemm_w4a16.cu:50-130, layout :6-19): C[M,N] = A[M,K] . W + bias with
// W[k,n] = (q[k,n] - zero[g,n]) * scale[g,n] rounded once to the activation
// type (the reference's torch statement, benchmarks/bench.py:1275-1284), then
// multiplied with fp32 accumulation.
//
// The GEMM is transposed onto the tensor core: the weight's N dimension is the
// UMMA M dimension (128 TMEM lanes), the tokens are the UMMA N dimension
// (16..128 columns), so a CTA streams 128 weight columns x 128 k per step ("unit").
// Two ways of handing the dequantised weights (the A operand) to the tensor core:
//
// Tensor-memory operand (token tiles of at most 32 rows, K a multiple of 256; default there):
//   warp 0        weight producer (TMA): boxes of two K-steps, [128 byte-rows x 128
//                 columns] = 16 KB straight from HBM, eight stages. (A warp keeps only
//                 about three TMA loads in flight whatever their size; 8 KB boxes cap a
//                 single producer warp near 2.5 TB/s, 16 KB boxes near 4.5 TB/s.)
//   warp 2        activation producer (TMA): one 3-D box per K-step (both 64-k swizzle
//                 atoms of the K-slice [tokens x 128], from L2)
//   warps 4-11    dequantisation, two groups of four warps on alternate units. A thread
//                 owns ONE weight column (= one TMEM lane) and walks down its 64 packed
//                 bytes: a byte holds the codes of k and k+1, exactly one 32-bit operand
//                 cell; b * 0x1001 and one mask-or build the pair (magic + q), two packed
//                 16-bit operations subtract (magic + zero) and apply the scale, and
//                 tcgen05.st writes 16 cells at a time. Scales and zero-points are read
//                 from global memory one unit ahead.
//   warps 1, 3    MMA issuers: 4 x tcgen05.mma kind::f16 (M128, N=tokens, K16) each per
//                 unit, A operand in tensor memory, into disjoint accumulators
// Shared-memory operand (everything else, or KS_B200_W4A16_OPERAND=smem):
//   warp 0        weight producer: packed tile [64 byte-rows x 128 columns] = 8 KB plus the
//                 group's 128 scales and zero-points (2 x 256 B) per unit
//   warp 2        activation producer (two 2-D boxes per unit)
//   warps 4-11    dequantisation: a thread owns 8 columns x 16 k of a unit, 8 packed bytes
//                 -> 16 weights per step by byte-permute into the (magic + q) pattern,
//                 written as the MN-major, 128-byte-swizzled UMMA A operand
//   warps 1, 3    MMA issuers, both operands from shared memory
// Both:
//   warps 12-15   epilogue: TMEM -> registers -> C, or -> an fp32 partial slot
// Measured on B200, decode shapes: both arrangements take ~39 us for K=4096, N=28672
// (~1000 cycles per unit against ~300 at the HBM rate). The shared-memory operand moves
// 64 KB per unit through shared memory (~650 cycles at 128 B/clk); the tensor-memory
// operand is bounded by tcgen05.st, which sustains only ~20 B/clk per scheduler whatever
// the store width (~400 cycles per unit), and by its per-unit chain of waits. Processing
// whole two-K-step boxes per iteration measured slower (48 us: two operand stages are too
// few), as did sixteen dequantisation warps.
// Work is cut stream-K style: the (column tile, K-step) units are dealt to the
// CTAs in equal contiguous runs, so every SM streams the same number of bytes
// whatever N is. A column tile whose K range is shared by several CTAs is
// finished by the last CTA to arrive: each writes its fp32 partial to its own
// slot, bumps the tile's counter, and the one that completes the count sums the
// slots in slot order (deterministic) and writes C. Slots and counters live in
// library-owned scratch memory that stays in L2.
//
// Roofline: HBM-bound for M <= 64; algorithmic bytes per launch
// K*N/2 + (K/gs)*N*2*(1 or 2) + M*K*2 + M*N*2.
#include <cstdio>
#include <mutex>

#include <cstdlib>

#include "common.cuh"
#include "sm100_host.cuh"
#include "sm100_ptx.cuh"
#include "sm100_w4a16.cuh"

namespace ksb {
namespace sm100 {
namespace {

constexpr int kTileN = 128;    // weight columns per tile = UMMA M
constexpr int kStepK = 128;    // k per pipeline step (one scale group when gs % 128 == 0)
constexpr int kRawBytes = (kStepK / 2) * kTileN;      // 8192
constexpr int kRawStage = kRawBytes + 2 * 256;        // + scales + zeros of the step
constexpr int kDeqBytes = kStepK * kTileN * 2;        // 32768: dequantised UMMA operand
constexpr int kDeqGroupWarps = 4;  // a group = one warp per TMEM lane quarter = one unit at a time
// The numbers of operand stages and of activation stages must be multiples of the number
// of issuers: an issuer's wait on a stage's `full` barrier is ordered after the stage's
// previous use only because the same issuer consumed that use. (Three issuers with four
// stages let an issuer pass a fresh barrier one phase early: intermittent bounded-wait
// timeouts on the GPU, and a deadlock in the protocol model under tests/.)
#ifndef KSB_W4_TMEM_ISSUERS
#define KSB_W4_TMEM_ISSUERS 2
#endif
#ifndef KSB_W4_TMEM_STAGES
#define KSB_W4_TMEM_STAGES 4
#endif
#ifndef KSB_W4_TMEM_GROUPS
#define KSB_W4_TMEM_GROUPS 4
#endif

// TA: the dequantised weights are handed to the tensor core through tensor memory
// (tcgen05.st, A operand in TMEM) instead of shared memory. Decode shapes only
// (MTMAX == 32): the accumulators of wider token tiles need all 512 TMEM columns.
template <int MTMAX, bool TA>
struct Cfg {
  static_assert(!TA || MTMAX <= 32, "the TMEM operand path is built for token tiles of at most 32 rows");
  // TA: a stage is one TMA box of two K-steps (16 KB); scales and zero-points do not
  // travel through it. A warp keeps only about three TMA loads in flight, so the box
  // has to be large for one producer warp to cover HBM latency.
  // Dequantisation groups working on different units at the same time. The tensor-memory
  // path is a chain of waits per unit (~1900 cycles per group); more groups in flight hide
  // it until tcgen05.st bandwidth (~400 cycles per unit) becomes the limit.
  static constexpr int kGroups = TA ? KSB_W4_TMEM_GROUPS : 2;
  static constexpr int kDeqWarps = kGroups * kDeqGroupWarps;
  // MMA issuers: warps 1 and 3, plus (TA) extra warps after the epilogue warps. An issuer
  // spends ~1000 cycles per unit it owns (barrier tests, eight MMAs, commits).
  static constexpr int kIssuers = TA ? KSB_W4_TMEM_ISSUERS : 2;
  static_assert(!TA || (KSB_W4_TMEM_STAGES % KSB_W4_TMEM_ISSUERS == 0 && 8 % KSB_W4_TMEM_ISSUERS == 0),
                "stage counts must be multiples of the number of issuers");
  static constexpr int kExtraIssuerWarp0 = 4 + kDeqWarps + 4;   // first warp index after the epilogue warps
  static constexpr int kThreads = 128 + kDeqWarps * 32 + 128 + (kIssuers - 2) * 32;
  static constexpr int kRawStages = TA ? 8 : (MTMAX <= 32 ? 9 : 6);
  static constexpr int kRawStageBytes = TA ? 2 * kRawBytes : kRawStage;
  static constexpr int kActStages = TA ? 8 : (MTMAX <= 32 ? 4 : 3);
  // TA: more operand stages than groups, so that a group can fill its next stage while the
  // MMAs of its previous unit are still queued
  static constexpr int kDeqStages = TA ? KSB_W4_TMEM_STAGES : (MTMAX <= 32 ? 3 : 2);
  // shared memory per dequantised stage; with TA a stage is 64 TMEM columns instead
  static constexpr int kDeqSmem = TA ? 0 : kDeqBytes;
  static constexpr int kDeqTmemCols = kStepK / 2;
  // Consecutive K=16 instructions of a step go to different TMEM accumulators:
  // an instruction that accumulates into the result of the previous one waits
  // for it, and with 16..32 token columns that latency, not throughput, would
  // set the pace. The epilogue adds the accumulators up.
  // TA: accumulators per issuer times issuers; the operand stages take the rest of TMEM
  static constexpr int kAccsPerIssuer = (TA && (KSB_W4_TMEM_STAGES > 4 || KSB_W4_TMEM_ISSUERS > 2)) ? 1 : 2;
  static constexpr int kAccs = TA ? kAccsPerIssuer * kIssuers : (MTMAX <= 32 ? 8 : 2);
  static constexpr int kAccCols = 2 * kAccs * MTMAX;   // two segment buffers
  static constexpr int kTmemCols = TA ? 512 : kAccCols;
  static constexpr int kOperandCol0 = kAccCols;         // TA: first column of the operand ring
  static_assert(!TA || kAccCols + kDeqStages * kDeqTmemCols <= 512, "TMEM holds 512 columns");
  static constexpr int kActStage = MTMAX * kStepK * 2;  // bytes reserved per activation stage
  static constexpr int kRing = kDeqStages * kDeqSmem + kActStages * kActStage + kRawStages * kRawStageBytes;
  static constexpr int kNumBars = 2 * kRawStages + 2 * kActStages + 2 * kDeqStages + 4;
  static constexpr int kSmemBytes = kRing + 1024 + 512;
};

struct Params {
  void* c;
  const void* bias;
  const void* scales;       // read directly by the tensor-memory path
  const void* zeros;
  float* slots;             // [tiles][max_parts][mt][128] fp32 partials
  unsigned int* counters;   // [tiles]
  unsigned int* fault_word;
  int m, n, k;
  int mt;                   // token tile, multiple of 16, <= MTMAX
  int m_tiles;
  int n_tiles, k_steps;
  int gs_steps;             // K-steps per scale group (group_size / 128)
  int max_parts;
  int has_zeros;
  uint32_t idesc;
};

template <typename T> struct Pack16;
template <> struct Pack16<__nv_bfloat16> {
  using V2 = __nv_bfloat162;
  static constexpr uint32_t kMagicBytes = 0x43434343u;  // high byte of bf16(128 + q)
  static constexpr float kMagic = 128.0f;
  static constexpr uint32_t kMaxZeroBits = 0x42FEu;     // bf16(127)
  __device__ static V2 from_bits(uint32_t b) { return *reinterpret_cast<V2*>(&b); }
  __device__ static uint32_t bits(V2 v) { return *reinterpret_cast<uint32_t*>(&v); }
  __device__ static V2 splat(float f) { return __float2bfloat162_rn(f); }
  __device__ static float lo(V2 v) { return __low2float(v); }
  __device__ static float hi(V2 v) { return __high2float(v); }
  __device__ static V2 make(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <> struct Pack16<__half> {
  using V2 = __half2;
  static constexpr uint32_t kMagicBytes = 0x64646464u;  // high byte of f16(1024 + q)
  static constexpr float kMagic = 1024.0f;
  static constexpr uint32_t kMaxZeroBits = 0x63FEu;     // f16(1023)
  __device__ static V2 from_bits(uint32_t b) { return *reinterpret_cast<V2*>(&b); }
  __device__ static uint32_t bits(V2 v) { return *reinterpret_cast<uint32_t*>(&v); }
  __device__ static V2 splat(float f) { return __float2half2_rn(f); }
  __device__ static float lo(V2 v) { return __low2float(v); }
  __device__ static float hi(V2 v) { return __high2float(v); }
  __device__ static V2 make(float a, float b) { return __floats2half2_rn(a, b); }
};

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <typename T, int MTMAX, bool TA>
__global__ void __launch_bounds__((Cfg<MTMAX, TA>::kThreads), 1)
w4a16_umma_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_s,
                  const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_a,
                  const Params p) {
  using C = Cfg<MTMAX, TA>;
  using P16 = Pack16<T>;
  using V2 = typename P16::V2;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  // ring: dequantised operand stages | activation stages | raw stages | barriers
  const uint32_t deq_base = base;
  const uint32_t act_base = deq_base + C::kDeqStages * C::kDeqSmem;
  const uint32_t rawst_base = act_base + C::kActStages * C::kActStage;
  const uint32_t bar_base = rawst_base + C::kRawStages * C::kRawStageBytes;
  uint8_t* deq_ptr = base_ptr;
  uint8_t* rawst_ptr = base_ptr + (rawst_base - base);
  uint8_t* ctrl_ptr = base_ptr + (bar_base - base);
  const uint32_t bar_raw_full = bar_base;
  const uint32_t bar_raw_empty = bar_raw_full + 8 * C::kRawStages;
  const uint32_t bar_act_full = bar_raw_empty + 8 * C::kRawStages;
  const uint32_t bar_act_empty = bar_act_full + 8 * C::kActStages;
  const uint32_t bar_deq_full = bar_act_empty + 8 * C::kActStages;
  const uint32_t bar_deq_empty = bar_deq_full + 8 * C::kDeqStages;
  const uint32_t bar_acc_full = bar_deq_empty + 8 * C::kDeqStages;
  const uint32_t bar_acc_empty = bar_acc_full + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl_ptr + 8 * C::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* last_flag = tmem_slot + 2;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx wctx{abort_flag, p.fault_word};

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kRawStages; ++s) {
      mbar_init(bar_raw_full + 8 * s, 1);
      mbar_init(bar_raw_empty + 8 * s, TA ? 2 * kDeqGroupWarps : kDeqGroupWarps);   // TA: both halves of a box
    }
    for (int s = 0; s < C::kActStages; ++s) {
      mbar_init(bar_act_full + 8 * s, 1);
      mbar_init(bar_act_empty + 8 * s, TA ? 1 : 2);   // TA: the issuer that owns the unit; else both
    }
    for (int s = 0; s < C::kDeqStages; ++s) {
      mbar_init(bar_deq_full + 8 * s, kDeqGroupWarps);
      mbar_init(bar_deq_empty + 8 * s, TA ? 1 : 2);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, C::kIssuers);
      mbar_init(bar_acc_empty + 8 * b, 4);
    }
    *abort_flag = 0u;
    fence_barrier_init();
    prefetch_tensormap(&tm_w);
    prefetch_tensormap(&tm_s);
    prefetch_tensormap(&tm_a);
    if (p.has_zeros) prefetch_tensormap(&tm_z);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Unit space: (token tile, column tile, K-step), K-step fastest. With one
  // token tile the units are dealt in exact equal runs (column tiles may be
  // split between CTAs); with several, runs are snapped to whole column tiles
  // so that no partial sums arise.
  const long long units = static_cast<long long>(p.n_tiles) * p.k_steps;   // per token tile
  const int ctas = gridDim.x;
  long long u_begin, u_end;
  if (p.m_tiles == 1) {
    u_begin = run_start(units, ctas, blockIdx.x);
    u_end = run_start(units, ctas, blockIdx.x + 1);
  } else {
    const long long tiles_total = static_cast<long long>(p.m_tiles) * p.n_tiles;
    u_begin = run_start(tiles_total, ctas, blockIdx.x) * p.k_steps;
    u_end = run_start(tiles_total, ctas, blockIdx.x + 1) * p.k_steps;
  }
  const uint32_t act_tx = static_cast<uint32_t>(p.mt) * kStepK * 2;
  const uint32_t raw_tx = kRawBytes + 256 + (p.has_zeros ? 256 : 0);
  // The next kernel on the stream may start its prologue now. This one touches what the
  // kernel before it may have produced or may still read (activations, C, the split-K
  // scratch) only behind grid_dependency_wait(): the activation producer and the epilogue.
  grid_launch_dependents();

  if (warp == 0) {
    // ------------------------- weight producer (TMA) -------------------------
    if constexpr (TA) {
      // boxes of two K-steps; k_steps is even here, so a box never straddles two column
      // tiles, and with a single token tile u indexes (tile, step) directly
      const long long b_end = (u_end + 1) >> 1;
      uint32_t itb = 0;
      // (tile, step) advance with the loop: a 64-bit division per box would cost hundreds of cycles
      int tile = static_cast<int>((u_begin & ~1ll) / p.k_steps);
      int step = static_cast<int>((u_begin & ~1ll) - static_cast<long long>(tile) * p.k_steps);
      for (long long b = u_begin >> 1; b < b_end; ++b, ++itb, step += 2) {
        if (step >= p.k_steps) { step -= p.k_steps; ++tile; }
        const uint32_t sr = itb % C::kRawStages, pr = (itb / C::kRawStages) & 1u;
        if (!mbar_wait(wctx, bar_raw_empty + 8 * sr, pr ^ 1u, 0x100u + sr)) break;
        const uint32_t full = bar_raw_full + 8 * sr;
        mbar_arrive_expect_tx_elect(full, 2 * kRawBytes);
        tma_load_2d_elect(rawst_base + sr * C::kRawStageBytes, &tm_w, full, tile * kTileN, step * (kStepK / 2));
      }
    } else {
    uint32_t it = 0;
    for (long long u = u_begin; u < u_end; ++u, ++it) {
      const long long ul = u % units;
      const int tile = static_cast<int>(ul / p.k_steps);
      const int step = static_cast<int>(ul - static_cast<long long>(tile) * p.k_steps);
      const uint32_t sr = it % C::kRawStages, pr = (it / C::kRawStages) & 1u;
      if (!mbar_wait(wctx, bar_raw_empty + 8 * sr, pr ^ 1u, 0x100u + sr)) break;
      {
        const uint32_t full = bar_raw_full + 8 * sr;
        const uint32_t dst = rawst_base + sr * kRawStage;
        mbar_arrive_expect_tx_elect(full, raw_tx);
        tma_load_2d_elect(dst, &tm_w, full, tile * kTileN, step * (kStepK / 2));
        tma_load_2d_elect(dst + kRawBytes, &tm_s, full, tile * kTileN, step / p.gs_steps);
        if (p.has_zeros) tma_load_2d_elect(dst + kRawBytes + 256, &tm_z, full, tile * kTileN, step / p.gs_steps);
      }
    }
    }
  } else if (warp == 2) {
    // ----------------------- activation producer (TMA) -----------------------
    grid_dependency_wait();
    uint32_t it = 0;
    int mtile = static_cast<int>(u_begin / units);
    int step = static_cast<int>((u_begin - static_cast<long long>(mtile) * units) % p.k_steps);
    long long next_mtile_at = (static_cast<long long>(mtile) + 1) * units;
    for (long long u = u_begin; u < u_end; ++u, ++it, step = (step + 1 == p.k_steps) ? 0 : step + 1) {
      if (u == next_mtile_at) { ++mtile; next_mtile_at += units; }
      const uint32_t sa = it % C::kActStages, pa = (it / C::kActStages) & 1u;
      if (!mbar_wait(wctx, bar_act_empty + 8 * sa, pa ^ 1u, 0x180u + sa)) break;
      {
        const uint32_t full = bar_act_full + 8 * sa;
        const uint32_t dst = act_base + sa * C::kActStage;
        mbar_arrive_expect_tx_elect(full, act_tx);
        if constexpr (TA) {
          // one load for both 64-k atoms: the map views A as [K/64][M][64]
          tma_load_3d_elect(dst, &tm_a, full, 0, mtile * p.mt, step * 2);
        } else {
          tma_load_2d_elect(dst, &tm_a, full, step * kStepK, mtile * p.mt);
          tma_load_2d_elect(dst + p.mt * 128, &tm_a, full, step * kStepK + 64, mtile * p.mt);
        }
      }
    }
  } else if (warp == 1 || warp == 3 || (warp >= C::kExtraIssuerWarp0 && warp < C::kExtraIssuerWarp0 + C::kIssuers - 2)) {
    // ------------------------------ MMA issuers ------------------------------
    // Issuing one tcgen05.mma costs its thread ~55 cycles; eight per unit from one
    // thread would set the pace of the whole kernel. Two warps issue four each,
    // into disjoint accumulators (an accumulator must have a single issuer).
    const int mma_half = warp == 1 ? 0 : (warp == 3 ? 1 : 2 + (warp - C::kExtraIssuerWarp0));   // issuer index
    constexpr int kHalfAccs = TA ? C::kAccsPerIssuer : C::kAccs / 2;
    uint32_t it = 0, seg = 0;
    if constexpr (TA) {
      // The issuers take the units in turn (unit it -> issuer it % kIssuers): per unit an
      // issuer pays its barrier tests (~100 cycles each), eight MMAs (~55 each) and the
      // commits; sharing every unit between all issuers made each of them pay the fixed part
      // for every unit. An issuer owns its accumulator(s) of the segment buffer and tells the
      // epilogue "done" after its last unit of the segment; an issuer without a unit in a
      // short segment arrives without a commit, and the epilogue skips its accumulators.
      int step = static_cast<int>(u_begin % p.k_steps);
      uint32_t n_in_seg = 0;
      for (long long u = u_begin; u < u_end; ++u, ++it, step = (step + 1 == p.k_steps) ? 0 : step + 1) {
        const bool seg_first = (u == u_begin) || (step == 0);
        const bool seg_last = (u + 1 == u_end) || (step == p.k_steps - 1);
        // last unit of this segment: end of the column tile or of this CTA's run
        const long long tile_last = u - step + p.k_steps - 1;
        const long long seg_last_u = tile_last < u_end - 1 ? tile_last : u_end - 1;
        const bool mine = static_cast<int>(it % C::kIssuers) == mma_half;
        const bool my_last = u + C::kIssuers > seg_last_u;   // no later unit of mine in this segment
        const uint32_t sd = it % C::kDeqStages, pd = (it / C::kDeqStages) & 1u;
        const uint32_t sa = it % C::kActStages, pa = (it / C::kActStages) & 1u;
        const uint32_t buf = seg & 1u, pacc = (seg >> 1) & 1u;
        if (seg_first) n_in_seg = 0;
        if (mine) {
          if (n_in_seg == 0 && !mbar_wait(wctx, bar_acc_empty + 8 * buf, pacc ^ 1u, 0x200u + buf)) break;
          if (!mbar_wait_both(wctx, bar_deq_full + 8 * sd, pd, 0x280u + sd, bar_act_full + 8 * sa, pa, 0x300u + sa)) break;
          tc_fence_after_sync();
          const uint32_t a_src = act_base + sa * C::kActStage;
          const uint32_t d_tmem = tmem_base + buf * (C::kAccs * MTMAX);
          const uint32_t w_stage = tmem_base + C::kOperandCol0 + sd * C::kDeqTmemCols;
#pragma unroll
          for (int kk = 0; kk < kStepK / 16; ++kk) {
            // tokens: K-major, two 64-k atoms of mt rows, 32 B per instruction inside an atom;
            // weights: 16 k = 8 columns of the operand stage in tensor memory
            const uint64_t a_desc = umma_smem_desc_sw128(a_src + (kk >> 2) * (p.mt * 128) + (kk & 3) * 32, 16, 1024);
            const uint32_t d_acc = d_tmem + (mma_half * kHalfAccs + (kk % kHalfAccs)) * MTMAX;
            umma_f16_tmem_a_elect(d_acc, w_stage + kk * 8, a_desc, p.idesc, (n_in_seg == 0 && kk < kHalfAccs) ? 0u : 1u);
          }
          ++n_in_seg;
          tc_commit_elect(bar_deq_empty + 8 * sd);
          tc_commit_elect(bar_act_empty + 8 * sa);
          if (my_last) tc_commit_elect(bar_acc_full + 8 * buf);   // my last unit of the segment
        } else if (seg_last && n_in_seg == 0) {
          // A short segment without a unit of mine. Like an issuer with work, wait until the
          // epilogue has drained this buffer's previous segment: otherwise this arrival could
          // overtake my own (asynchronous) commit for that segment and complete its phase early.
          if (!mbar_wait(wctx, bar_acc_empty + 8 * buf, pacc ^ 1u, 0x200u + buf)) break;
          mbar_arrive_elect(bar_acc_full + 8 * buf);
        }
        if (seg_last) ++seg;
      }
    } else {
      int step = static_cast<int>(u_begin % p.k_steps);
      for (long long u = u_begin; u < u_end; ++u, ++it, step = (step + 1 == p.k_steps) ? 0 : step + 1) {
        const bool seg_first = (u == u_begin) || (step == 0);
        const bool seg_last = (u + 1 == u_end) || (step == p.k_steps - 1);
        const uint32_t sd = it % C::kDeqStages, pd = (it / C::kDeqStages) & 1u;
        const uint32_t sa = it % C::kActStages, pa = (it / C::kActStages) & 1u;
        const uint32_t buf = seg & 1u, pacc = (seg >> 1) & 1u;
        if (seg_first && !mbar_wait(wctx, bar_acc_empty + 8 * buf, pacc ^ 1u, 0x200u + buf)) break;
        if (!mbar_wait(wctx, bar_deq_full + 8 * sd, pd, 0x280u + sd)) break;
        if (!mbar_wait(wctx, bar_act_full + 8 * sa, pa, 0x300u + sa)) break;
        tc_fence_after_sync();
        {
          // all 32 lanes run this code; each instruction elects its one issuing lane
          const uint32_t w_src = deq_base + sd * C::kDeqSmem;
          const uint32_t a_src = act_base + sa * C::kActStage;
          const uint32_t d_tmem = tmem_base + buf * (C::kAccs * MTMAX);
#pragma unroll
          for (int kq = 0; kq < kStepK / 32; ++kq) {
            const int kk = mma_half * (kStepK / 32) + kq;
            // Weights: MN-major, 64-column atoms 16 KB apart, 8-k groups 1024 B
            // apart, 16 k = 2048 B per instruction. Tokens: K-major, two 64-k
            // atoms of mt rows, 32 B per instruction inside an atom.
            const uint64_t a_desc = umma_smem_desc_sw128(a_src + (kk >> 2) * (p.mt * 128) + (kk & 3) * 32, 16, 1024);
            const uint32_t d_acc = d_tmem + (mma_half * kHalfAccs + (kq % kHalfAccs)) * MTMAX;
            const uint32_t first = (seg_first && kq < kHalfAccs) ? 0u : 1u;
            const uint64_t w_desc = umma_smem_desc_sw128(w_src + kk * 2048, 16384, 1024);
            umma_f16_elect(d_acc, w_desc, a_desc, p.idesc, first);
          }
          tc_commit_elect(bar_deq_empty + 8 * sd);
          tc_commit_elect(bar_act_empty + 8 * sa);
          if (seg_last) tc_commit_elect(bar_acc_full + 8 * buf);
        }
        if (seg_last) ++seg;
      }
    }
  } else if (warp >= 4 && warp < 4 + C::kDeqWarps) {
    // ----------------------------- dequantisation -----------------------------
    const int group = (warp - 4) >> 2;          // which units of this CTA's run: u % kGroups == group
    const int tt = (threadIdx.x - 128) & 127;   // thread inside its group
    const int oct = tt & 15;   // 8 weight columns: n_local = 8*oct .. 8*oct+7
    const int rg = tt >> 4;    // 8 packed byte-rows: k_local = 16*rg .. 16*rg+15
    const uint32_t atom_off = (oct >> 3) * 16384u;
    const uint32_t chunk = oct & 7;
    const V2 magic2 = P16::splat(P16::kMagic);
    if constexpr (TA) {
      // A thread owns one weight column (= one TMEM lane; warp w may only touch the lane
      // quarter w % 4) and walks down its 64 packed bytes. A byte holds the codes of k and
      // k+1, which is exactly one 32-bit operand cell: b * 0x1001 puts the low nibble at bit
      // 0 and the high nibble at bit 16, one mask-and-or makes the pair (magic + q), and
      // two packed operations subtract (magic + zero) and apply the scale.
      const int quarter = warp & 3;
      const int n_local = quarter * 32 + lane;
      constexpr uint32_t kMagic2 = P16::kMagicBytes & 0xFF00FF00u;
      // Group g owns the units u with u % kGroups == g: K-step half (g & 1) of every box b
      // with b % (kGroups / 2) == g >> 1. Scales and zero-points come straight from global
      // memory, fetched one unit of the group ahead; (tile, step) of the unit being fetched
      // advance without any 64-bit division (k_steps and kGroups are even, so the parity of
      // step is fixed).
      constexpr int kBoxStride = C::kGroups / 2;
      const int half = group & 1;
      const unsigned short* gscales = static_cast<const unsigned short*>(p.scales);
      const unsigned short* gzeros = static_cast<const unsigned short*>(p.zeros);
      const long long b_begin = u_begin >> 1, b_end = (u_end + 1) >> 1;
      long long b_first = b_begin;
      while ((b_first % kBoxStride) != (group >> 1)) ++b_first;
      long long u_first = (b_first << 1) + half;
      if (u_first < u_begin) u_first += C::kGroups;
      int f_tile = static_cast<int>(u_first / p.k_steps);
      int f_step = static_cast<int>(u_first - static_cast<long long>(f_tile) * p.k_steps);
      int f_row = f_step / p.gs_steps, f_in_row = f_step - f_row * p.gs_steps;
      auto fetch_sz = [&](uint32_t* s_out, uint32_t* z_out) {
        const int n = f_tile * kTileN + n_local;
        const size_t idx = static_cast<size_t>(f_row) * p.n + n;
        const bool n_ok = n < p.n;
        *s_out = n_ok ? __ldg(gscales + idx) : 0u;
        *z_out = (n_ok && p.has_zeros) ? __ldg(gzeros + idx) : 0u;
        f_step += C::kGroups;
        f_in_row += C::kGroups;
        if (f_step >= p.k_steps) {
          while (f_step >= p.k_steps) { f_step -= p.k_steps; ++f_tile; }
          f_row = 0;
          f_in_row = f_step;
        }
        while (f_in_row >= p.gs_steps) { f_in_row -= p.gs_steps; ++f_row; }
      };
      uint32_t s_next = 0u, z_next = 0u;
      if (u_first < u_end) fetch_sz(&s_next, &z_next);
      for (long long b = b_first; b < b_end; b += kBoxStride) {
        const uint32_t itb = static_cast<uint32_t>(b - b_begin);
        const uint32_t sr = itb % C::kRawStages, pr = (itb / C::kRawStages) & 1u;
        const long long u = (b << 1) + half;
        if (u < u_begin || u >= u_end) {
          // this half of the box belongs to a neighbouring CTA's run
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_raw_empty + 8 * sr);
          continue;
        }
        const uint32_t it = static_cast<uint32_t>(u - u_begin);
        const uint32_t sd = it % C::kDeqStages, pd = (it / C::kDeqStages) & 1u;
        const uint32_t s16 = s_next, z16 = z_next;
        if (u + C::kGroups < u_end) fetch_sz(&s_next, &z_next);
        if (!mbar_wait_both(wctx, bar_raw_full + 8 * sr, pr, 0x400u + sr, bar_deq_empty + 8 * sd, pd ^ 1u, 0x480u + sd)) break;
        const uint8_t* col = rawst_ptr + sr * C::kRawStageBytes + half * kRawBytes + n_local;
        const V2 sc = P16::from_bits(s16 | (s16 << 16));
        const uint32_t zw = z16 | (z16 << 16);
        const V2 zz = __hadd2(P16::from_bits(zw), magic2);
        // (magic + zero) exact and |q - zero| exact: non-negative integer zero-points up to kMaxZero
        const uint32_t back = P16::bits(__hsub2(zz, magic2));
        const bool simple = ((back ^ zw) | (zw & 0x80008000u)) == 0u && z16 <= P16::kMaxZeroBits;
        const uint32_t t_dst = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + C::kOperandCol0 +
                               sd * C::kDeqTmemCols;
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          uint32_t cells[16];
          if (simple) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const uint32_t b = col[(c4 * 16 + j) * kTileN];
              const uint32_t x = ((b * 0x1001u) & 0x000F000Fu) | kMagic2;
              cells[j] = P16::bits(__hmul2(__hsub2(P16::from_bits(x), zz), sc));
            }
          } else {
            // zero-points that are not small integers: the fp32 statement, verbatim
            const float z0 = P16::lo(P16::from_bits(zw)), s0 = P16::lo(sc);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const uint32_t b = col[(c4 * 16 + j) * kTileN];
              cells[j] = P16::bits(P16::make(__fmul_rn(__fsub_rn(static_cast<float>(b & 15u), z0), s0),
                                             __fmul_rn(__fsub_rn(static_cast<float>(b >> 4), z0), s0)));
            }
          }
          tmem_st(t_dst + c4 * 16, cells);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_raw_empty + 8 * sr);   // every byte of the packed stage has been read
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_deq_full + 8 * sd);
      }
    } else {
      for (long long u = u_begin + group; u < u_end; u += 2) {
        const uint32_t it = static_cast<uint32_t>(u - u_begin);
        const uint32_t sr = it % C::kRawStages, pr = (it / C::kRawStages) & 1u;
        const uint32_t sd = it % C::kDeqStages, pd = (it / C::kDeqStages) & 1u;
        if (!mbar_wait(wctx, bar_raw_full + 8 * sr, pr, 0x400u + sr)) break;
        const uint8_t* raw = rawst_ptr + sr * kRawStage;
        // the packed bytes this thread owns, and the group constants of its 8 columns
        uint2 pk[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) pk[i] = *reinterpret_cast<const uint2*>(raw + (rg * 8 + i) * kTileN + oct * 8);
        const uint4 s4 = *reinterpret_cast<const uint4*>(raw + kRawBytes + oct * 16);
        uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
        if (p.has_zeros) z4 = *reinterpret_cast<const uint4*>(raw + kRawBytes + 256 + oct * 16);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_raw_empty + 8 * sr);  // the packed stage is in registers
        const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w};
        const uint32_t zw[4] = {z4.x, z4.y, z4.z, z4.w};
        V2 sc[4], zz[4];
        // (magic + zero) must be exact and |q - zero| small enough to be exact too:
        // true for non-negative integer zero-points up to kMaxZero, which a packed
        // add / subtract round trip plus two range checks establish.
        uint32_t bad = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sc[j] = P16::from_bits(sw[j]);
          const V2 z = P16::from_bits(zw[j]);
          zz[j] = __hadd2(z, magic2);
          const uint32_t back = P16::bits(__hsub2(zz[j], magic2));
          bad |= (back ^ zw[j]) | (zw[j] & 0x80008000u);
          bad |= ((zw[j] & 0xFFFFu) > P16::kMaxZeroBits) ? 1u : 0u;
          bad |= ((zw[j] >> 16) > P16::kMaxZeroBits) ? 1u : 0u;
        }
        const bool simple = bad == 0u;
        if (!mbar_wait(wctx, bar_deq_empty + 8 * sd, pd ^ 1u, 0x480u + sd)) break;
        uint8_t* deq = deq_ptr + sd * kDeqBytes + atom_off;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r_even = rg * 16 + 2 * i;
          uint32_t even[4], odd[4];
          if (simple) {
            const uint32_t words[2] = {pk[i].x, pk[i].y};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t e = words[h] & 0x0F0F0F0Fu;
              const uint32_t o = (words[h] >> 4) & 0x0F0F0F0Fu;
              // bytes (q0,q1,q2,q3) -> 16-bit patterns magic|q for (q0,q1) and (q2,q3)
              const V2 e01 = P16::from_bits(__byte_perm(e, P16::kMagicBytes, 0x4140));
              const V2 e23 = P16::from_bits(__byte_perm(e, P16::kMagicBytes, 0x4342));
              const V2 o01 = P16::from_bits(__byte_perm(o, P16::kMagicBytes, 0x4140));
              const V2 o23 = P16::from_bits(__byte_perm(o, P16::kMagicBytes, 0x4342));
              even[2 * h] = P16::bits(__hmul2(__hsub2(e01, zz[2 * h]), sc[2 * h]));
              even[2 * h + 1] = P16::bits(__hmul2(__hsub2(e23, zz[2 * h + 1]), sc[2 * h + 1]));
              odd[2 * h] = P16::bits(__hmul2(__hsub2(o01, zz[2 * h]), sc[2 * h]));
              odd[2 * h + 1] = P16::bits(__hmul2(__hsub2(o23, zz[2 * h + 1]), sc[2 * h + 1]));
            }
          } else {
            // zero-points that are not small integers: the fp32 statement, verbatim
            const uint64_t w64 = (static_cast<uint64_t>(pk[i].y) << 32) | pk[i].x;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const V2 z = P16::from_bits(zw[j]);
              const float z0 = P16::lo(z), z1 = P16::hi(z);
              const float s0 = P16::lo(sc[j]), s1 = P16::hi(sc[j]);
              const uint32_t b0 = static_cast<uint32_t>(w64 >> (16 * j)) & 0xFFu;
              const uint32_t b1 = static_cast<uint32_t>(w64 >> (16 * j + 8)) & 0xFFu;
              even[j] = P16::bits(P16::make(__fmul_rn(__fsub_rn(static_cast<float>(b0 & 15u), z0), s0),
                                            __fmul_rn(__fsub_rn(static_cast<float>(b1 & 15u), z1), s1)));
              odd[j] = P16::bits(P16::make(__fmul_rn(__fsub_rn(static_cast<float>(b0 >> 4), z0), s0),
                                           __fmul_rn(__fsub_rn(static_cast<float>(b1 >> 4), z1), s1)));
            }
          }
          // rows r_even and r_even+1 of the operand: 128 B per 64 columns, 16-byte
          // chunks xor-swizzled with the row index inside each group of 8 rows
          *reinterpret_cast<uint4*>(deq + r_even * 128 + ((chunk ^ (r_even & 7)) << 4)) =
              make_uint4(even[0], even[1], even[2], even[3]);
          *reinterpret_cast<uint4*>(deq + (r_even + 1) * 128 + ((chunk ^ ((r_even + 1) & 7)) << 4)) =
              make_uint4(odd[0], odd[1], odd[2], odd[3]);
        }
        fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_deq_full + 8 * sd);
      }
    }
  } else if (warp >= 4 + C::kDeqWarps) {
    // -------------------------------- epilogue --------------------------------
    const int quarter = warp & 3;
    const int n_local = quarter * 32 + lane;   // TMEM lane = weight column inside the tile
    const int et = threadIdx.x - (128 + C::kDeqWarps * 32);
    grid_dependency_wait();
    T* c = static_cast<T*>(p.c);
    const T* bias = static_cast<const T*>(p.bias);
    uint32_t seg = 0;
    {
      long long u = u_begin;
      while (u < u_end) {
        const int mtile = static_cast<int>(u / units);
        const int m0 = mtile * p.mt;
        const long long ul = u - static_cast<long long>(mtile) * units;
        const int tile = static_cast<int>(ul / p.k_steps);
        const int step0 = static_cast<int>(ul - static_cast<long long>(tile) * p.k_steps);
        const long long tile_end = u - step0 + p.k_steps;
        const long long seg_end = tile_end < u_end ? tile_end : u_end;
        const bool whole = (step0 == 0) && (seg_end == tile_end);
        // TA: the MMA issuers take alternate units of the CTA's run; in a one-unit segment
        // only one of them has written its accumulators
        bool issuer_has_units[C::kIssuers];
#pragma unroll
        for (int i = 0; i < C::kIssuers; ++i) {
          // units of the segment are it0 .. it0 + len - 1; issuer i owns those with it % kIssuers == i
          const long long it0 = u - u_begin, len = seg_end - u;
          const long long first = it0 + ((i - it0 % C::kIssuers) + C::kIssuers) % C::kIssuers;
          issuer_has_units[i] = first < it0 + len;
        }
        const uint32_t buf = seg & 1u, pacc = (seg >> 1) & 1u;
        ++seg;
        u = seg_end;
        if (!mbar_wait_long(wctx, bar_acc_full + 8 * buf, pacc, 0x500u + buf)) break;
        tc_fence_after_sync();
        const int n = tile * kTileN + n_local;
        const bool n_ok = n < p.n;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * (C::kAccs * MTMAX);
        // which slot of the tile this CTA's segment is
        // (only reached with a single token tile, where u indexes `units` directly)
        const int first_cta = whole ? 0 : cta_of_unit(units, ctas, static_cast<long long>(tile) * p.k_steps);
        const int last_cta = whole ? 0 : cta_of_unit(units, ctas, tile_end - 1);
        const int parts = last_cta - first_cta + 1;
        const int part = static_cast<int>(blockIdx.x) - first_cta;
        float* slot = p.slots + (static_cast<size_t>(tile) * p.max_parts + part) * (static_cast<size_t>(p.mt) * kTileN);
        const float bias_v = (whole && bias != nullptr && n_ok) ? to_f32<T>(bias[n]) : 0.f;
        for (int cc = 0; cc < p.mt; cc += 16) {
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
#pragma unroll
          for (int acc = 0; acc < C::kAccs; ++acc) {
            if (TA && !issuer_has_units[acc / (C::kAccs / C::kIssuers)]) continue;   // stale accumulators
            uint32_t r[16];
            tmem_ld(taddr + acc * MTMAX + cc, r);
            tmem_wait_ld(r);
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(r[j]);
          }
          if (whole) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = m0 + cc + j;
              if (m < p.m && n_ok) c[static_cast<size_t>(m) * p.n + n] = from_f32<T>(v[j] + bias_v);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) slot[(cc + j) * kTileN + n_local] = v[j];
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
        if (!whole) {
          // publish the partial, then find out whether this CTA completes the tile
          __threadfence();
          named_barrier_sync(1, 128);
          if (et == 0) {
            const unsigned int prev = atomicAdd(p.counters + tile, 1u);
            *last_flag = (prev == static_cast<unsigned int>(parts - 1)) ? 1u : 0u;
            if (prev == static_cast<unsigned int>(parts - 1)) p.counters[tile] = 0u;  // ready for the next launch
          }
          named_barrier_sync(1, 128);
          if (*last_flag != 0u) {
            __threadfence();
            const float* tile_slots = p.slots + static_cast<size_t>(tile) * p.max_parts * (static_cast<size_t>(p.mt) * kTileN);
            const float bv = (bias != nullptr && n_ok) ? to_f32<T>(bias[n]) : 0.f;
            // eight rows at a time, all their loads issued before any is consumed
            for (int mm0 = 0; mm0 < p.mt && m0 + mm0 < p.m; mm0 += 8) {
              float sum[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) sum[j] = 0.f;
              for (int q = 0; q < parts; ++q) {
                const float* src = tile_slots + (static_cast<size_t>(q) * p.mt + mm0) * kTileN + n_local;
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = __ldcg(src + j * kTileN);
#pragma unroll
                for (int j = 0; j < 8; ++j) sum[j] += v[j];
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int m = m0 + mm0 + j;
                if (m < p.m && n_ok) c[static_cast<size_t>(m) * p.n + n] = from_f32<T>(sum[j] + bv);
              }
            }
          }
          named_barrier_sync(1, 128);  // last_flag may be rewritten only after everyone has read it
        }
      }
    }
  }

  // ------------------------------- teardown -------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <typename T, int MTMAX, bool TA>
ks_status_t launch_t(const W4A16Args& a, const CUtensorMap& tm_w, const CUtensorMap& tm_s, const CUtensorMap& tm_z,
                     const CUtensorMap& tm_a, const Params& p, int grid, cudaStream_t stream) {
  using C = Cfg<MTMAX, TA>;
  auto kernel = w4a16_umma_kernel<T, MTMAX, TA>;
  static std::mutex mu;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
      if (e != cudaSuccess) return cuda_status(e, "ks_gemm_w4a16");
      attr_done[dev] = true;
    }
  }
  return cuda_status(launch_programmatic(kernel, static_cast<unsigned>(grid), C::kThreads, C::kSmemBytes, stream, tm_w,
                                         tm_s, tm_z, tm_a, p),
                     "ks_gemm_w4a16");
}

}  // namespace

bool w4a16_eligible(const W4A16Args& a) {
  if (a.k % kStepK != 0) return false;
  if (a.group_size % kStepK != 0) return false;   // one scale row per 128-k step
  if (a.n % 16 != 0) return false;                // 16-byte row pitch of the packed weight and of the scales
  if (!aligned16(a.a) || !aligned16(a.b_packed) || !aligned16(a.scales)) return false;
  if (a.zeros != nullptr && !aligned16(a.zeros)) return false;
  if (a.m > (1 << 24) || a.n > (1 << 28) || a.k > (1 << 28)) return false;
  return tma_available();
}

namespace {

struct Geometry {
  int mt = 0, mtmax = 0, n_tiles = 0, k_steps = 0, grid = 0, max_parts = 0;
  size_t counter_bytes = 0, slot_bytes = 0;
};

Geometry geometry_of(const W4A16Args& a) {
  Geometry g;
  const int mt_raw = static_cast<int>(a.m < 128 ? a.m : 128);
  g.mt = (mt_raw + 15) & ~15;
  g.mtmax = g.mt <= 32 ? 32 : 128;
  g.n_tiles = static_cast<int>((a.n + kTileN - 1) / kTileN);
  g.k_steps = static_cast<int>(a.k / kStepK);
  const long long units = static_cast<long long>(g.n_tiles) * g.k_steps;
  const int sms = sm_count();
  g.grid = static_cast<int>(units < sms ? units : sms);
  const long long per_cta = units / g.grid;  // shortest run
  g.max_parts = static_cast<int>((g.k_steps + per_cta - 1) / per_cta) + 1;
  g.slot_bytes = static_cast<size_t>(g.n_tiles) * g.max_parts * g.mt * kTileN * sizeof(float);
  g.counter_bytes = (static_cast<size_t>(g.n_tiles) * sizeof(unsigned int) + 255) & ~size_t(255);
  return g;
}

// Encodes the tensor maps and enqueues the kernel on scratch memory the caller of this
// function has already obtained: the per-tile arrival counters (all zero on entry; the
// kernel leaves them zero) and the fp32 partial slots.
ks_status_t enqueue_w4a16(const W4A16Args& a, const Geometry& g, unsigned int* counters, float* slots,
                          unsigned int* fault_word, cudaStream_t stream) {
  const bool bf16 = a.dtype == KS_DTYPE_BF16;
  const int mt = g.mt, mtmax = g.mtmax, n_tiles = g.n_tiles, k_steps = g.k_steps, grid = g.grid,
            max_parts = g.max_parts;
  const CUtensorMapDataType dt16 = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  // Decode shapes hand the weights over in tensor memory unless told otherwise; that path
  // loads the packed weight two K-steps at a time.
  const bool tmem_operand = mtmax == 32 && a.operand_path != 1 && (k_steps % 2 == 0);
  CUtensorMap tm_w, tm_s, tm_z, tm_a;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.k / 2)};
    const uint64_t str[1] = {static_cast<uint64_t>(a.n)};
    const uint32_t box[2] = {static_cast<uint32_t>(kTileN), static_cast<uint32_t>(tmem_operand ? kStepK : kStepK / 2)};
    if (!tma_encode(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.b_packed, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE))
      KSB_FAIL(KS_ERROR_INTERNAL, "ks_gemm_w4a16: tensor map for the packed weight rejected");
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.k / a.group_size)};
    const uint64_t str[1] = {static_cast<uint64_t>(a.n) * 2};
    const uint32_t box[2] = {static_cast<uint32_t>(kTileN), 1u};
    if (!tma_encode(&tm_s, dt16, 2, a.scales, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE))
      KSB_FAIL(KS_ERROR_INTERNAL, "ks_gemm_w4a16: tensor map for the scales rejected");
    if (!tma_encode(&tm_z, dt16, 2, a.zeros != nullptr ? a.zeros : a.scales, dims, str, box,
                    CU_TENSOR_MAP_SWIZZLE_NONE))
      KSB_FAIL(KS_ERROR_INTERNAL, "ks_gemm_w4a16: tensor map for the zero-points rejected");
  }
  if (tmem_operand) {
    // A[M,K] seen as [K/64][M][64]: one box brings both 64-k swizzle atoms of a K-step
    const uint64_t dims[3] = {64u, static_cast<uint64_t>(a.m), static_cast<uint64_t>(a.k / 64)};
    const uint64_t str[2] = {static_cast<uint64_t>(a.k) * 2, 128u};
    const uint32_t box[3] = {64u, static_cast<uint32_t>(mt), 2u};
    if (!tma_encode(&tm_a, dt16, 3, a.a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      KSB_FAIL(KS_ERROR_INTERNAL, "ks_gemm_w4a16: tensor map for the activations rejected");
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.m)};
    const uint64_t str[1] = {static_cast<uint64_t>(a.k) * 2};
    const uint32_t box[2] = {64u, static_cast<uint32_t>(mt)};
    if (!tma_encode(&tm_a, dt16, 2, a.a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      KSB_FAIL(KS_ERROR_INTERNAL, "ks_gemm_w4a16: tensor map for the activations rejected");
  }

  Params p;
  p.c = a.c;
  p.bias = a.bias;
  p.scales = a.scales;
  p.zeros = a.zeros;
  p.counters = counters;
  p.slots = slots;
  p.fault_word = fault_word;
  p.m = static_cast<int>(a.m);
  p.n = static_cast<int>(a.n);
  p.k = static_cast<int>(a.k);
  p.mt = mt;
  p.m_tiles = static_cast<int>((a.m + mt - 1) / mt);
  p.n_tiles = n_tiles;
  p.k_steps = k_steps;
  p.gs_steps = a.group_size / kStepK;
  p.max_parts = max_parts;
  p.has_zeros = a.zeros != nullptr ? 1 : 0;
  const uint32_t fmt = bf16 ? 1u : 0u;
  // weights: MN-major in shared memory, K along the columns in tensor memory
  p.idesc = umma_instr_desc(fmt, fmt, tmem_operand ? 0u : 1u, 0u, 128u, static_cast<uint32_t>(mt));

  if (bf16) {
    if (tmem_operand) return launch_t<__nv_bfloat16, 32, true>(a, tm_w, tm_s, tm_z, tm_a, p, grid, stream);
    return mtmax == 32 ? launch_t<__nv_bfloat16, 32, false>(a, tm_w, tm_s, tm_z, tm_a, p, grid, stream)
                       : launch_t<__nv_bfloat16, 128, false>(a, tm_w, tm_s, tm_z, tm_a, p, grid, stream);
  }
  if (tmem_operand) return launch_t<__half, 32, true>(a, tm_w, tm_s, tm_z, tm_a, p, grid, stream);
  return mtmax == 32 ? launch_t<__half, 32, false>(a, tm_w, tm_s, tm_z, tm_a, p, grid, stream)
                     : launch_t<__half, 128, false>(a, tm_w, tm_s, tm_z, tm_a, p, grid, stream);
}

}  // namespace

// Which fast kernel. The register-operand decode kernel feeds legacy mma.sync, whose rate on
// this part is about a tenth of tcgen05's (measured: ~100 bf16 FMA per clock and SM
// sub-partition): up to 8 tokens (one MMA per 16 x 16 weight block) it is well ahead of the
// tcgen05 kernel on wide weights (K=4096, N=28672, queued launches: 24.6 us against 29.7), at
// 16 tokens slightly (29.0 against 30.4), beyond that it is MMA-bound (32 tokens: 41 us
// against 33). On problems with few units per CTA (K=14336, N=4096: 6 per CTA) its pipeline
// fill and the split-K fix-up of every CTA cost what they save (19.8 us against 19.1).
// Chosen: at most 16 tokens and at least 10 units per CTA; the caller can pin either kernel.
bool use_decode_kernel(const W4A16Args& a) {
  if (a.kernel == 1 || !decode::eligible(a)) return false;
  if (a.kernel == 2 || !w4a16_eligible(a)) return true;
  const long long units = ((a.n + 255) / 256) * (a.k / 128);
  return a.m <= 16 && units >= 20ll * sm_count();
}

ks_status_t launch_w4a16(const W4A16Args& a, cudaStream_t stream) {
  // Counters and slots are separate allocations: the counters must be zero whenever no
  // kernel is running, and a region that another shape used for partial sums is not.
  // The tcgen05 kernels can give up on a bounded wait and leave counters non-zero; when
  // the fault poll has reported such a launch on this device, every stream's counters are
  // cleared before their next use (stream_scratch_dirty).
  const bool dec = use_decode_kernel(a);
  const Geometry g = dec ? Geometry{} : geometry_of(a);
  const decode::Geometry gd = dec ? decode::geometry_of(a) : decode::Geometry{};
  const size_t slot_bytes = dec ? gd.slot_bytes : g.slot_bytes;
  const size_t counter_bytes = dec ? gd.counter_bytes : g.counter_bytes;
  float* slots = static_cast<float*>(stream_scratch(stream, slot_bytes, 0));
  unsigned int* counters = static_cast<unsigned int*>(stream_scratch(stream, counter_bytes, 1));
  if (slots == nullptr || counters == nullptr)
    KSB_FAIL(KS_ERROR_OUT_OF_MEMORY, "ks_gemm_w4a16: workspace allocation failed");
  if (std::getenv("KS_B200_ENV_RELOAD") != nullptr && std::getenv("KS_B200_TEST_DIRTY_COUNTERS") != nullptr) {
    // test hook: what a launch that gave up half-way leaves behind, without any GPU fault:
    // garbage in the counters and the mark that the fault poll would have set
    cudaMemsetAsync(counters, 0xFF, stream_scratch_bytes(stream, 1), stream);
    stream_scratch_mark_dirty(1);
  }
  if (stream_scratch_take_dirty(stream, 1)) {
    cudaError_t e = cudaMemsetAsync(counters, 0, stream_scratch_bytes(stream, 1), stream);
    if (e != cudaSuccess) return cuda_status(e, "ks_gemm_w4a16: clearing the split-K counters");
  }
  if (dec) return decode::enqueue(a, gd, counters, slots, stream);
  return enqueue_w4a16(a, g, counters, slots, kernel_fault_word(), stream);
}

// ---------------------------------------------------------------------------
// Variant for callers that must not allocate: the split-K slots and counters
// live in a fixed array inside the library image instead of scratch memory
// obtained from the CUDA allocator.
//
// `g_static_scratch` below is a __device__ array. In host code its name only
// stands for the symbol: it is not an address a kernel may dereference. The
// device address is asked for once per device (with that device current) with
// cudaGetSymbolAddress, and that pointer is what the kernel receives.
// ---------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;  // 16 MiB on every GPU that loads the library
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_static_mutex;
void* g_static_ptr[64] = {};

// Device address of the array on the current device; resolved on the first
// call per device. No allocation is involved.
ks_status_t static_scratch_address(uint8_t** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e, "ks_gemm_w4a16_static_scratch");
  if (dev < 0 || dev >= 64)
    KSB_FAIL(KS_ERROR_INTERNAL, "ks_gemm_w4a16_static_scratch: device ordinal out of the supported range");
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return cuda_status(e, "ks_gemm_w4a16_static_scratch: cudaGetSymbolAddress");
    if (ptr == nullptr)
      KSB_FAIL(KS_ERROR_INTERNAL, "ks_gemm_w4a16_static_scratch: the scratch symbol resolved to a null address");
    g_static_ptr[dev] = ptr;
  }
  *out = static_cast<uint8_t*>(g_static_ptr[dev]);
  return KS_SUCCESS;
}

}  // namespace

size_t w4a16_static_scratch_capacity() { return kStaticScratchBytes; }

ks_status_t launch_w4a16_static(const W4A16Args& a, cudaStream_t stream) {
  const bool dec = use_decode_kernel(a);
  const Geometry g = dec ? Geometry{} : geometry_of(a);
  const decode::Geometry gd = dec ? decode::geometry_of(a) : decode::Geometry{};
  const size_t counter_bytes = dec ? gd.counter_bytes : g.counter_bytes;
  // With several token tiles the tcgen05 kernel snaps its runs to whole column tiles and
  // never touches the partial slots.
  const size_t slot_bytes = dec ? gd.slot_bytes : (a.m > 128 ? 0 : g.slot_bytes);
  const size_t need = counter_bytes + slot_bytes;
  if (need > kStaticScratchBytes) {
    char msg[224];
    snprintf(msg, sizeof(msg),
             "ks_gemm_w4a16_static_scratch: this shape needs %zu bytes of split-K scratch, the built-in array "
             "holds %zu; use ks_gemm_w4a16 or fewer rows per call",
             need, kStaticScratchBytes);
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, msg);
  }
  uint8_t* scratch = nullptr;
  ks_status_t st = static_scratch_address(&scratch);
  if (st != KS_SUCCESS) return st;
  // The array keeps whatever the previous call left. The kernels require the
  // arrival counters to be zero on entry (a clean run leaves them so, an aborted
  // one may not, and another shape lays them out differently); the slots are
  // fully overwritten before being read.
  cudaError_t e = cudaMemsetAsync(scratch, 0, counter_bytes, stream);
  if (e != cudaSuccess) return cuda_status(e, "ks_gemm_w4a16_static_scratch: cudaMemsetAsync");
  unsigned int* counters = reinterpret_cast<unsigned int*>(scratch);
  float* slots = reinterpret_cast<float*>(scratch + counter_bytes);
  if (dec) return decode::enqueue(a, gd, counters, slots, stream);
  // The word through which a tcgen05 kernel reports a bounded wait that ran out is a pinned
  // host allocation made by the first allocating entry point on the device; a process that
  // only ever calls this entry point runs the tcgen05 kernel without it (the decode kernel
  // has no such wait).
  return enqueue_w4a16(a, g, counters, slots, kernel_fault_word_if_ready(), stream);
}

}  // namespace sm100
}  // namespace ksb

