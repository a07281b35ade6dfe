// FP8 block-scaled GEMM for sm_100a: TMA-fed shared-memory ring, tcgen05.mma
// (kind::f8f6f4) into double-buffered TMEM partials, and an fp32 promotion of
// every 128-deep K-block partial by a_scale * b_scale in the epilogue warps.
//
// Computes what ks_gemm_fp8_blockwise / _nt / ks_moe_grouped_gemm_fp8_blockwise
// declare, for block_n = block_k = 128 (reference algebra:
// kernels/src/gemm/gemm_fp8_blockwise.cu:107-150 — an fp32 inner product per
// K-block, folded into the fp32 output with the block's scale product).
//
// CTA anatomy (one CTA per SM, persistent over output tiles of 128 x BN):
//   warp 0      TMA producer: A tile 128 x 128 B and B tile BN x 128 B per stage,
//               128-byte swizzle, completion counted on the stage's `full` barrier
//   warp 1      MMA issuer: 4 UMMAs (M128, N=BN, K32) per K-block into one of the TMEM
//               accumulator buffers (two of 256 columns, four of 128); ONE
//               tcgen05.commit per K-block both releases the stage to the producer
//               and tells the epilogue that the partial product is complete
//   warps 2,3   idle (they complete warpgroup 0 so that register budgets can be
//               moved between warpgroups with setmaxnreg)
//   warps 4-11  epilogue: warp w reads TMEM lanes 32*(w%4).. and BN/2 columns in
//               16-column loads, double-buffered so that one load is in flight
//               while the previous one is folded in:
//               acc = fma(partial, a_scale[row,kb] * b_scale[kb,nb], acc) in
//               registers (packed two-wide), frees the TMEM buffer, and after
//               the last K-block rounds once to the output type. Dense problems
//               stage the tile in swizzled shared memory and leave by TMA store;
//               grouped and unaligned ones store row segments from registers.
// Last partial round of a dense problem: when T tiles leave T mod #CTAs tiles for a final
// round that would keep most SMs idle (896 tiles on 148 SMs: 8 tiles, 140 idle SMs for a
// whole tile time), those tiles are cut along K into S parts (S <= 8, parts x tiles <=
// #CTAs), each a CTA's first work item. A part's epilogue warps write their fp32 partial to
// a slot; split_reduce_kernel, launched behind the GEMM on the same stream, adds the parts in
// part order (reproducible) and writes the tiles. (Letting the last part to arrive reduce a
// tile inside the GEMM kernel measured 3-4 % gain instead of the 10 % the idle round costs:
// one CTA then reads S x 128 KB behind a fence and four dependent atomics while its tensor
// core waits.)
// Measured on B200 with work-skipping builds of this kernel (M=4096, N=K=7168; the full kernel
// 201-204 us): MMAs and operand loads without any epilogue work 152 us (TMA writes 48 KB and
// the MMAs read 48 KB of shared memory per K-block; MMAs alone, from resident shared memory,
// 125 us); the epilogue alone 155 us, of which the eight TMEM loads per K-block are nearly
// free and the 128 FMAs per thread cost ~540 cycles (two epilogue warps per scheduler), the
// scale fetches ~10 %; barriers alone 58 us. The two sides are equally long and the two
// accumulator buffers couple them instead of letting them overlap fully. Measured and not
// better: handing the accumulator over in two 128-column halves (eight N=128 MMAs per
// K-block read A twice: 232 us), wider loads, more loads in flight, sixteen narrower epilogue
// warps, 224-wide tiles, scalar FMAs, paced MMA issue, sleeping or spinning waits.
// B may be stored [N,K] (K-major UMMA operand) or [K,N] (MN-major operand, the
// layout of the reference C ABI); both are loaded by TMA without a transpose.
//
// Roofline: tensor-bound for M >= ~1024 (2*M*N*K flop over 4.5 PFLOP/s dense
// FP8); bytes per launch M*K + N*K + M*N*sizeof(out) + scales.
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "sm100_fp8_gemm.cuh"
#include "sm100_fp8_store.cuh"
#include "sm100_host.cuh"
#include "sm100_ptx.cuh"

namespace ksb {
namespace sm100 {
namespace {

#ifndef KSB_FP8_EPI_COLS
#define KSB_FP8_EPI_COLS 128
#endif
#ifndef KSB_FP8_ACC_BUFS_128
#define KSB_FP8_ACC_BUFS_128 4
#endif
#ifndef KSB_FP8_PANEL
#define KSB_FP8_PANEL 4
#endif
#ifndef KSB_FP8_SCALE_GROUP
#define KSB_FP8_SCALE_GROUP 2
#endif
#ifndef KSB_FP8_EPI_CHUNK
#define KSB_FP8_EPI_CHUNK 16
#endif

constexpr int kBM = 128;
constexpr int kBK = 128;
constexpr int kMaxExperts = 1024;

template <int BN>
struct Cfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = kBM * kBK;
  static constexpr int kBBytes = BN * kBK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // An epilogue warp owns 32 TMEM lanes x kEpiCols columns. Narrow slices keep
  // the per-K-block chain (wait, TMEM loads, FMAs, release) short: with 64
  // columns it is ~440 cycles, under the ~512 the MMAs of a K-block take.
  static constexpr int kEpiCols = BN == 256 ? KSB_FP8_EPI_COLS : 64;
  static constexpr int kEpiWarps = (BN / kEpiCols) * 4;
  static constexpr int kThreads = 128 + kEpiWarps * 32;
  // Warpgroup 0 (TMA, MMA issue) hands registers to the epilogue warpgroups,
  // which hold the accumulators plus the TMEM values in flight. The budgets must add up to no more than
  // the CTA's launch-time pool (threads x launch registers): setmaxnreg.inc
  // blocks, without a time limit, until the pool can satisfy it.
  static constexpr bool kRebalanceRegs = (BN == 256);
  // 64-column slices: 20 warps, 96 registers at launch -> 32 / 112.
  // 128-column slices: 12 warps, 168 registers at launch -> 40 / 232.
  static constexpr int kRegsIssue = kEpiCols == 64 ? 32 : 40;
  static constexpr int kRegsEpi = kEpiCols == 64 ? 112 : 232;
  // Accumulator buffers in TMEM (512 columns): the MMA warp runs this many K-blocks
  // ahead of the epilogue. A K-block's round trip (issue -> complete -> drained ->
  // handed back) is about 1400 cycles whatever the tile width, so narrow tiles,
  // whose MMAs are short, need more buffers in flight to keep the tensor core fed.
  static constexpr int kAccBufs = BN == 256 ? 2 : KSB_FP8_ACC_BUFS_128;
  static constexpr int kTmemCols = 512;
  // Dense problems stage the finished tile for TMA stores: 32 rows x 128 B per epilogue warp.
  static constexpr int kStoreStageBytes = 32 * 128;
  // ring + 1024 B alignment slack + barriers/flags, then either the store staging
  // (dense) or the tile prefix, first rows and end rows of the experts (grouped)
  static constexpr int smem_bytes(bool grouped) {
    return kStages * kStageBytes + 1024 + 256 +
           (grouped ? 3 * 4 * (kMaxExperts + 1) : kEpiWarps * kStoreStageBytes);
  }
};

struct Params {
  void* out;
  const float* a_scale;
  const float* b_scale;
  const int32_t* offsets;  // [E+1] when grouped
  unsigned int* fault_word;
  int num_experts;
  int m;        // rows of A (all experts together when grouped)
  int n, k;
  int nkb, nnb;
  int tiles_n;
  int tiles_m;  // dense only
  uint32_t idesc;
  int vec_store;  // 16-byte output stores are legal
  int tma_store;  // dense problems: finished tiles leave through shared memory and TMA stores
  // K-split of the last partial round (dense only): work items [0, split_from) are whole
  // tiles; item split_from + r is part r % split_s of tile split_from + r / split_s.
  int split_from;
  int split_items;        // number of K-part items (tail tiles x split_s), at most the grid size
  int split_s;            // 1 = no split
  float4* split_slots;    // [tail tile][part][epilogue warp][16-byte column chunk][lane]
  // MODE 1 / 2 (one scale per row and per column, the whole K range accumulated in TMEM)
  int64_t as_row_stride, as_kb_stride;   // a_scale[row * as_row_stride + kb * as_kb_stride]
  const void* bias;       // [N] in the output type or NULL
  int a_per_row;          // a_scale is [M] (else one value)
  int b_per_col;          // b_scale is [N] (else one value)
  // grouped, masked layout: expert e owns rows [e * max_m, e * max_m + masked_m[e])
  const int32_t* masked_m;
  int max_m;
  // scattered output (dense, TMA-store epilogue only): rows [b * rows_per_part, (b + 1) *
  // rows_per_part) leave through output tensor map b, as rows 0.. of that map; 0 = one output
  int rows_per_part;
};

// Output tensor maps: one, or one per destination of a scattered output.
constexpr int kMaxOutParts = 8;
struct OutMaps {
  CUtensorMap m[kMaxOutParts];
};

struct TileCoord {
  int expert, row0, row_end, n0;
  int kb0, kb1;   // K-blocks of this work item
  int part;       // -1: whole tile; else index of this K-part
  int tail;       // index of the tile among the split tiles
};

template <int BN, bool GROUPED>
__device__ __forceinline__ bool locate_tile(const Params& p, const int* prefix, const int* offs, int t,
                                            TileCoord* tc) {
  if constexpr (!GROUPED) {
    tc->kb0 = 0;
    tc->kb1 = p.nkb;
    tc->part = -1;
    tc->tail = 0;
    if (t >= p.split_from) {
      const int r = t - p.split_from;
      tc->tail = r / p.split_s;
      tc->part = r - tc->tail * p.split_s;
      tc->kb0 = (tc->part * p.nkb) / p.split_s;
      tc->kb1 = ((tc->part + 1) * p.nkb) / p.split_s;
      t = p.split_from + tc->tail;
    }
    if (t >= p.tiles_m * p.tiles_n) return false;
    // Column panels of kPanel tiles, all row tiles of a panel before the next panel: the
    // tiles in flight at any time then share a few B panels and sweep A, so the set that has
    // to stay in L2 between rounds is A (small) instead of all of B.
    constexpr int kPanel = KSB_FP8_PANEL;
    const int per_panel = kPanel * p.tiles_m;
    const int panel = t / per_panel;
    const int r = t - panel * per_panel;
    const int width = (p.tiles_n - panel * kPanel) < kPanel ? (p.tiles_n - panel * kPanel) : kPanel;
    const int mt = r / width;
    const int nt = panel * kPanel + (r - mt * width);
    tc->expert = 0;
    tc->row0 = mt * kBM;
    tc->row_end = p.m;
    tc->n0 = nt * BN;
    return true;
  } else {
    tc->kb0 = 0;
    tc->kb1 = p.nkb;
    tc->part = -1;
    tc->tail = 0;
    const int total_mt = prefix[p.num_experts];
    if (t >= total_mt * p.tiles_n) return false;
    const int mt = t / p.tiles_n;
    int lo = 0, hi = p.num_experts - 1;  // last e with prefix[e] <= mt
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (prefix[mid] <= mt) lo = mid; else hi = mid - 1;
    }
    tc->expert = lo;
    tc->row0 = offs[lo] + (mt - prefix[lo]) * kBM;
    tc->row_end = offs[kMaxExperts + 1 + lo];   // ends[lo]
    tc->n0 = (t - mt * p.tiles_n) * BN;
    return true;
  }
}

// Work items of a CTA in the order it processes them: its K-part of a split tile first (if
// it has one), then whole tiles blockIdx.x, blockIdx.x + gridDim.x, ...
struct ItemWalk {
  int n;
  __device__ explicit ItemWalk(const Params& p)
      : n((p.split_s > 1 && static_cast<int>(blockIdx.x) < p.split_items) ? -1 : 0) {}
  template <int BN, bool GROUPED>
  __device__ __forceinline__ bool next(const Params& p, const int* prefix, const int* offs, TileCoord* tc) {
    const int t = n < 0 ? p.split_from + static_cast<int>(blockIdx.x)
                        : static_cast<int>(blockIdx.x) + n * static_cast<int>(gridDim.x);
    if (n >= 0 && t >= p.split_from) return false;
    ++n;
    return locate_tile<BN, GROUPED>(p, prefix, offs, t, tc);
  }
};

static_assert(Cfg<256>::smem_bytes(false) <= 232448 && Cfg<256>::smem_bytes(true) <= 232448 &&
                  Cfg<128>::smem_bytes(false) <= 232448 && Cfg<128>::smem_bytes(true) <= 232448,
              "shared memory layout exceeds the 227 KB a CTA can opt in to");
static_assert(128 * Cfg<256>::kRegsIssue + (Cfg<256>::kThreads - 128) * Cfg<256>::kRegsEpi <=
                  Cfg<256>::kThreads * ((65536 / Cfg<256>::kThreads) & ~7),
              "setmaxnreg budgets exceed the register pool the CTA is launched with");

// MODE 0: block-scaled FP8 (a partial per K-block, promoted in registers).
// MODE 1: FP8 with one scale per row of A and one per column of B: the whole K range
//         accumulates in tensor memory, the epilogue runs once per tile.
// MODE 2: the same with int8 operands (kind::i8, int32 accumulators) and an optional bias.
// MODE 3: f16 / bf16 operands (kind::f16), no scales: a K-block is 64 elements (the same 128
//         bytes per row), B stored [K,N] is loaded in 64-column atoms. The unscaled grouped GEMM.
template <int BN, bool NT, bool GROUPED, typename OutT, int MODE = 0>
__global__ void __launch_bounds__(Cfg<BN>::kThreads, 1)
fp8_blockwise_umma_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                          const __grid_constant__ OutMaps tm_cs, const Params p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t ring = (raw_addr + 1023u) & ~1023u;  // 1024-byte aligned for the 128 B swizzle
  // dense: [ring | store staging | control]; grouped: [ring | control | prefix, offsets]
  constexpr int kStagingBytes = GROUPED ? 0 : C::kEpiWarps * C::kStoreStageBytes;
  const uint32_t staging = ring + C::kStages * C::kStageBytes;
  uint8_t* ctrl = smem_raw + (ring - raw_addr) + C::kStages * C::kStageBytes + kStagingBytes;
  const uint32_t ctrl_addr = staging + kStagingBytes;
  // control block: full[S] | empty[S] | tmem_empty[B] | tmem slot | abort flag
  const uint32_t bar_full = ctrl_addr;
  const uint32_t bar_empty = ctrl_addr + 8 * C::kStages;
  const uint32_t bar_tempty = ctrl_addr + 16 * C::kStages;
  const uint32_t bar_accfull = bar_tempty + 8 * C::kAccBufs;   // MODE 1 / 2: a tile's accumulator is complete
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 16 * C::kStages + 16 * C::kAccBufs);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  int* prefix = reinterpret_cast<int*>(ctrl + 256);
  int* offs = prefix + (kMaxExperts + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx wctx{abort_flag, p.fault_word};

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < C::kAccBufs; ++b) {
      mbar_init(bar_tempty + 8 * b, C::kEpiWarps);
      mbar_init(bar_accfull + 8 * b, 1);
    }
    *abort_flag = 0u;
    fence_barrier_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
    if (!GROUPED && p.tma_store) prefetch_tensormap(&tm_cs.m[0]);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
    tmem_relinquish();
  }
  if constexpr (GROUPED) {
    // offs[e] = first row of expert e; with the masked layout the rows of an expert end at
    // offs[e] + masked_m[e] instead of at offs[e + 1] (ends[] holds either)
    int* ends = offs + (kMaxExperts + 1);
    for (int e = threadIdx.x; e <= p.num_experts; e += blockDim.x) {
      if (p.masked_m != nullptr) {
        offs[e] = e * p.max_m;
        if (e < p.num_experts) {
          int mm = p.masked_m[e];
          mm = mm < 0 ? 0 : (mm > p.max_m ? p.max_m : mm);
          ends[e] = e * p.max_m + mm;
        }
      } else {
        offs[e] = p.offsets[e];
        if (e < p.num_experts) ends[e] = p.offsets[e + 1];
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = 0;
      for (int e = 0; e < p.num_experts; ++e) {
        prefix[e] = run;
        const int rows = ends[e] - offs[e];
        run += rows > 0 ? (rows + kBM - 1) / kBM : 0;
      }
      prefix[p.num_experts] = run;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if constexpr (C::kRebalanceRegs) setmaxnreg_dec<C::kRegsIssue>();
    uint32_t it = 0;
    bool ok = true;
    TileCoord tc;
    for (ItemWalk walk(p); ok && walk.template next<BN, GROUPED>(p, prefix, offs, &tc);) {
      for (int kb = tc.kb0; kb < tc.kb1; ++kb, ++it) {
        const uint32_t s = it % C::kStages;
        const uint32_t ph = (it / C::kStages) & 1u;
        if (!mbar_wait(wctx, bar_empty + 8 * s, ph ^ 1u, 0x100u + s)) { ok = false; break; }
        {
          const uint32_t full = bar_full + 8 * s;
          const uint32_t a_dst = ring + s * C::kStageBytes;
          const uint32_t b_dst = a_dst + C::kABytes;
          mbar_arrive_expect_tx_elect(full, C::kStageBytes);
          tma_load_2d_elect(a_dst, &tm_a, full, kb * kBK, tc.row0);
          if constexpr (NT) {
            tma_load_3d_elect(b_dst, &tm_b, full, kb * kBK, tc.n0, tc.expert);
          } else if constexpr (MODE == 3) {
            // the map sees B as bytes: 64 columns of 16 bits = one 128-byte atom, 64 k-rows per K-block
#pragma unroll
            for (int h = 0; h < BN / 64; ++h)
              tma_load_3d_elect(b_dst + h * (64 * 128), &tm_b, full, 2 * tc.n0 + h * 128, kb * 64, tc.expert);
          } else {
#pragma unroll
            for (int h = 0; h < BN / 128; ++h)
              tma_load_3d_elect(b_dst + h * (128 * kBK), &tm_b, full, tc.n0 + h * 128, kb * kBK, tc.expert);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if constexpr (C::kRebalanceRegs) setmaxnreg_dec<C::kRegsIssue>();
    uint32_t it = 0;
    uint32_t tile_n = 0;   // MODE 1 / 2: tiles so far (one accumulator buffer per tile)
    bool ok = true;
    TileCoord tc;
    for (ItemWalk walk(p); ok && walk.template next<BN, GROUPED>(p, prefix, offs, &tc);) {
      if constexpr (MODE != 0) {
        const uint32_t tbuf = tile_n % C::kAccBufs, tph = (tile_n / C::kAccBufs) & 1u;
        if (!mbar_wait(wctx, bar_tempty + 8 * tbuf, tph ^ 1u, 0x200u + tbuf)) { ok = false; break; }
      }
      for (int kb = tc.kb0; kb < tc.kb1; ++kb, ++it) {
        const uint32_t s = it % C::kStages;
        const uint32_t ph = (it / C::kStages) & 1u;
        const uint32_t buf = MODE != 0 ? tile_n % C::kAccBufs : it % C::kAccBufs;
        if constexpr (MODE == 0) {
          const uint32_t aph = (it / C::kAccBufs) & 1u;
          if (!mbar_wait(wctx, bar_tempty + 8 * buf, aph ^ 1u, 0x200u + buf)) { ok = false; break; }
        }
        if (!mbar_wait(wctx, bar_full + 8 * s, ph, 0x300u + s)) { ok = false; break; }
        tc_fence_after_sync();
        {
          // all 32 lanes run this code; each instruction elects its one issuing lane
          const uint32_t a_src = ring + s * C::kStageBytes;
          const uint32_t b_src = a_src + C::kABytes;
          const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
          for (int kk = 0; kk < kBK / 32; ++kk) {
            // A and (NT) B are K-major: 8-row groups 1024 B apart, a K step of 32
            // elements is 32 B inside the swizzle atom. B stored [K,N] is MN-major:
            // 128-column atoms 16 KB apart, 8-k groups 1024 B apart, a K step of 32
            // rows is 32 * 128 B.
            const uint64_t a_desc = umma_smem_desc_sw128(a_src + kk * 32, 16, 1024);
            // (16-bit operands, MODE 3: the same bytes per instruction, 16 elements; an MN-major
            // atom is 64 columns x 64 k-rows = 8 KB and a K step of 16 rows is 16 * 128 B)
            const uint64_t b_desc = NT ? umma_smem_desc_sw128(b_src + kk * 32, 16, 1024)
                                    : MODE == 3 ? umma_smem_desc_sw128(b_src + kk * 16 * 128, 64 * 128, 1024)
                                                : umma_smem_desc_sw128(b_src + kk * 32 * 128, 128 * kBK, 1024);
            const uint32_t accumulate = (kk > 0 || (MODE != 0 && kb > tc.kb0)) ? 1u : 0u;
            if constexpr (MODE == 2) umma_i8_elect(d_tmem, a_desc, b_desc, p.idesc, accumulate);
            else if constexpr (MODE == 3) umma_f16_elect(d_tmem, a_desc, b_desc, p.idesc, accumulate);
            else umma_f8f6f4_elect(d_tmem, a_desc, b_desc, p.idesc, accumulate);
          }
          tc_commit_elect(bar_empty + 8 * s);
          if constexpr (MODE != 0) {
            if (kb == tc.kb1 - 1) tc_commit_elect(bar_accfull + 8 * buf);
          }
        }
      }
      ++tile_n;
    }
  } else if (warp >= 4) {
    // -------------------------------- epilogue --------------------------------
    if constexpr (C::kRebalanceRegs) setmaxnreg_inc<C::kRegsEpi>();
    const int quarter = warp & 3;         // TMEM lane quarter this warp can address
    const int slice = (warp - 4) >> 2;    // which kEpiCols-wide column slice of the tile
    constexpr int EC = C::kEpiCols;
    const int row_in_tile = quarter * 32 + lane;
    OutT* out = static_cast<OutT*>(p.out);
    uint32_t it = 0;
    uint32_t tile_n = 0;   // MODE 1 / 2: tiles so far
    bool ok = true;
    TileCoord tc;
    for (ItemWalk walk(p); ok && walk.template next<BN, GROUPED>(p, prefix, offs, &tc);) {
      const int row = tc.row0 + row_in_tile;
      const bool row_ok = row < tc.row_end;
      const int col0 = tc.n0 + slice * EC;
      int nb = col0 >> 7;
      if (nb > p.nnb - 1) nb = p.nnb - 1;
      const float* as_ptr = MODE == 3 ? nullptr : p.a_scale + static_cast<size_t>(row_ok ? row : 0) * p.as_row_stride;
      const float* bs_ptr = MODE == 3 ? nullptr
                                      : p.b_scale + static_cast<size_t>(tc.expert) * p.nkb * p.nnb +
                                            (NT ? static_cast<size_t>(nb) * p.nkb : static_cast<size_t>(nb));
      const size_t bs_step = NT ? 1 : static_cast<size_t>(p.nnb);

      float2 acc[EC / 2];
#pragma unroll
      for (int i = 0; i < EC / 2; ++i) acc[i] = make_float2(0.f, 0.f);

      if constexpr (MODE != 0) {
        // the tile's accumulator is complete: scale by a_scale[row] * b_scale[col] (and add
        // the bias) on the way out of tensor memory, as kernels/src/gemm/gemm_fp8.cu:147-153
        // and gemm_w8a8.cu:134-141 of the reference do
        const uint32_t tbuf = tile_n % C::kAccBufs, tph = (tile_n / C::kAccBufs) & 1u;
        ++tile_n;
        if (!mbar_wait_long(wctx, bar_accfull + 8 * tbuf, tph, 0x400u + tbuf)) { ok = false; break; }
        tc_fence_after_sync();
        float a_sc = 1.f, b_one = 1.f;
        if constexpr (MODE != 3) {
          a_sc = (p.a_per_row && row_ok) ? __ldg(p.a_scale + row) : __ldg(p.a_scale);
          b_one = __ldg(p.b_scale);
        }
        const OutT* bias = static_cast<const OutT*>(p.bias);
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + tbuf * BN + slice * EC;
#pragma unroll
        for (int c = 0; c < EC / 16; ++c) {
          uint32_t r[16];
          tmem_ld(taddr + c * 16, r);
          tmem_wait_ld(r);
          if (c == EC / 16 - 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * tbuf);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int col = col0 + c * 16 + j;
            const bool col_ok = col < p.n;
            const float raw = MODE == 2 ? static_cast<float>(static_cast<int32_t>(r[j])) : __uint_as_float(r[j]);
            float v = raw;
            if constexpr (MODE != 3) {
              const float b_sc = (p.b_per_col && col_ok) ? __ldg(p.b_scale + col) : b_one;
              v = __fmul_rn(__fmul_rn(raw, a_sc), b_sc);
              if (bias != nullptr && col_ok) v = __fadd_rn(v, to_f32<OutT>(bias[col]));
            }
            if (j & 1) acc[c * 8 + (j >> 1)].y = v; else acc[c * 8 + (j >> 1)].x = v;
          }
        }
      }

      // Scales are fetched two K-blocks at a time, one group ahead of use: an
      // L2 round trip is longer than one K-block, so a load issued for the next
      // block alone would sit on the critical path.
      constexpr int G = KSB_FP8_SCALE_GROUP;
      constexpr int CW = KSB_FP8_EPI_CHUNK;  // TMEM columns per load
      float as_nxt[G], bs_nxt[G];
      auto fetch_scales = [&](int kb0) {
#pragma unroll
        for (int j = 0; j < G; ++j) {
          const int kb = kb0 + j;
          const bool in = kb < tc.kb1;
          as_nxt[j] = (in && row_ok) ? __ldg(as_ptr + kb * p.as_kb_stride) : 0.f;
          bs_nxt[j] = in ? __ldg(bs_ptr + static_cast<size_t>(kb) * bs_step) : 0.f;
        }
      };
      if constexpr (MODE == 0) fetch_scales(tc.kb0);

      for (int kb0 = tc.kb0; MODE == 0 && kb0 < tc.kb1 && ok; kb0 += G) {
        float sc[G];
#pragma unroll
        for (int j = 0; j < G; ++j) sc[j] = as_nxt[j] * bs_nxt[j];
        fetch_scales(kb0 + G);
#pragma unroll
        for (int j4 = 0; j4 < G; ++j4) {
          if (kb0 + j4 >= tc.kb1) break;
          const float2 scale2 = make_float2(sc[j4], sc[j4]);
          const uint32_t buf = it % C::kAccBufs;
          const uint32_t aph = (it / C::kAccBufs) & 1u;
          ++it;
          // short suspend hint: these warps are the critical path of every K-block, and a
          // waiter parked for the default period is resumed later than one that re-polls
          // One tcgen05.commit per K-block serves both consumers: the barrier that hands the
          // shared-memory stage back to the producer also tells the epilogue that the
          // accumulator is complete (each extra commit costs the tensor core ~50 idle cycles).
          {
            const uint32_t s_done = (it - 1) % C::kStages, ph_done = ((it - 1) / C::kStages) & 1u;
            if (!mbar_wait_hinted(wctx, bar_empty + 8 * s_done, ph_done, 0x400u + buf, 50u)) { ok = false; break; }
          }

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
              // every column of this warp's slice is in registers: hand the buffer back
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
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
      bool stored = false;
      if constexpr (!GROUPED) {
        if (ok && tc.part >= 0) {
          // One K-part of a split tile. The warp's 32 x EC partial goes to its slot (16 bytes
          // per lane and column chunk, chunks 512 B apart: every store of the warp is one
          // contiguous 512-byte piece); split_reduce_kernel adds the parts up afterwards.
          constexpr int kChunks = EC / 4;      // float4 chunks per lane
          const int ew = warp - 4;
          const size_t warp_f4 = static_cast<size_t>(kChunks) * 32;
          float4* mine = p.split_slots + ((static_cast<size_t>(tc.tail) * p.split_s + tc.part) * C::kEpiWarps + ew) * warp_f4 + lane;
#pragma unroll
          for (int c4 = 0; c4 < kChunks; ++c4)
            __stcg(mine + c4 * 32, make_float4(acc[2 * c4].x, acc[2 * c4].y, acc[2 * c4 + 1].x, acc[2 * c4 + 1].y));
          stored = true;
        }
        if (ok && !stored && p.tma_store) {
          // The warp's 32 x EC block leaves in pieces of 32 rows x 128 bytes: written
          // to shared memory in the 128-byte swizzle (conflict-free: lanes 0-7 hit eight
          // different 16-byte columns), then one TMA store, which clips rows and columns
          // outside the matrix. The next tile's K loop starts while the store drains.
          constexpr int kPieceCols = 128 / static_cast<int>(sizeof(OutT));
          constexpr int kChunkCols = 16 / static_cast<int>(sizeof(OutT));
          const uint32_t my_stage = staging + (warp - 4) * C::kStoreStageBytes;
          const int store_row = tc.row0 + quarter * 32;
          // a tile lies inside one part: rows_per_part is a multiple of the tile height
          const int part_of_tile = p.rows_per_part > 0 ? tc.row0 / p.rows_per_part : 0;
          const int part_row = store_row - part_of_tile * p.rows_per_part;
          const CUtensorMap* out_map = &tm_cs.m[part_of_tile];
#pragma unroll
          for (int pc = 0; pc < EC / kPieceCols; ++pc) {
            const int pcol = col0 + pc * kPieceCols;
            if (pcol >= p.n || store_row >= p.m) break;   // warp-uniform
            if (lane == 0) bulk_wait_group_read_all();     // the previous piece has left the buffer
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint4 w = pack_16_bytes<OutT>(acc, pc * kPieceCols + j * kChunkCols);
              st_shared_v4(my_stage + lane * 128 + ((j ^ (lane & 7)) << 4), w.x, w.y, w.z, w.w);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(out_map, my_stage, pcol, part_row);
              bulk_commit_group();
            }
          }
          stored = true;
        }
      }
      if (ok && row_ok && !stored) {
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
    if (lane == 0) bulk_wait_group_all();   // shared memory must outlive the stores that read it
  } else {
    // warps 2 and 3 only complete warpgroup 0
    if constexpr (C::kRebalanceRegs) setmaxnreg_dec<C::kRegsIssue>();
  }

  // ------------------------------- teardown -------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    // A wait gave up: give copies and MMAs still in flight time to land
    // before shared memory and TMEM are released.
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// Sum of the K-parts of the split tiles: one thread per (tile, epilogue warp, column chunk,
// lane) reads its 16 bytes of every part in part order and writes four outputs.
template <int BN, typename OutT>
__global__ void __launch_bounds__(256)
split_reduce_kernel(OutT* __restrict__ out, const float4* __restrict__ slots, int split_from, int split_s, int tails,
                    int tiles_m, int tiles_n, int m, int n, int vec_ok) {
  using C = Cfg<BN>;
  constexpr int EC = C::kEpiCols;
  constexpr int kChunks = EC / 4;
  constexpr int kPerTile = C::kEpiWarps * kChunks * 32;   // float4 per (tile, part)
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tails * kPerTile) return;
  const int tail = idx / kPerTile;
  const int r = idx - tail * kPerTile;
  const int ew = r / (kChunks * 32);
  const int c4 = (r / 32) % kChunks;
  const int lane = r & 31;
  // the tile's place in the output: the column-panel order of locate_tile
  constexpr int kPanel = KSB_FP8_PANEL;
  const int t = split_from + tail;
  const int per_panel = kPanel * tiles_m;
  const int panel = t / per_panel;
  const int rr = t - panel * per_panel;
  const int width = (tiles_n - panel * kPanel) < kPanel ? (tiles_n - panel * kPanel) : kPanel;
  const int mt = rr / width;
  const int nt = panel * kPanel + (rr - mt * width);
  const int row = mt * kBM + (ew & 3) * 32 + lane;
  const int col = nt * BN + (ew >> 2) * EC + 4 * c4;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4* src = slots + static_cast<size_t>(tail) * split_s * kPerTile + r;
  for (int q = 0; q < split_s; ++q) {
    const float4 v = __ldcs(src + static_cast<size_t>(q) * kPerTile);
    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
  }
  if (row >= m || col >= n) return;
  OutT* dst = out + static_cast<size_t>(row) * n + col;
  const float v4[4] = {sum.x, sum.y, sum.z, sum.w};
  if (vec_ok && col + 4 <= n) {
    if constexpr (std::is_same<OutT, float>::value) {
      *reinterpret_cast<float4*>(dst) = sum;
    } else {
      OutT o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = from_f32<OutT>(v4[j]);
      *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (col + j < n) dst[j] = from_f32<OutT>(v4[j]);
  }
}

// ------------------------------- host side --------------------------------
// Byte tensor of rank 2 or 3 (innermost first), 128-byte swizzled boxes.
bool encode_u8(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
               const uint32_t* box) {
  return tma_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, base, dims, strides_bytes, box,
                    CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int BN, bool NT, bool GROUPED, typename OutT, int MODE = 0>
ks_status_t launch_one(const Fp8GemmArgs& a, const CUtensorMap& tm_a, const CUtensorMap& tm_b, Params p,
                       int grid, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kernel = fp8_blockwise_umma_kernel<BN, NT, GROUPED, OutT, MODE>;
  static std::mutex mu;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
      cudaError_t e =
          cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::smem_bytes(GROUPED));
      if (e != cudaSuccess) return cuda_status(e, a.where);
      attr_done[dev] = true;
    }
  }
  // Output tensor map for the TMA-store epilogue (dense problems whose rows keep
  // 16-byte alignment); otherwise the kernel stores from registers.
  OutMaps tm_cs;
  for (int i = 0; i < kMaxOutParts; ++i) tm_cs.m[i] = tm_a;
  p.tma_store = 0;
  p.rows_per_part = 0;
  if (!GROUPED && p.vec_store) {
    const CUtensorMapDataType dt = std::is_same<OutT, float>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : std::is_same<OutT, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                       : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const uint64_t str[1] = {static_cast<uint64_t>(a.n) * sizeof(OutT)};
    const uint32_t box[2] = {static_cast<uint32_t>(128 / sizeof(OutT)), 32u};
    if (a.num_out_parts > 0) {
      // every part is a [rows_per_part, n] matrix of its own (possibly in another GPU's memory)
      bool ok = true;
      for (int i = 0; i < a.num_out_parts && ok; ++i) {
        const uint64_t dims[2] = {static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.rows_per_part)};
        ok = tma_encode(&tm_cs.m[i], dt, 2, a.out_parts[i], dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
      }
      if (ok) {
        p.tma_store = 1;
        p.rows_per_part = static_cast<int>(a.rows_per_part);
      }
    } else {
      const uint64_t dims[2] = {static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.m)};
      if (tma_encode(&tm_cs.m[0], dt, 2, a.out, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) p.tma_store = 1;
    }
  }
  if (a.num_out_parts > 0 && !p.tma_store)
    KSB_FAIL(KS_ERROR_UNSUPPORTED_SHAPE, std::string(a.where) + ": the scattered output needs 16-byte aligned rows and parts");
  // (Programmatic dependent launch was measured on the quantizer -> GEMM -> reducer chain and
  // lost 1 % there: these kernels have no input-independent prologue worth overlapping, and
  // the dependency wait costs more than an ordinary kernel boundary.)
  kernel<<<grid, C::kThreads, C::smem_bytes(GROUPED), stream>>>(tm_a, tm_b, tm_cs, p);
  if constexpr (!GROUPED) {
    if (p.split_s > 1) {
      const int tails = p.split_items / p.split_s;
      const int work = tails * C::kEpiWarps * (C::kEpiCols / 4) * 32;
      split_reduce_kernel<BN, OutT><<<(work + 255) / 256, 256, 0, stream>>>(
          static_cast<OutT*>(p.out), p.split_slots, p.split_from, p.split_s, tails, p.tiles_m, p.tiles_n, p.m, p.n,
          p.vec_store);
    }
  }
  return cuda_status(cudaGetLastError(), a.where);
}

template <int BN, bool NT, bool GROUPED, int MODE = 0>
ks_status_t launch_out(const Fp8GemmArgs& a, const CUtensorMap& tm_a, const CUtensorMap& tm_b, const Params& p,
                       int grid, cudaStream_t stream) {
  switch (a.out_dtype) {
    case KS_DTYPE_F32: return launch_one<BN, NT, GROUPED, float, MODE>(a, tm_a, tm_b, p, grid, stream);
    case KS_DTYPE_F16: return launch_one<BN, NT, GROUPED, __half, MODE>(a, tm_a, tm_b, p, grid, stream);
    default: return launch_one<BN, NT, GROUPED, __nv_bfloat16, MODE>(a, tm_a, tm_b, p, grid, stream);
  }
}

template <int BN>
ks_status_t launch_bn(const Fp8GemmArgs& a, const CUtensorMap& tm_a, const CUtensorMap& tm_b, const Params& p,
                      int grid, cudaStream_t stream) {
  const bool grouped = a.offsets != nullptr || a.masked_m != nullptr;
  // the per-row / per-column scaled kernels exist for the reference's layout (B stored [K,N]), dense
  if (a.mode == 1) return launch_out<BN, false, false, 1>(a, tm_a, tm_b, p, grid, stream);
  if (a.mode == 2) return launch_out<BN, false, false, 2>(a, tm_a, tm_b, p, grid, stream);
  // 16-bit operands, B stored [K,N]: the output has the operands' type
  if (a.mode == 3) {
    if (a.out_dtype == KS_DTYPE_F16)
      return grouped ? launch_one<BN, false, true, __half, 3>(a, tm_a, tm_b, p, grid, stream)
                     : launch_one<BN, false, false, __half, 3>(a, tm_a, tm_b, p, grid, stream);
    return grouped ? launch_one<BN, false, true, __nv_bfloat16, 3>(a, tm_a, tm_b, p, grid, stream)
                   : launch_one<BN, false, false, __nv_bfloat16, 3>(a, tm_a, tm_b, p, grid, stream);
  }
  if (a.nt) return grouped ? launch_out<BN, true, true>(a, tm_a, tm_b, p, grid, stream)
                           : launch_out<BN, true, false>(a, tm_a, tm_b, p, grid, stream);
  return grouped ? launch_out<BN, false, true>(a, tm_a, tm_b, p, grid, stream)
                 : launch_out<BN, false, false>(a, tm_a, tm_b, p, grid, stream);
}

}  // namespace

bool fp8_blockwise_eligible(const Fp8GemmArgs& a) {
  if (a.mode == 0 && (a.block_n != 128 || a.block_k != 128)) return false;
  if ((a.mode == 1 || a.mode == 2) && (a.nt || a.offsets != nullptr || a.masked_m != nullptr)) return false;
  if (a.mode == 3) {
    // 16-bit operands: 16-byte row pitches of A [M,K] and B [K,N]
    if (a.nt || a.masked_m != nullptr || a.k % 8 != 0 || a.n % 8 != 0) return false;
    if (a.out_dtype != KS_DTYPE_F16 && a.out_dtype != KS_DTYPE_BF16) return false;
  } else {
    if (a.k % 16 != 0) return false;
    if (!a.nt && a.n % 16 != 0) return false;
  }
  if (!aligned16(a.a) || !aligned16(a.b)) return false;
  if (a.m > INT32_MAX / 2 || a.n > INT32_MAX / 2 || a.k > INT32_MAX / 2) return false;
  if ((a.offsets != nullptr || a.masked_m != nullptr) && (a.num_experts > kMaxExperts || a.num_experts < 1)) return false;
  if (a.masked_m != nullptr && (a.max_m < 1 || a.max_m * a.num_experts != a.m)) return false;
  return tma_available();
}

ks_status_t launch_fp8_blockwise(const Fp8GemmArgs& a, cudaStream_t stream) {
  const bool grouped = a.offsets != nullptr || a.masked_m != nullptr;
  const int experts = grouped ? a.num_experts : 1;
  const int sms = sm_count();
  const int64_t tiles_m_bound = grouped ? (a.m + kBM - 1) / kBM + experts : (a.m + kBM - 1) / kBM;
  // Tile width by estimated time: rounds of tiles over the SMs times the measured cost of a
  // K-block of that width (~850 cycles for 128 x 256, ~550 for 128 x 128). Wide tiles win
  // as soon as they do not need more rounds than narrow ones would save.
  const int64_t tiles256 = tiles_m_bound * ((a.n + 255) / 256);
  const int64_t tiles128 = tiles_m_bound * ((a.n + 127) / 128);
  // (with one scale per row and column nothing is promoted per K-block: the MMAs run back to
  // back, ~512 / ~300 cycles per K-block, and the wide tile wins whenever it needs no more rounds)
  const int64_t cost256 = ((tiles256 + sms - 1) / sms) * (a.mode == 0 ? 850 : 512);
  const int64_t cost128 = ((tiles128 + sms - 1) / sms) * (a.mode == 0 ? 550 : 300);
  const int bn = (a.force_bn == 128 || a.force_bn == 256) ? a.force_bn : (cost256 <= cost128 ? 256 : 128);

  CUtensorMap tm_a, tm_b;
  // 16-bit operands (mode 3) are described to TMA as bytes: a row of A is 2K bytes, of B 2N
  const int64_t k_bytes = a.mode == 3 ? 2 * a.k : a.k;
  if (a.mode == 3) {
    const uint64_t dims[2] = {static_cast<uint64_t>(k_bytes), static_cast<uint64_t>(a.m)};
    const uint64_t str[1] = {static_cast<uint64_t>(k_bytes)};
    const uint32_t box[2] = {static_cast<uint32_t>(kBK), static_cast<uint32_t>(kBM)};
    if (!encode_u8(&tm_a, a.a, 2, dims, str, box))
      KSB_FAIL(KS_ERROR_INTERNAL, std::string(a.where) + ": tensor map for A rejected");
    const uint64_t bdims[3] = {static_cast<uint64_t>(2 * a.n), static_cast<uint64_t>(a.k), static_cast<uint64_t>(experts)};
    const uint64_t bstr[2] = {static_cast<uint64_t>(2 * a.n), static_cast<uint64_t>(2 * a.n) * static_cast<uint64_t>(a.k)};
    const uint32_t bbox[3] = {128u, 64u, 1u};
    if (!encode_u8(&tm_b, a.b, 3, bdims, bstr, bbox))
      KSB_FAIL(KS_ERROR_INTERNAL, std::string(a.where) + ": tensor map for B rejected");
  } else {
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.m)};
    const uint64_t str[1] = {static_cast<uint64_t>(a.k)};
    const uint32_t box[2] = {static_cast<uint32_t>(kBK), static_cast<uint32_t>(kBM)};
    if (!encode_u8(&tm_a, a.a, 2, dims, str, box))
      KSB_FAIL(KS_ERROR_INTERNAL, std::string(a.where) + ": tensor map for A rejected");
  }
  if (a.nt) {
    const uint64_t dims[3] = {static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.n), static_cast<uint64_t>(experts)};
    const uint64_t str[2] = {static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.k) * static_cast<uint64_t>(a.n)};
    const uint32_t box[3] = {static_cast<uint32_t>(kBK), static_cast<uint32_t>(bn), 1u};
    if (!encode_u8(&tm_b, a.b, 3, dims, str, box))
      KSB_FAIL(KS_ERROR_INTERNAL, std::string(a.where) + ": tensor map for B rejected");
  } else {
    const uint64_t dims[3] = {static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.k), static_cast<uint64_t>(experts)};
    const uint64_t str[2] = {static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.k) * static_cast<uint64_t>(a.n)};
    const uint32_t box[3] = {128u, static_cast<uint32_t>(kBK), 1u};
    if (!encode_u8(&tm_b, a.b, 3, dims, str, box))
      KSB_FAIL(KS_ERROR_INTERNAL, std::string(a.where) + ": tensor map for B rejected");
  }
  }

  Params p;
  p.out = a.out;
  p.a_scale = a.a_scale;
  p.b_scale = a.b_scale;
  p.offsets = a.offsets;
  p.as_row_stride = a.a_scale_ld > 0 ? 1 : (a.k + kBK - 1) / kBK;
  p.as_kb_stride = a.a_scale_ld > 0 ? a.a_scale_ld : 1;
  p.masked_m = a.masked_m;
  p.max_m = static_cast<int>(a.max_m);
  p.bias = a.bias;
  p.a_per_row = a.a_per_row ? 1 : 0;
  p.b_per_col = a.b_per_col ? 1 : 0;
  p.fault_word = kernel_fault_word();
  p.num_experts = experts;
  p.m = static_cast<int>(a.m);
  p.n = static_cast<int>(a.n);
  p.k = static_cast<int>(a.k);
  p.nkb = static_cast<int>((k_bytes + kBK - 1) / kBK);
  p.nnb = static_cast<int>((a.n + 127) / 128);
  p.tiles_n = static_cast<int>((a.n + bn - 1) / bn);
  p.tiles_m = static_cast<int>((a.m + kBM - 1) / kBM);
  // operand formats: e4m3 / e5m2 for the fp8 kinds; signed 8-bit integers with an int32
  // accumulator for kind::i8
  // (kind::f16: 0 = f16, 1 = bf16)
  const uint32_t fmt = a.mode == 2 ? 1u : (a.mode == 3 ? (a.out_dtype == KS_DTYPE_BF16 ? 1u : 0u) : (a.e5m2 ? 1u : 0u));
  p.idesc = umma_instr_desc(fmt, fmt, 0u, a.nt ? 0u : 1u, kBM, static_cast<uint32_t>(bn), a.mode == 2 ? 2u : 1u);
  const size_t out_elt = a.out_dtype == KS_DTYPE_F32 ? 4 : 2;
  bool out_aligned = a.num_out_parts > 0 ? true : aligned16(a.out);
  for (int i = 0; i < a.num_out_parts; ++i) out_aligned = out_aligned && aligned16(a.out_parts[i]);
  p.vec_store = (out_aligned && (static_cast<size_t>(a.n) * out_elt) % 16 == 0) ? 1 : 0;

  int64_t tiles = tiles_m_bound * p.tiles_n;
  const int grid = static_cast<int>(tiles < sms ? (tiles < 1 ? 1 : tiles) : sms);

  // K-split of the last partial round (dense problems only). Worth it when the tiles left
  // over after the full rounds occupy at most half of the CTAs and every part keeps at least
  // four K-blocks; the part count is capped at eight (each part costs the finishing warp one
  // more partial to read).
  p.split_from = static_cast<int>(tiles);
  p.split_items = 0;
  p.split_s = 1;
  p.split_slots = nullptr;
  if (!grouped && a.mode == 0 && a.force_split != 0 && a.num_out_parts == 0 && tiles > grid) {
    const int rem = static_cast<int>(tiles % grid);
    int s = rem > 0 ? grid / rem : 1;
    if (s > 8) s = 8;
    while (s > 1 && p.nkb / s < 4) --s;
    if (rem > 0 && s >= 2) {
      const size_t slot_bytes = static_cast<size_t>(rem) * s * kBM * bn * sizeof(float);
      float4* slots = static_cast<float4*>(stream_scratch(stream, slot_bytes, 2));
      if (slots != nullptr) {
        p.split_from = static_cast<int>(tiles) - rem;
        p.split_items = rem * s;
        p.split_s = s;
        p.split_slots = slots;
      }
    }
  }
  return bn == 256 ? launch_bn<256>(a, tm_a, tm_b, p, grid, stream) : launch_bn<128>(a, tm_a, tm_b, p, grid, stream);
}

}  // namespace sm100
}  // namespace ksb
