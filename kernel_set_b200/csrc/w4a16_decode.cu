// int4 weight-only GEMM, decode regime (at most 64 activation rows): the packed
// weight is streamed once from HBM and never leaves the register file between
// unpacking and the tensor core.
//
// Computes what ks_gemm_w4a16 declares (reference: kernels/src/gemm/
// gemm_w4a16.cu:50-130, layout :6-19): C[M,N] = A[M,K] . W + bias with
// W[k,n] = (q[k,n] - zero[g,n]) * scale[g,n] rounded once to the activation
// type (the reference's torch statement, benchmarks/bench.py:1275-1284), then
// multiplied with fp32 accumulation.
//
// Why not tcgen05 here: with M tokens the path does 4*M flop per weight byte, so
// the tensor core idles; what bounds the kernel is how many instructions and
// hand-offs lie between a packed byte arriving and its product being issued.
// Feeding tcgen05.mma needs the dequantised operand in shared memory (2 x 32 KB
// of shared-memory traffic per 8 KB of packed weight) or in tensor memory
// (tcgen05.st, 220-300 B/clk per SM when measured alone, plus two more barrier
// hops per unit). A register-operand mma.sync takes the dequantised pairs where
// they are made.
//
// Two CTAs per SM of 8 warps each, no producer warp and no spin-wait anywhere:
//   * all threads copy unit u+S-1 with cp.async (16 B each, rows of 256 contiguous
//     bytes of the packed matrix = 256 weight columns x 64 byte-rows = 128 k;
//     plus the unit's activation slice and its scale / zero-point rows) into a
//     ring of S stages, xor-swizzled on the way in; one __syncthreads per unit;
//   * warp w owns weight columns 32w..32w+31 of the tile. ldmatrix.x4.trans hands
//     lane (g = lane/4, s = lane%4) a register with the bytes
//     (row 2s, n 2g) (row 2s, n 2g+1) (row 2s+1, n 2g) (row 2s+1, n 2g+1):
//     four masks/shifts give the four A-fragment registers of one m16n8k16
//     (A = W^T: 16 columns x 16 k), each two codes of ONE column, OR-ed with the
//     exponent of 128 (bf16) / 1024 (f16); one packed subtract of (magic + zero)
//     and one packed multiply by the scale finish them, bit-identical to the
//     torch statement for integer zero-points (others take an fp32 path);
//   * the k order inside a 16-k block is permuted (slot pairs hold k = 4s, 4s+2
//     and 4s+1, 4s+3); the thread that copied an activation chunk puts it into that
//     order in shared memory once, so that the consumers' 8-byte loads are the B
//     fragments as they are;
//   * tokens are the n8 dimension of the MMA: 8 tokens per instruction, MG
//     instructions for up to 8*MG tokens.
// Work is cut stream-K style: (column tile, K-step) units are dealt to the CTAs
// in equal contiguous runs. A tile shared by several CTAs is finished per WARP:
// every warp writes its fp32 partial (32 columns) to its slot and, once its CTA's
// run is over and no copy is in flight, bumps the counter of (tile, warp); the warp
// that completes the count adds the slots in slot order (run-to-run reproducible)
// and writes C. No CTA ever waits for another.
//
// Roofline: HBM-bound; algorithmic bytes per launch
// K*N/2 + (K/gs)*N*2*(1 or 2) + M*K*2 + M*N*2.
#include <mutex>
#include <type_traits>

#include <cstdlib>

#include "common.cuh"
#include "sm100_host.cuh"
#include "sm100_ptx.cuh"
#include "sm100_w4a16.cuh"

namespace ksb {
namespace sm100 {
namespace decode {
namespace {

constexpr int kTileN = 256;             // weight columns per tile
constexpr int kStepK = 128;             // k per unit
constexpr int kRows = kStepK / 2;       // packed byte-rows per unit
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kWBytes = kRows * kTileN; // 16 KB of packed weight per unit

template <int MG>
struct Cfg {
  static constexpr int kTokens = 8 * MG;
  static constexpr int kXBytes = kTokens * kStepK * 2;   // activation slice of the unit
  static constexpr int kSZBytes = 2 * kTileN * 2;        // one row of scales, one of zero-points
  static constexpr int kStageBytes = kWBytes + kXBytes + kSZBytes;
  // Two CTAs per SM (16 warps) up to 32 tokens: a warp spends about half of its time
  // between dependent instructions, and the __syncthreads of one CTA overlaps the other's
  // work. Their rings together keep 100+ KB of copies in flight per SM.
  static constexpr int kCtasPerSm = MG <= 4 ? 2 : 1;
  static constexpr int kStages = MG <= 2 ? 5 : (MG == 4 ? 4 : 6);   // at least 4: units it+2 .. it+S-1 are in flight
  static constexpr int kSmemBytes = kStages * kStageBytes + 128;
  static constexpr int kAccRegs = MG * 2 * 4;            // per lane: token groups x column chunks x 4
  static_assert(kSmemBytes * kCtasPerSm + 1024 * kCtasPerSm <= 233472, "stage rings exceed the shared memory of an SM");
};

struct Params {
  void* c;
  const void* a;
  const uint8_t* w;
  const void* scales;
  const void* zeros;
  const void* bias;
  float* slots;             // [tiles][max_parts][warp][acc register][lane] fp32 partials
  unsigned int* counters;   // [tiles][warp]
  int m, n, k;
  int n_tiles, k_steps;
  int gs_steps;             // K-steps per scale group (group_size / 128)
  int max_parts;
  int has_zeros;
};

template <typename T> struct Pack16;
template <> struct Pack16<__nv_bfloat16> {
  using V2 = __nv_bfloat162;
  static constexpr uint32_t kMagic2 = 0x43004300u;      // bf16(128) twice: 128 + q once the code is OR-ed in
  static constexpr float kMagic = 128.0f;
  static constexpr uint32_t kMaxZeroBits = 0x42FEu;     // bf16(127)
  __device__ static V2 from_bits(uint32_t b) { return *reinterpret_cast<V2*>(&b); }
  __device__ static uint32_t bits(V2 v) { return *reinterpret_cast<uint32_t*>(&v); }
  __device__ static V2 splat(float f) { return __float2bfloat162_rn(f); }
  __device__ static float to_float(uint32_t b16) { return __uint_as_float(b16 << 16); }
  __device__ static uint32_t make(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ static void mma(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
};
template <> struct Pack16<__half> {
  using V2 = __half2;
  static constexpr uint32_t kMagic2 = 0x64006400u;      // f16(1024) twice
  static constexpr float kMagic = 1024.0f;
  static constexpr uint32_t kMaxZeroBits = 0x63FEu;     // f16(1023)
  __device__ static V2 from_bits(uint32_t b) { return *reinterpret_cast<V2*>(&b); }
  __device__ static uint32_t bits(V2 v) { return *reinterpret_cast<uint32_t*>(&v); }
  __device__ static V2 splat(float f) { return __float2half2_rn(f); }
  __device__ static float to_float(uint32_t b16) { return __half2float(__ushort_as_half(static_cast<unsigned short>(b16))); }
  __device__ static uint32_t make(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ static void mma(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// 16-byte asynchronous copy global -> shared, bypassing L1; src_bytes = 0 writes zeros.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// Four 8x8 matrices of 16-bit elements, transposed on the way: lane l supplies the
// address of row l%8 of matrix l/8; lane (g, s) receives elements (rows 2s and 2s+1,
// column g) of each matrix, the lower row in the low half.
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr)
               : "memory");
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

// 16-byte chunk `cc` (0..15) of byte-row `row` of the packed tile lives at this chunk of
// the row in shared memory: eight consecutive rows of one chunk column fall into eight
// different bank groups (what ldmatrix reads in one go).
__device__ __forceinline__ uint32_t w_chunk(uint32_t cc, uint32_t row) { return (cc & 8u) | ((cc & 7u) ^ (row & 7u)); }
// Chunk of a token row of the activation slice: four consecutive tokens' 32-byte pieces
// of one 16-k block fall into four different bank quarters (one 8-byte load per lane).
__device__ __forceinline__ uint32_t x_chunk(uint32_t cc, uint32_t tok) { return cc ^ ((tok & 3u) << 1); }

// (a & b) | c in one instruction.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename T, int MG>
__global__ void __launch_bounds__(kThreads, Cfg<MG>::kCtasPerSm) w4a16_decode_kernel(const Params p) {
  using C = Cfg<MG>;
  using P16 = Pack16<T>;
  using V2 = typename P16::V2;
  constexpr int S = C::kStages;
  constexpr int kXChunks = (C::kTokens + 15) / 16;   // activation chunks a thread stages per unit
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_addr(smem_raw) + 127u) & ~127u;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, s = lane & 3;
  // the next kernel on the stream may start its own prologue as soon as it finds room
  grid_launch_dependents();

  const long long units = static_cast<long long>(p.n_tiles) * p.k_steps;
  const int ctas = gridDim.x;
  const long long u_begin = run_start(units, ctas, blockIdx.x);
  const long long u_end = run_start(units, ctas, blockIdx.x + 1);
  const int n_units = static_cast<int>(u_end - u_begin);
  const int tile0 = static_cast<int>(u_begin / p.k_steps);
  const int step0 = static_cast<int>(u_begin - static_cast<long long>(tile0) * p.k_steps);

  // ------------------------------ loader state ------------------------------
  // Every thread copies the same chunks of every unit: 16-byte chunk cc of byte-rows
  // r0, r0 + 16, r0 + 32, r0 + 48 of the packed tile, chunk cc of token rows r0, r0 + 16, ...
  // of the activation slice, and (warps 0 and 1) chunk `lane` of the scale / zero-point row.
  // Source pointers advance by a constant per K-step and are rebuilt when the tile changes.
  int tile_l = tile0, step_l = step0;
  int grp_l = step_l / p.gs_steps, in_grp_l = step_l - grp_l * p.gs_steps;
  int loaded = 0;
  uint32_t st_load = ring;                       // stage the next copy goes to
  const uint32_t ld_r0 = tid >> 4, ld_cc = tid & 15u;
  const uint32_t w_dst = ld_r0 * kTileN + (w_chunk(ld_cc, ld_r0) << 4);
  const uint32_t x_dst = kWBytes + ld_r0 * (kStepK * 2) + (x_chunk(ld_cc, ld_r0) << 4);
  const size_t w_row16 = static_cast<size_t>(16) * p.n;            // 16 byte-rows further down
  const size_t w_step = static_cast<size_t>(kRows) * p.n;          // one K-step further down
  const size_t x_row16 = static_cast<size_t>(16) * p.k * 2;        // 16 tokens further down
  const uint8_t* const a_bytes = static_cast<const uint8_t*>(p.a);
  const uint8_t* const sz_base = static_cast<const uint8_t*>(warp == 0 ? p.scales : p.zeros);
  const bool sz_active = warp == 0 || (warp == 1 && p.has_zeros);
  const uint32_t sz_dst = kWBytes + C::kXBytes + (warp == 1 ? kTileN * 2 : 0) + (lane << 4);
  // tokens this thread stages: ld_r0 + 16 i; rows at or beyond M are written as zeros
  uint32_t x_bytes[kXChunks];
#pragma unroll
  for (int i = 0; i < kXChunks; ++i) x_bytes[i] = static_cast<int>(ld_r0) + 16 * i < p.m ? 16u : 0u;
  const uint8_t* w_src;
  const uint8_t* x_src = a_bytes + (static_cast<size_t>(ld_r0) * p.k + ld_cc * 8) * 2 + static_cast<size_t>(step_l) * (kStepK * 2);
  const uint8_t* sz_src;
  uint32_t w_bytes, sz_bytes;
  auto enter_tile = [&](int tile, int step, int grp) {
    const int col0 = tile * kTileN;
    const bool w_ok = col0 + static_cast<int>(ld_cc) * 16 < p.n;
    w_bytes = w_ok ? 16u : 0u;
    w_src = w_ok ? p.w + (static_cast<size_t>(step) * kRows + ld_r0) * p.n + col0 + ld_cc * 16 : p.w;
    const bool s_ok = sz_active && col0 + lane * 8 < p.n;
    sz_bytes = s_ok ? 16u : 0u;
    sz_src = s_ok ? sz_base + (static_cast<size_t>(grp) * p.n + col0 + lane * 8) * 2 : a_bytes;
  };
  enter_tile(tile_l, step_l, grp_l);
  // The activations may be the output of the kernel that runs before this one on the stream;
  // the weights are not. A launch with programmatic stream serialization starts while that
  // kernel is still running, so the prologue copies weights, scales and zero-points only and
  // hands in the activations of the same units after the grid dependency has resolved.
  auto issue_x = [&](uint32_t stage, const uint8_t* src) {
#pragma unroll
    for (int i = 0; i < kXChunks; ++i) {
      if (16 * i + 15 < C::kTokens || static_cast<int>(ld_r0) + 16 * i < C::kTokens)
        cp_async16(stage + x_dst + i * (16 * kStepK * 2), x_bytes[i] ? src + i * x_row16 : a_bytes, x_bytes[i]);
    }
  };
  const uint8_t* late_x_src[S - 1];
  auto issue = [&](auto with_x_tag, int slot) {
    constexpr bool kWithX = decltype(with_x_tag)::value;
    if (loaded < n_units) {
      // a chunk outside the matrix keeps the (valid) base pointer and copies zero bytes
      const size_t wr = w_bytes ? w_row16 : 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) cp_async16(st_load + w_dst + i * (16 * kTileN), w_src + i * wr, w_bytes);
      if constexpr (kWithX) issue_x(st_load, x_src); else late_x_src[slot] = x_src;
      if (sz_active) cp_async16(st_load + sz_dst, sz_src, sz_bytes);
      ++loaded;
      st_load = (st_load == ring + (S - 1) * C::kStageBytes) ? ring : st_load + C::kStageBytes;
      if (++step_l == p.k_steps) {
        step_l = 0; grp_l = 0; in_grp_l = 0; ++tile_l;
        x_src -= static_cast<size_t>(p.k_steps - 1) * (kStepK * 2);
        enter_tile(tile_l, 0, 0);
      } else {
        x_src += kStepK * 2;
        if (w_bytes) w_src += w_step;
        if (++in_grp_l == p.gs_steps) {
          in_grp_l = 0; ++grp_l;
          if (sz_bytes) sz_src += static_cast<size_t>(p.n) * 2;
        }
      }
    }
    cp_async_commit();
  };
  // The k order inside a 16-k block that the weight fragments imply (slot pairs hold
  // k = 4s, 4s+2 and 4s+1, 4s+3) is given to the activations once, by the thread that
  // copied the chunk, in place: [x0 x1 x2 x3] -> [x0 x2 x1 x3] for both 4-k groups of the
  // chunk. The consumers' 8-byte loads then are the two B-fragment registers as they are.
  auto permute_x = [&](uint32_t st) {
#pragma unroll
    for (int i = 0; i < kXChunks; ++i) {
      if (16 * i + 15 < C::kTokens || static_cast<int>(ld_r0) + 16 * i < C::kTokens) {
        const uint32_t addr = st + x_dst + i * (16 * kStepK * 2);
        const uint4 v = lds128(addr);
        sts128(addr, make_uint4(__byte_perm(v.x, v.y, 0x5410), __byte_perm(v.x, v.y, 0x7632),
                                __byte_perm(v.z, v.w, 0x5410), __byte_perm(v.z, v.w, 0x7632)));
      }
    }
  };

  // ------------------------------ compute state ------------------------------
  float acc[MG][2][4];
#pragma unroll
  for (int t = 0; t < MG; ++t)
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[t][c][j] = 0.f;

  int tile = tile0, step = step0;
  int seg_first_step = step;
  // partial segments of this run (at most two: the head of the run and its tail), published
  // after the main loop
  int pub_tile[2] = {-1, -1};
  int n_pub = 0;

  // lane's row address inside a stage for ldmatrix: matrix mi = lane / 8 covers K-block
  // (mi / 2) of the pair and column chunk (mi % 2) of this warp; row = lane % 8
  const uint32_t ld_mi = lane >> 3, ld_i = lane & 7u;
  const uint32_t ld_off = (8u * (ld_mi >> 1) + ld_i) * kTileN + (w_chunk(2u * warp + (ld_mi & 1u), ld_i) << 4);
  // lane's 8 bytes of an activation row: token 8*tg + g, k-slots of lane s in K-block kb sit in
  // chunk (2 kb + s/2) ^ ((g % 4) * 2) = 2 (kb ^ (g % 4)) + s/2; kb ^ (g % 4) = (kb & 4) | ((kb & 3) ^ (g % 4))
  const uint32_t x_row_off = kWBytes + static_cast<uint32_t>(g) * (kStepK * 2) + 8u * (s & 1u) + 16u * (s >> 1);
  uint32_t x_kb_off[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) x_kb_off[q] = x_row_off + 32u * (static_cast<uint32_t>(q) ^ (static_cast<uint32_t>(g) & 3u));
  const uint32_t sz_off = kWBytes + C::kXBytes + (32u * warp + 2u * g) * 2u;
  const V2 magic2 = P16::splat(P16::kMagic);
  const uint32_t kMask = 0x000F000Fu, kMagicBits = P16::kMagic2;
  T* cmat = static_cast<T*>(p.c);
  const T* bias = static_cast<const T*>(p.bias);
  constexpr int kSlotFloats = C::kAccRegs * 32;
  const size_t part_stride = static_cast<size_t>(kWarps) * kSlotFloats;

  auto store_c = [&](float (&v)[MG][2][4], int tile_of) {
    const int n_base = tile_of * kTileN + 32 * warp + 2 * g;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int n = n_base + 16 * c;
      if (n < p.n) {   // N is a multiple of 16 and n is even: n + 1 is inside too
        const float b0 = bias != nullptr ? to_f32<T>(bias[n]) : 0.f;
        const float b1 = bias != nullptr ? to_f32<T>(bias[n + 1]) : 0.f;
#pragma unroll
        for (int t = 0; t < MG; ++t) {
          const int tok = 8 * t + 2 * s;
          // d0 (n, tok) d1 (n, tok+1) d2 (n+1, tok) d3 (n+1, tok+1)
          if (tok < p.m)
            *reinterpret_cast<uint32_t*>(cmat + static_cast<size_t>(tok) * p.n + n) =
                P16::make(v[t][c][0] + b0, v[t][c][2] + b1);
          if (tok + 1 < p.m)
            *reinterpret_cast<uint32_t*>(cmat + static_cast<size_t>(tok + 1) * p.n + n) =
                P16::make(v[t][c][1] + b0, v[t][c][3] + b1);
        }
      }
    }
  };

  // prologue: S-1 units on their way; the first one's activations in consumer order
#pragma unroll
  for (int i = 0; i < S - 1; ++i) issue(std::false_type{}, i);
  grid_dependency_wait();   // everything the previous kernel wrote is visible from here on
#pragma unroll
  for (int i = 0; i < S - 1; ++i) {
    if (i < n_units) issue_x(ring + i * C::kStageBytes, late_x_src[i]);
    cp_async_commit();
  }
  // groups so far: S-1 of weights, then S-1 of activations; the first S of them cover unit 0
  cp_async_wait<S - 2>();
  permute_x(ring);
  uint32_t st = ring;            // stage of the unit being computed
  uint32_t st_next = n_units > 1 ? ring + C::kStageBytes : ring;

#pragma unroll 1
  for (int it = 0; it < n_units; ++it) {
    cp_async_wait<S - 3>();   // this thread's copies of units it and it+1 have landed ...
    __syncthreads();          // ... everyone's of unit it (and its permuted activations) too;
                              // and everyone has finished reading unit it-1
    issue(std::true_type{}, 0);   // refill the stage unit it-1 occupied
    if (it + 1 < n_units) permute_x(st_next);   // own chunks only: no other thread touches them before the next barrier

    // scales and zero-points of this lane's columns: chunk c, columns 2g and 2g+1
    V2 sc[2][2], zz[2][2];
    uint32_t sraw[2], zraw[2];
    uint32_t bad = 0u;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      sraw[c] = lds32(st + sz_off + 32u * c);
      zraw[c] = p.has_zeros ? lds32(st + sz_off + 32u * c + kTileN * 2) : 0u;
      sc[c][0] = P16::from_bits(__byte_perm(sraw[c], sraw[c], 0x1010));
      sc[c][1] = P16::from_bits(__byte_perm(sraw[c], sraw[c], 0x3232));
      // (magic + zero) must be exact; then (magic + q) - (magic + zero) is exact too: true for
      // every non-negative integer zero-point that survives the round trip
      const V2 zp = __hadd2(P16::from_bits(zraw[c]), magic2);
      bad |= (P16::bits(__hsub2(zp, magic2)) ^ zraw[c]) | (zraw[c] & 0x80008000u);
      const uint32_t zb = P16::bits(zp);
      zz[c][0] = P16::from_bits(__byte_perm(zb, zb, 0x1010));
      zz[c][1] = P16::from_bits(__byte_perm(zb, zb, 0x3232));
    }
    const bool simple = !__any_sync(0xFFFFFFFFu, bad != 0u);

    auto pair_body = [&](int pr, auto fast_tag) {
      constexpr bool kFast = decltype(fast_tag)::value;
      uint32_t r[4];
      ldmatrix_x4_trans(r, st + ld_off + pr * (16 * kTileN));
#pragma unroll
      for (int kbi = 0; kbi < 2; ++kbi) {
        const int kb = 2 * pr + kbi;
        uint32_t b[MG][2];
#pragma unroll
        for (int t = 0; t < MG; ++t) {
          uint32_t xo;
          if constexpr (kFast) xo = x_kb_off[kb & 3] + (kb >> 2) * 128;   // kb is a compile-time constant here
          else xo = x_row_off + 32u * (static_cast<uint32_t>(kb) ^ (static_cast<uint32_t>(g) & 3u));
          const uint2 x = lds64(st + xo + t * (8 * kStepK * 2));
          b[t][0] = x.x;   // k = 4s, 4s+2
          b[t][1] = x.y;   // k = 4s+1, 4s+3
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const uint32_t w = r[kbi * 2 + c];
          // bytes of w: (row 2s, n 2g) (row 2s, n 2g+1) (row 2s+1, n 2g) (row 2s+1, n 2g+1);
          // low nibble = even k of the row, high nibble = odd k
          const uint32_t ws[4] = {w, w >> 8, w >> 4, w >> 12};
          uint32_t a[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if constexpr (kFast) {
              a[j] = P16::bits(__hmul2(__hsub2(P16::from_bits(and_or(ws[j], kMask, kMagicBits)), zz[c][j & 1]), sc[c][j & 1]));
            } else {
              // zero-points that are not small integers: the fp32 statement, verbatim
              const uint32_t q = ws[j] & kMask;
              const uint32_t sh = (j & 1) ? 16u : 0u;
              const float zf = P16::to_float((zraw[c] >> sh) & 0xFFFFu), sf = P16::to_float((sraw[c] >> sh) & 0xFFFFu);
              a[j] = P16::make(__fmul_rn(__fsub_rn(static_cast<float>(q & 15u), zf), sf),
                               __fmul_rn(__fsub_rn(static_cast<float>(q >> 16), zf), sf));
            }
          }
#pragma unroll
          for (int t = 0; t < MG; ++t) P16::mma(acc[t][c], a, b[t]);
        }
      }
    };
    if (simple) {
#pragma unroll
      for (int pr = 0; pr < 4; ++pr) pair_body(pr, std::true_type{});
    } else {
#pragma unroll 1
      for (int pr = 0; pr < 4; ++pr) pair_body(pr, std::false_type{});
    }

    const bool seg_last = (step == p.k_steps - 1) || (it == n_units - 1);
    if (seg_last) {
      const bool whole = (seg_first_step == 0) && (step == p.k_steps - 1);
      if (whole) {
        store_c(acc, tile);
      } else {
        // this CTA's share of the tile goes to its slot; the arrival is announced after the
        // main loop, when no copy is in flight any more (a fence here would wait for all of them)
        const int first_cta = cta_of_unit(units, ctas, static_cast<long long>(tile) * p.k_steps);
        const int part = static_cast<int>(blockIdx.x) - first_cta;
        float* mine = p.slots + ((static_cast<size_t>(tile) * p.max_parts + part) * kWarps + warp) * kSlotFloats + lane;
#pragma unroll
        for (int t = 0; t < MG; ++t)
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int j = 0; j < 4; ++j) __stcg(mine + ((t * 2 + c) * 4 + j) * 32, acc[t][c][j]);
        if (n_pub == 0) pub_tile[0] = tile; else pub_tile[1] = tile;
        ++n_pub;
      }
#pragma unroll
      for (int t = 0; t < MG; ++t)
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[t][c][j] = 0.f;
      seg_first_step = (step == p.k_steps - 1) ? 0 : step + 1;
    }
    if (++step == p.k_steps) { step = 0; ++tile; }
    st = st_next;
    st_next = (st_next == ring + (S - 1) * C::kStageBytes) ? ring : st_next + C::kStageBytes;
  }
  cp_async_wait<0>();

  // ------------------------------ split tiles ------------------------------
  // Announce this warp's partials; the warp that completes a (tile, warp) count adds the
  // parts in part order and writes C.
  if (n_pub > 0) {
    __threadfence();
    __syncwarp();
    // both arrivals go out before either answer is needed (an atomic's round trip is ~1 us)
    int tls[2], parts_of[2];
    unsigned int prevs[2] = {0u, 0u};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tls[r] = r == 0 ? pub_tile[0] : pub_tile[1];
      parts_of[r] = 0;
      if (r < n_pub) {
        const long long tile_u0 = static_cast<long long>(tls[r]) * p.k_steps;
        const int first_cta = cta_of_unit(units, ctas, tile_u0);
        parts_of[r] = cta_of_unit(units, ctas, tile_u0 + p.k_steps - 1) - first_cta + 1;
        if (lane == 0) prevs[r] = atomicAdd(p.counters + tls[r] * kWarps + warp, 1u);
      }
    }
#pragma unroll 1
    for (int r = 0; r < n_pub; ++r) {
      const int tl = r == 0 ? tls[0] : tls[1];
      const int parts = r == 0 ? parts_of[0] : parts_of[1];
      const unsigned int prev = __shfl_sync(0xFFFFFFFFu, r == 0 ? prevs[0] : prevs[1], 0);
      if (prev != static_cast<unsigned int>(parts - 1)) continue;
      if (lane == 0) p.counters[tl * kWarps + warp] = 0u;   // ready for the next launch
      __threadfence();
      const float* tile_slots = p.slots + (static_cast<size_t>(tl) * p.max_parts * kWarps + warp) * kSlotFloats + lane;
#pragma unroll
      for (int t = 0; t < MG; ++t)
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[t][c][j] = 0.f;
      // parts are added in part order; the loads of kAhead parts are in flight together
      constexpr int kAhead = MG == 1 ? 4 : (MG == 2 ? 2 : 1);
      for (int qd = 0; qd < parts; qd += kAhead) {
        float v[kAhead][MG][2][4];
#pragma unroll
        for (int h = 0; h < kAhead; ++h) {
          const float* src = tile_slots + (qd + h) * part_stride;
#pragma unroll
          for (int t = 0; t < MG; ++t)
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int j = 0; j < 4; ++j)
                v[h][t][c][j] = qd + h < parts ? __ldcg(src + ((t * 2 + c) * 4 + j) * 32) : 0.f;
        }
#pragma unroll
        for (int h = 0; h < kAhead; ++h)
#pragma unroll
          for (int t = 0; t < MG; ++t)
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int j = 0; j < 4; ++j) acc[t][c][j] += v[h][t][c][j];
      }
      store_c(acc, tl);
    }
  }
}

template <typename T, int MG>
ks_status_t launch_t(const Params& p, int grid, cudaStream_t stream) {
  using C = Cfg<MG>;
  auto kernel = w4a16_decode_kernel<T, MG>;
  static std::mutex mu;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
      if (e != cudaSuccess) return cuda_status(e, "ks_gemm_w4a16");
      // all of the SM's unified storage as shared memory, or the second CTA does not fit
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      if (e != cudaSuccess) return cuda_status(e, "ks_gemm_w4a16");
      attr_done[dev] = true;
    }
  }
  return cuda_status(launch_programmatic(kernel, static_cast<unsigned>(grid), kThreads, C::kSmemBytes, stream, p),
                     "ks_gemm_w4a16");
}

template <typename T>
ks_status_t launch_mg(int mg, const Params& p, int grid, cudaStream_t stream) {
  switch (mg) {
    case 1: return launch_t<T, 1>(p, grid, stream);
    case 2: return launch_t<T, 2>(p, grid, stream);
    case 4: return launch_t<T, 4>(p, grid, stream);
    default: return launch_t<T, 8>(p, grid, stream);
  }
}

}  // namespace

bool eligible(const W4A16Args& a) {
  if (a.m > kMaxTokens) return false;
  if (a.k % kStepK != 0) return false;
  if (a.group_size % kStepK != 0) return false;   // one scale row per 128-k step
  if (a.n % 16 != 0) return false;                // 16-byte chunks of the packed rows and of the scale rows
  if (!aligned16(a.a) || !aligned16(a.b_packed) || !aligned16(a.scales)) return false;
  if (a.zeros != nullptr && !aligned16(a.zeros)) return false;
  if ((reinterpret_cast<uintptr_t>(a.c) & 3u) != 0) return false;   // pairs of outputs are stored as one word
  const long long tiles = (a.n + kTileN - 1) / kTileN;
  if (tiles * (a.k / kStepK) > (1ll << 30)) return false;
  return true;
}

Geometry geometry_of(const W4A16Args& a) {
  Geometry g;
  g.mg = a.m <= 8 ? 1 : (a.m <= 16 ? 2 : (a.m <= 32 ? 4 : 8));
  g.n_tiles = static_cast<int>((a.n + kTileN - 1) / kTileN);
  g.k_steps = static_cast<int>(a.k / kStepK);
  const long long units = static_cast<long long>(g.n_tiles) * g.k_steps;
  const int ctas = sm_count() * (g.mg <= 4 ? 2 : 1);
  g.grid = static_cast<int>(units < ctas ? units : ctas);
  const long long per_cta = units / g.grid;   // shortest run
  g.max_parts = static_cast<int>((g.k_steps + per_cta - 1) / per_cta) + 1;
  g.slot_bytes = static_cast<size_t>(g.n_tiles) * g.max_parts * kWarps * (g.mg * 8 * 32) * sizeof(float);
  g.counter_bytes = (static_cast<size_t>(g.n_tiles) * kWarps * sizeof(unsigned int) + 255) & ~size_t(255);
  return g;
}

ks_status_t enqueue(const W4A16Args& a, const Geometry& g, unsigned int* counters, float* slots,
                    cudaStream_t stream) {
  Params p;
  p.c = a.c;
  p.a = a.a;
  p.w = static_cast<const uint8_t*>(a.b_packed);
  p.scales = a.scales;
  p.zeros = a.zeros;
  p.bias = a.bias;
  p.slots = slots;
  p.counters = counters;
  p.m = static_cast<int>(a.m);
  p.n = static_cast<int>(a.n);
  p.k = static_cast<int>(a.k);
  p.n_tiles = g.n_tiles;
  p.k_steps = g.k_steps;
  p.gs_steps = a.group_size / kStepK;
  p.max_parts = g.max_parts;
  p.has_zeros = a.zeros != nullptr ? 1 : 0;
  if (a.dtype == KS_DTYPE_BF16) return launch_mg<__nv_bfloat16>(g.mg, p, g.grid, stream);
  return launch_mg<__half>(g.mg, p, g.grid, stream);
}

}  // namespace decode
}  // namespace sm100
}  // namespace ksb
