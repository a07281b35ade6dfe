// Thin inline-PTX wrappers for the sm_100a features the fast kernels use:
// mbarrier with bounded waits, TMA tiled loads, TMEM allocation, tcgen05
// MMA / commit / load, and the UMMA shared-memory and instruction descriptors.
//
// Every wait in this file is bounded: after `kWaitLimitNs` a waiter raises a
// CTA-wide abort flag, records a code in a host-visible word and returns
// false; the kernels then drain and release TMEM instead of hanging.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ksb {
namespace sm100 {

constexpr unsigned long long kWaitLimitNs = 2000ull * 1000ull * 1000ull;  // 2 s per wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// True in exactly one lane of a converged warp. Code guarded by it is known to
// the compiler to run in a single thread, which lets tcgen05 / TMA operands
// travel in uniform registers instead of through a per-lane fallback loop.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .b32 rx;\n\t"
      ".reg .pred px;\n\t"
      "elect.sync rx|px, 0xFFFFFFFF;\n\t"
      "selp.u32 %0, 1, 0, px;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
// Makes barrier initialisation visible to the async (TMA / tcgen05) proxy.
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Same test, but the thread may stay suspended in hardware for up to `hint_ns`
// while the phase is incomplete (it is still resumed when the phase completes).
// For waits known to be long: a sleeping waiter leaves the issue slots of its
// scheduler to the warps that have work.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

// Shared state of a CTA's bounded waits.
struct WaitCtx {
  volatile uint32_t* abort_flag;  // shared memory, zero while healthy
  unsigned int* fault_word;       // host-mapped, may be NULL
};

// Waits for the phase with the given parity to complete. Returns false when
// another waiter of this CTA has already given up or when this one times out;
// `code` identifies the wait site in the recorded fault word.
__device__ __forceinline__ bool mbar_wait(const WaitCtx& ctx, uint32_t bar, uint32_t parity, uint32_t code);

// Bounded wait for barriers that normally take thousands of cycles to complete
// (an accumulator that needs a whole run of K-steps): polls with a suspend hint.
__device__ __forceinline__ bool mbar_wait_long(const WaitCtx& ctx, uint32_t bar, uint32_t parity, uint32_t code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
    if (*ctx.abort_flag != 0u) return false;
    if (global_ns() - t0 > kWaitLimitNs) {
      *ctx.abort_flag = 1u;
      if (ctx.fault_word != nullptr) {
        *reinterpret_cast<volatile unsigned int*>(ctx.fault_word) = 0x80000000u | code;
        __threadfence_system();
      }
      return false;
    }
  }
}

// Waits for two barriers whose phases are usually both complete already: both are
// tested before either result is used, so the two ~100-cycle round trips overlap.
__device__ __forceinline__ bool mbar_wait_both(const WaitCtx& ctx, uint32_t bar_a, uint32_t parity_a, uint32_t code_a,
                                               uint32_t bar_b, uint32_t parity_b, uint32_t code_b) {
  const bool a = mbar_try_wait(bar_a, parity_a);
  const bool b = mbar_try_wait(bar_b, parity_b);
  if (a && b) return true;
  if (!a && !mbar_wait(ctx, bar_a, parity_a, code_a)) return false;
  if (!b && !mbar_wait(ctx, bar_b, parity_b, code_b)) return false;
  return true;
}

// mbar_wait whose polls carry a suspend-time hint: the hardware parks the waiter for
// about `hint_ns` at most before the next poll. For waits on a kernel's critical path.
__device__ __forceinline__ bool mbar_wait_hinted(const WaitCtx& ctx, uint32_t bar, uint32_t parity, uint32_t code,
                                                 uint32_t hint_ns) {
#pragma unroll 1
  for (int i = 0; i < 4096; ++i)
    if (mbar_try_wait_hint(bar, parity, hint_ns)) return true;
  const unsigned long long t0 = global_ns();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait_hint(bar, parity, hint_ns)) return true;
    if (*ctx.abort_flag != 0u) return false;
    if (global_ns() - t0 > kWaitLimitNs) {
      *ctx.abort_flag = 1u;
      if (ctx.fault_word != nullptr) {
        *reinterpret_cast<volatile unsigned int*>(ctx.fault_word) = 0x80000000u | code;
        __threadfence_system();
      }
      return false;
    }
  }
}

__device__ __forceinline__ bool mbar_wait(const WaitCtx& ctx, uint32_t bar, uint32_t parity, uint32_t code) {
  // Fast path: plain polling, no timer and no shared-memory traffic besides the
  // barrier itself. Each failed try_wait may itself block for a short,
  // hardware-defined time, so this phase already covers every healthy wait.
#pragma unroll 1
  for (int i = 0; i < 4096; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  // Slow path: something upstream is late. Keep polling, but watch the clock
  // and the CTA's abort flag.
  const unsigned long long t0 = global_ns();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*ctx.abort_flag != 0u) return false;
    if (global_ns() - t0 > kWaitLimitNs) {
      *ctx.abort_flag = 1u;
      if (ctx.fault_word != nullptr) {
        *reinterpret_cast<volatile unsigned int*>(ctx.fault_word) = 0x80000000u | code;
        __threadfence_system();
      }
      return false;
    }
  }
}

// ---- programmatic dependent launch --------------------------------------------------
// A kernel launched with programmatic stream serialization may start while the kernel before
// it on the stream is still running. grid_dependency_wait() returns once that kernel has
// completed and its writes are visible: every thread that reads what it produced, or
// overwrites what it may still read, calls it first. grid_launch_dependents() tells the
// runtime that the NEXT kernel on the stream may begin to occupy free resources. Both are
// no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

// ---- TMA (tiled bulk tensor loads, one CTA, completion on an mbarrier) --------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// x is the innermost (contiguous) coordinate; x * element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// ---- TMEM ------------------------------------------------------------------------
// Whole-warp operations (.sync.aligned): call with all 32 lanes converged.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result_addr, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result_addr),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives once on `bar` when every tcgen05 operation this thread issued so
// far has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Same wait, but the loaded registers pass through the statement as in/out
// operands: code that consumes them is then data-dependent on the wait and
// cannot be scheduled ahead of it.
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                 "+r"(r[15])
               :
               : "memory");
}
// Lane i of the warp receives 16 consecutive fp32 columns of TMEM lane
// (taddr.lane + i). A warp may only address the 32-lane quarter warp_id % 4.
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Lane i of the warp writes 16 consecutive 32-bit columns of TMEM lane (taddr.lane + i).
__device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// Returns once the tcgen05.st of this thread have been performed.
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32-column variant: lane i receives columns [col, col+32) of its TMEM lane.
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                 "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                 "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                 "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

// ---- register budget per warpgroup (all four warps of the group execute it) ----
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// acc = a * b + acc on two fp32 lanes. KSB_FFMA2=1 uses the packed
// fma.rn.f32x2 instruction (operands travel as 64-bit register pairs);
// KSB_FFMA2=0 issues two scalar FMAs.
#ifndef KSB_FFMA2
#define KSB_FFMA2 1
#endif
__device__ __forceinline__ void ffma2(float2& acc, float a_lo, float a_hi, float2 b) {
#if KSB_FFMA2
  uint64_t d, a, bb;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(acc.x), "f"(acc.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a_lo), "f"(a_hi));
  asm("mov.b64 %0, {%1, %2};" : "=l"(bb) : "f"(b.x), "f"(b.y));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(bb));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(acc.x), "=f"(acc.y) : "l"(d));
#else
  acc.x = fmaf(a_lo, b.x, acc.x);
  acc.y = fmaf(a_hi, b.y, acc.y);
#endif
}

// ---- UMMA descriptors --------------------------------------------------------------
// 64-bit shared-memory matrix descriptor: start address, leading-dimension and
// stride-dimension byte offsets (all in 16-byte units), descriptor version 1
// (bits 46-47), 128-byte swizzle (layout type 2 in bits 61-63). The tile must
// start on a 1024-byte boundary; stepping along K inside a swizzle atom adds the
// byte offset to the start address.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// 32-bit instruction descriptor, dense. Formats: for kind::f8f6f4 0 = e4m3,
// 1 = e5m2; for kind::f16 0 = f16, 1 = bf16; for kind::i8 0 = unsigned, 1 = signed.
// major: 0 = K-major operand, 1 = MN-major operand. acc_fmt: 1 = fp32 accumulator
// (the floating-point kinds), 2 = int32 (kind::i8).
__host__ __device__ constexpr uint32_t umma_instr_desc(uint32_t a_fmt, uint32_t b_fmt, uint32_t a_mn_major,
                                                       uint32_t b_mn_major, uint32_t m, uint32_t n,
                                                       uint32_t acc_fmt = 1u) {
  return (acc_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread for the whole CTA.
__device__ __forceinline__ void umma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}


// ---- single-lane issue from converged code -----------------------------------------
// The *_elect wrappers below are called by all 32 lanes of a converged warp;
// elect.sync picks one lane and the instruction is predicated on it inside the
// same asm statement. Issued this way a tcgen05.mma costs ~55 cycles; issued
// from inside an `if (lane == 0)` branch it measured ~160 cycles, which made
// instruction issue, not the tensor pipe, the bound. Successive elections in a
// converged warp pick the same lane, so a commit tracks the MMAs before it.
#define KSB_ELECT_PROLOGUE ".reg .pred q;\n\t.reg .b32 rx;\n\telect.sync rx|q, 0xFFFFFFFF;\n\t"

__device__ __forceinline__ void umma_f8f6f4_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t" KSB_ELECT_PROLOGUE
               "setp.ne.b32 p, %4, 0;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
               "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}
// int8 x int8 -> int32 (signedness of each operand comes from the instruction descriptor)
__device__ __forceinline__ void umma_i8_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t" KSB_ELECT_PROLOGUE
               "setp.ne.b32 p, %4, 0;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
               "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void umma_f16_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t" KSB_ELECT_PROLOGUE
               "setp.ne.b32 p, %4, 0;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
               "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}
// Same, with the A operand in tensor memory: 128 lanes (rows of A) x K/2 columns, a
// 32-bit cell holding two consecutive 16-bit K elements (lower k in the low half).
__device__ __forceinline__ void umma_f16_tmem_a_elect(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                                      uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t" KSB_ELECT_PROLOGUE
               "setp.ne.b32 p, %4, 0;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
               "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void tc_commit_elect(uint32_t bar) {
  asm volatile("{\n\t" KSB_ELECT_PROLOGUE
               "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}\n" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_elect(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t" KSB_ELECT_PROLOGUE
               "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}\n" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_elect(uint32_t bar) {
  asm volatile("{\n\t" KSB_ELECT_PROLOGUE "@q mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}\n" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma_load_2d_elect(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x,
                                                  int y) {
  asm volatile("{\n\t" KSB_ELECT_PROLOGUE
               "@q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
               "[%2];\n\t}\n" ::"r"(smem_dst),
               "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_load_3d_elect(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y,
                                                  int z) {
  asm volatile("{\n\t" KSB_ELECT_PROLOGUE
               "@q cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
               "%5}], [%2];\n\t}\n" ::"r"(smem_dst),
               "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
               : "memory");
}

// ---- TMA stores (shared -> global), tracked in per-thread bulk groups ---------------------
// x (innermost coordinate) times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once the bulk groups of this thread have finished READING shared memory.
__device__ __forceinline__ void bulk_wait_group_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Returns once the bulk groups of this thread are complete.
__device__ __forceinline__ void bulk_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

}  // namespace sm100
}  // namespace ksb
