// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor, never multicast),
// tcgen05 (TMEM allocation, UMMA issue/commit, TMEM load/store) and the UMMA descriptors.
// Every wait on an mbarrier is bounded: when the cycle budget runs out the waiter records an
// error code and returns false, and the kernel tears down normally.
#pragma once
#include <cstdio>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef FG_WAIT_HINT_NS
#define FG_WAIT_HINT_NS 2000
#endif

namespace fg {

// ---------------------------------------------------------------------------------------------
// misc
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// Register re-balancing between warpgroups (every warp of the warpgroup must execute it).
template <int N>
__device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// generic-proxy writes to shared memory -> visible to the async proxy (UMMA / TMA reads)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Shared abort state of one CTA.  `flag` != 0 means some waiter gave up; everybody leaves.
struct AbortState {
  volatile int flag;
};

constexpr long long kWaitBudgetCycles = 3000000000LL;   // roughly 1.5-2 s at B200 clocks

// Bounded wait.  Returns false when the CTA is aborting (own time-out or somebody else's).
// `code` identifies the barrier in the error word written to `err` (global, may be null);
// `budget` is the number of cycles after which the waiter gives up.
__device__ __forceinline__ bool mbar_wait_budget(uint32_t bar, uint32_t parity, AbortState* ab, int* err, int code,
                                                 long long budget) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0) {
      if (ab->flag) {
#ifdef FG_WAIT_REPORT
        if ((threadIdx.x & 31) == 0) printf("block %d warp %d: gave up in wait %d (parity %u) after another waiter's time-out\n", blockIdx.x, threadIdx.x >> 5, code, parity);
#endif
        return false;
      }
      if (clock64() - t0 > budget) {
        ab->flag = 1;
        if (err) atomicCAS(err, 0, code);
#ifdef FG_WAIT_REPORT
        if ((threadIdx.x & 31) == 0) printf("block %d warp %d: time-out in wait %d (parity %u)\n", blockIdx.x, threadIdx.x >> 5, code, parity);
#endif
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, AbortState* ab, int* err, int code) {
  return mbar_wait_budget(bar, parity, ab, err, code, kWaitBudgetCycles);
}

// Same bounded wait for roles whose waits are long and not latency critical (TMA producers, the
// scheduler): the warp sleeps between polls instead of occupying an issue slot.
#ifndef FG_WAIT_SLEEP_NS
#define FG_WAIT_SLEEP_NS 64
#endif
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, AbortState* ab, int* err, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    __nanosleep(FG_WAIT_SLEEP_NS);
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0) {
      if (ab->flag) return false;
      if (clock64() - t0 > kWaitBudgetCycles) {
        ab->flag = 1;
        if (err) atomicCAS(err, 0, code);
        return false;
      }
    }
  }
}

// Whole-warp variant for warp-uniform control flow (the UMMA issuer): every lane polls, the outcome
// is made uniform so that a following elect.sync sees a converged warp.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, AbortState* ab, int* err, int code) {
  const bool ok = mbar_wait(bar, parity, ab, err, code);
  return __all_sync(0xffffffffu, ok);
}

// Wait used only on the abort path: short budget, no error recording.
__device__ __forceinline__ void mbar_wait_brief(uint32_t bar, uint32_t parity) {
  long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > 2000000LL) return;
  }
}

// ---------------------------------------------------------------------------------------------
// TMA tile loads (global -> shared), completion on an mbarrier.  No multicast anywhere.
// The innermost coordinate times the element size must be a multiple of 16 bytes.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: tensor memory management
// ---------------------------------------------------------------------------------------------
// One full warp calls alloc; the TMEM base address lands in shared memory at `dst_smem`.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// tcgen05: UMMA descriptors
// ---------------------------------------------------------------------------------------------
// Instruction descriptor for kind::f16 with bf16 A/B and fp32 accumulation.
//   bits [4,6) D format (1 = f32), [7,10) A format (1 = bf16), [10,13) B format (1 = bf16),
//   bit 15 A major (0 = K-major), bit 16 B major (1 = MN-major), [17,23) N>>3, [24,29) M>>4.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | (uint32_t(N >> 3) << 17) |
         (uint32_t(M >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle.  Rows of the operand tile are 128 bytes
// (64 bf16) apart, groups of 8 rows are `sbo_bytes` apart.
//   K-major operand  : a row is one M/N index holding 64 consecutive K elements; one UMMA (K=16)
//                      reads 32 bytes of each row, so successive K steps advance the start
//                      address by 32 bytes; LBO is unused.
//   MN-major operand : a row is one K index holding 64 consecutive M/N elements; 8-row groups
//                      (K) are `sbo_bytes` apart and successive 64-element MN chunks are
//                      `lbo_bytes` apart.
//   bits [0,14) address>>4, [16,30) LBO>>4, [32,46) SBO>>4, [46,48) version = 1, [61,64) layout = 2.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return uint64_t((saddr & 0x3FFFFu) >> 4) | (uint64_t((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         (uint64_t((sbo_bytes >> 4) & 0x3FFFu) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}

// ---------------------------------------------------------------------------------------------
// tcgen05: MMA issue (one thread), commit
// ---------------------------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]   (A is K-major, bf16 packed two per 32-bit TMEM column)
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Issue pattern: the issuing warp stays converged, elects one lane ONCE per product (`if (elect_one()) { all
// the product's tcgen05.mma and its commits } __syncwarp();`) and keeps the surrounding loop warp-uniform.
// Electing a lane for every single instruction makes the issue itself the limit as soon as a product has more
// than four shared-memory-operand instructions: measured, with products issued back to back, 115 clocks per
// 128x128x16 UMMA against the 64 clocks the tensor pipe needs (the D = 128 score product then takes 918 clocks
// instead of 513; inside the attention kernels, where other things bound a step, the difference is 0-7 %).
// mbarrier arrives once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void umma_commit_elect(uint32_t bar) {
  if (elect_one()) umma_commit(bar);
}

// ---------------------------------------------------------------------------------------------
// tcgen05: TMEM <-> registers.  Shape 32x32b: warp w of a warpgroup touches TMEM lanes
// [32*(w%4), 32*(w%4)+32); thread t gets lane 32*(w%4)+t and N consecutive 32-bit columns.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// numerics helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Packed fp32 pairs (sm_100 f32x2 instructions): half the instruction count of scalar FFMA/FADD.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// 2^x for a pair of values on the FMA pipe instead of the MUFU: x = n + f with n = round(x) taken from the
// low mantissa bits of x + 1.5 * 2^23, f in [-0.5, 0.5], a cubic minimax polynomial for 2^f (relative error
// below 1e-4, far under the resolution of the bf16 probabilities it feeds) and n added into the exponent
// field.  Inputs are clamped at -126 (results below 2^-126 do not matter to a softmax).
__device__ __forceinline__ void ex2_poly2(uint64_t x2, float& p0, float& p1) {
  float x0, x1;
  f2_unpack(x2, x0, x1);
  x0 = fmaxf(x0, -126.0f);
  x1 = fmaxf(x1, -126.0f);
  const uint64_t x = f2_pack(x0, x1);
  const uint64_t magic = f2_pack(12582912.0f, 12582912.0f);            // 1.5 * 2^23
  const uint64_t xr = f2_add(x, magic);                                // integer part in the low mantissa bits
  const uint64_t xi = f2_add(xr, f2_pack(-12582912.0f, -12582912.0f));
  const uint64_t f = f2_fma(xi, f2_pack(-1.0f, -1.0f), x);
  uint64_t q = f2_fma(f, f2_pack(0.05517160892486572f, 0.05517160892486572f),
                      f2_pack(0.2426111102104187f, 0.2426111102104187f));
  q = f2_fma(q, f, f2_pack(0.6932609677314758f, 0.6932609677314758f));
  q = f2_fma(q, f, f2_pack(0.9999280571937561f, 0.9999280571937561f));
  float q0, q1, r0, r1;
  f2_unpack(q, q0, q1);
  f2_unpack(xr, r0, r1);
  p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(r0) << 23));
  p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(r1) << 23));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Byte offset of the 16-byte chunk `chunk` (0..7) of row `row` inside a 128B-swizzled tile whose
// rows are 128 bytes; the tile base must be 1024-byte aligned.
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

}  // namespace fg

// Cycle accounting for tuning builds (-DFG_STATS); compiled out otherwise.
#ifdef FG_STATS
#define FG_TW(acc, expr) do { long long t__ = clock64(); expr; acc += clock64() - t__; } while (0)
#define FG_CLK() clock64()
#else
#define FG_TW(acc, expr) do { expr; } while (0)
#define FG_CLK() 0ll
#endif
