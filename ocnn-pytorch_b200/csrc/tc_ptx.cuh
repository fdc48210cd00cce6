// Inline-PTX wrappers for the Blackwell (sm_100a) primitives used by the
// tensor-core convolution kernels: mbarriers, cp.async, bulk copies, tcgen05
// MMA / TMEM.  Every wait is bounded: after about a second (WAIT_CYCLES, or SPIN_LIMIT polls) it gives up, raises
// the CTA-wide abort flag and the sticky device status word, and the kernel
// unwinds (frees its TMEM and returns) instead of hanging the GPU.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace oc {
namespace tc {

constexpr uint32_t SPIN_LIMIT = 1u << 24;
constexpr long long WAIT_CYCLES = 2000000000LL;  // about one second of SM clock

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar),
               "r"(bytes)
               : "memory");
}
// One poll.  The suspend-time hint lets the hardware park the thread until the
// phase completes or `hint_ns` elapse, instead of burning issue slots.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// Non-blocking poll (never parks the thread).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Busy-polling variant for the short, latency-critical waits of the main loop.
__device__ __forceinline__ bool mbar_spin(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status_word, int code) {
  if (mbar_test_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 0; i < 0xffffffffu; ++i) {
    if (mbar_test_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > WAIT_CYCLES) break;
    }
  }
  *abort_flag = 1;
  atomicMax(status_word, code);
  return false;
}
// Returns false if the wait was abandoned (own limit reached or another role
// already aborted).  `abort_flag` lives in shared memory.  `backoff_ns` > 0 adds a
// sleep between polls for roles whose waits are long (epilogue).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status_word, int code, uint32_t backoff_ns = 0) {
  if (mbar_try_wait(bar, parity, 2000u)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
    if (backoff_ns) __nanosleep(backoff_ns);
    if (mbar_try_wait(bar, parity, 20000u)) return true;
    if ((i & 15u) == 15u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > WAIT_CYCLES) break;
    }
  }
  *abort_flag = 1;
  atomicMax(status_word, code);
  return false;
}

// ---- cp.async (16-byte, L2 only), zero-fill when src_bytes == 0 -------------
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// wait until at most n (0..4) commit groups of this thread are pending
__device__ __forceinline__ void cp_async_wait_dyn(int n) {
  switch (n) {
    case 0: cp_async_wait<0>(); break;
    case 1: cp_async_wait<1>(); break;
    case 2: cp_async_wait<2>(); break;
    case 3: cp_async_wait<3>(); break;
    default: cp_async_wait<4>(); break;
  }
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// mbarrier arrival triggered by the completion of all prior cp.async of this thread;
// .noinc: it counts as one of the arrivals the barrier was initialised to expect.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// generic-proxy writes (st.shared) -> visible to the async proxy (tcgen05.mma).  The gathered
// operands need none: they arrive by cp.async whose completion is counted on the stage's
// mbarrier (cp.async.mbarrier.arrive.noinc), and the MMA warp issues after waiting on that
// barrier - the producer / consumer hand-off of CUTLASS's sm100 cp.async mainloop.  A fence per
// stage in the MMA warp was measured at 5 % of the benchmark step and changed no result.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- bulk copy global -> shared, completion counted on an mbarrier ----------
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Four rows of a 2-D tensor (tensor map with a box of `cols` x 1 and 128-byte swizzle) into four
// consecutive 128-byte lines of shared memory; rows outside the tensor read as zeros.  Completes
// 4 x box bytes on the mbarrier.  `col` x element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const void* tmap, int col, int r0, int r1, int r2, int r3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, "
      "%5, %6}], [%7];" ::"r"(dst),
      "l"(tmap), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(bar)
      : "memory");
}

// ---- TMEM -------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
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

// D[tmem] (+)= A[smem] * B[smem], fp16/bf16 inputs, fp32 accumulate; one thread issues.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// True in exactly one lane of a converged warp (always the same one).  The MMA-issuing
// warp runs its loop with all 32 lanes and predicates only the tcgen05 instructions with
// this: the loop state stays warp-uniform, so descriptors and addresses live in uniform
// registers and an MMA issues in ~11 cycles instead of ~54 when a single diverged
// thread runs the loop.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t.reg .b32 r;\n\t"
      "elect.sync r|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
// Arrives on `bar` when all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 16 consecutive fp32 columns: lane i of the warp gets row (lane base + i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- descriptors ------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100).
//   bits [0,14) start address >> 4, [16,30) leading byte offset >> 4,
//   [32,46) stride byte offset >> 4, [46,48) version, [61,64) layout (2 = SWIZZLE_128B)
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor for kind::f16: fp32 accumulator, A/B format 0 = f16, 1 = bf16,
// major 0 = K-major, 1 = MN-major; N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ __forceinline__ uint32_t make_idesc(int bf16, int a_mn_major, int b_mn_major, int M, int N) {
  return (1u << 4) | ((uint32_t)bf16 << 7) | ((uint32_t)bf16 << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Pins a value in a register.  Kernel parameters and values derived from them are otherwise
// re-read from the constant bank wherever they are used; in a warp that has just queued
// dozens of cp.async instructions such a load waits behind them (~300 cycles measured on the
// back edge of the producer loop).
__device__ __forceinline__ uint32_t pin_reg(uint32_t v) { asm volatile("" : "+r"(v)); return v; }
__device__ __forceinline__ int pin_reg(int v) { asm volatile("" : "+r"(v)); return v; }
__device__ __forceinline__ const uint8_t* pin_reg(const uint8_t* v) { asm volatile("" : "+l"(v)); return v; }

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace tc
}  // namespace oc
