// Shared device-side primitives for the sm_100a kernels: mbarrier, TMA
// (cp.async.bulk.tensor), tcgen05 (TMEM alloc / mma / commit / ld / st) and
// the UMMA shared-memory / instruction descriptors, all as inline PTX.
//
// Waiting policy: every spin on an mbarrier is bounded by wall time
// (globaltimer).  When a wait runs out the kernel records a status word in
// global memory, raises a CTA-wide abort flag in shared memory, and every
// role falls through to the common exit (TMEM freed, no trap).  The host
// turns a non-zero status word into an exception.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace imf {

#define IMF_DEVICE __device__ __forceinline__

// ---------------------------------------------------------------- misc ----
IMF_DEVICE uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
IMF_DEVICE uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
IMF_DEVICE bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P1;\n\t"
      "elect.sync _|P1, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// status codes written to the global status word (0 = ok)
enum : int {
  STATUS_OK = 0,
  STATUS_TIMEOUT_TMA = 1,     // a consumer waited too long for a TMA load
  STATUS_TIMEOUT_MMA = 2,     // waited too long for a tcgen05.commit arrival
  STATUS_TIMEOUT_SOFTMAX = 3, // MMA warp waited too long for the softmax warps
  STATUS_TIMEOUT_EMPTY = 4,   // producer waited too long for a free stage
  STATUS_BAD_ARG = 5,
  STATUS_TIMEOUT_PEER = 6,    // waited too long for another rank's flag
  STATUS_TIMEOUT_TURN = 7,    // waited too long for its turn in a fixed-order accumulation
};

// -------------------------------------------------------------- mbarrier ---
IMF_DEVICE void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
IMF_DEVICE void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
IMF_DEVICE void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
IMF_DEVICE void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
IMF_DEVICE void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
IMF_DEVICE bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// non-blocking probe of a phase (never suspends the thread)
IMF_DEVICE bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

#ifndef IMF_WAIT_LIMIT_NS
#define IMF_WAIT_LIMIT_NS 2000000000ull  // 2 s
#endif

// Bounded wait.  Returns false (and raises the abort flag) on timeout or when
// another role already aborted.  `abort_flag` lives in shared memory.
IMF_DEVICE bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                          int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > IMF_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

// Fixed-order accumulation: wait (bounded) until the counter of a query tile shows this CTA's
// ordinal / hand the tile on after this CTA's add has been performed.  A CTA that gives up
// records it in the status word; everyone else who is waiting sees the word and gives up too.
IMF_DEVICE bool turn_wait(const int* addr, int want, volatile int* abort_flag, int* status) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    if (v == want) {
      asm volatile("fence.proxy.async.global;" ::: "memory");   // the add that follows is a TMA op
      return true;
    }
    if ((++spins & 31u) == 0) {
      if (*abort_flag) return false;
      if (status && *reinterpret_cast<volatile int*>(status) != 0) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > IMF_WAIT_LIMIT_NS) {
        if (status) atomicCAS(status, 0, STATUS_TIMEOUT_TURN);
        return false;
      }
    }
  }
}
IMF_DEVICE void turn_pass(int* addr, int value) {
  asm volatile("fence.proxy.async.global;" ::: "memory");
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(addr), "r"(value) : "memory");
}

// ------------------------------------------------------------------ TMA ----
IMF_DEVICE void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
IMF_DEVICE void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0),
      "r"(c1)
      : "memory");
}
IMF_DEVICE void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0),
      "r"(c1), "r"(c2)
      : "memory");
}
IMF_DEVICE void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0),
      "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
IMF_DEVICE void tma_store_2d(const CUtensorMap* m, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}
IMF_DEVICE void tma_store_3d(const CUtensorMap* m, const void* src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
// the shared-memory source of every committed bulk store has been read
IMF_DEVICE void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
IMF_DEVICE void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
IMF_DEVICE void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// --------------------------------------------------------------- tcgen05 ---
IMF_DEVICE void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
IMF_DEVICE void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
IMF_DEVICE void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
IMF_DEVICE void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
IMF_DEVICE void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
IMF_DEVICE void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
IMF_DEVICE void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// mbarrier arrive when all previously issued tcgen05 async ops of this thread
// have completed
IMF_DEVICE void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar))
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
IMF_DEVICE void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
IMF_DEVICE void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// fp8 (e4m3 / e5m2, chosen by the instruction descriptor) x fp8 -> fp32; K = 32 per instruction
IMF_DEVICE void mma_ss_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// int8 x int8 -> int32
IMF_DEVICE void mma_ss_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor (kind::f16 / kind::i8), M in {64,128}, N % 8 == 0.
//   [4,6) D format (1 = f32, 2 = s32)   [7,10) A format   [10,13) B format
//   [15] A major (0 = K)   [16] B major (0 = K, 1 = MN)
//   [17,23) N >> 3   [24,29) M >> 4
constexpr uint32_t FMT_F16 = 0, FMT_BF16 = 1, FMT_S8 = 1;
constexpr uint32_t FMT_E4M3 = 0, FMT_E5M2 = 1;      // kind::f8f6f4
__host__ __device__ constexpr uint32_t make_idesc(uint32_t m, uint32_t n, uint32_t a_fmt,
                                                  uint32_t b_fmt, uint32_t d_fmt,
                                                  uint32_t a_mn_major, uint32_t b_mn_major) {
  return (d_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}
__host__ __device__ constexpr uint32_t idesc_bf16(uint32_t m, uint32_t n, uint32_t a_mn = 0,
                                                  uint32_t b_mn = 0) {
  return make_idesc(m, n, FMT_BF16, FMT_BF16, 1, a_mn, b_mn);
}

// Shared-memory matrix descriptor for the 128-byte-swizzled canonical layouts
// (tile base 1024-byte aligned, rows of 128 bytes as written by TMA
// SWIZZLE_128B).
//   K-major operand  [rows = M or N][64 x 16-bit along K]: 8-row groups are
//     1024 B apart (SBO); a K step of 16 elements advances the start by 32 B.
//   MN-major operand [rows = K][64 x 16-bit along M or N]: 8-row K groups are
//     1024 B apart (SBO); 64-element MN panels are LBO bytes apart.
//   bits [0,14) start >> 4, [16,30) LBO >> 4, [32,46) SBO >> 4, [46,48) = 1,
//   [61,64) layout (2 = SWIZZLE_128B).
IMF_DEVICE uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}
IMF_DEVICE uint64_t sdesc_kmajor(uint32_t smem_addr) { return make_sdesc(smem_addr, 16, 1024); }
IMF_DEVICE uint64_t sdesc_mnmajor(uint32_t smem_addr, uint32_t panel_bytes) {
  return make_sdesc(smem_addr, panel_bytes, 1024);
}

// K-major operand with 32-byte rows (16 x 16-bit along K = one MMA K-step), SWIZZLE_32B:
// 8-row groups are 256 B apart.  Used for the narrow "constant" operand bands that let the
// tensor core add a per-row term to an accumulator (rows of ones on one side, the term as a
// bf16 (hi, lo) pair on the other).
IMF_DEVICE uint64_t sdesc_kmajor_sw32(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(256 >> 4) << 32;
  d |= 1ull << 46;
  d |= 6ull << 61;                               // SWIZZLE_32B
  return d;
}

// TMEM address helpers: bits [16,32) lane, [0,16) column
IMF_DEVICE uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// tcgen05.ld 32x32b: thread i of the warp gets TMEM lane (base lane + i),
// N consecutive 32-bit columns.
#define IMF_LD_ARGS8(r, o)                                                                  \
  "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]),            \
      "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7])
#define IMF_ST_ARGS8(r, o)                                                                  \
  "r"(r[o + 0]), "r"(r[o + 1]), "r"(r[o + 2]), "r"(r[o + 3]), "r"(r[o + 4]), "r"(r[o + 5]),  \
      "r"(r[o + 6]), "r"(r[o + 7])

IMF_DEVICE void tmem_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : IMF_LD_ARGS8(r, 0)
               : "r"(taddr)
               : "memory");
}
IMF_DEVICE void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : IMF_LD_ARGS8(r, 0), IMF_LD_ARGS8(r, 8)
      : "r"(taddr)
      : "memory");
}
IMF_DEVICE void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : IMF_LD_ARGS8(r, 0), IMF_LD_ARGS8(r, 8), IMF_LD_ARGS8(r, 16), IMF_LD_ARGS8(r, 24)
      : "r"(taddr)
      : "memory");
}
IMF_DEVICE void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(taddr), IMF_ST_ARGS8(r, 0)
               : "memory");
}
IMF_DEVICE void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), IMF_ST_ARGS8(r, 0), IMF_ST_ARGS8(r, 8)
      : "memory");
}
IMF_DEVICE void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), IMF_ST_ARGS8(r, 0), IMF_ST_ARGS8(r, 8), IMF_ST_ARGS8(r, 16),
      IMF_ST_ARGS8(r, 24)
      : "memory");
}

// ------------------------------------------------------------- numerics ----
IMF_DEVICE float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
IMF_DEVICE uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
IMF_DEVICE float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
IMF_DEVICE float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

}  // namespace imf
