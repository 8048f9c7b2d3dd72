// Inline-PTX wrappers for the Blackwell (sm_100a) units the Flash-MVPA kernels use:
// mbarrier, TMA (cp.async.bulk.tensor, no cluster multicast anywhere), tcgen05 MMA with
// TMEM accumulators, tcgen05.ld/st, and the shared-memory / instruction descriptors.
//
// Every wait is bounded in time: once a deadline on the %globaltimer clock has passed it records a
// code in a status word and returns false, so a protocol bug surfaces as an error status instead
// of a hung GPU.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace mvpa {
namespace ptx {

constexpr uint64_t kDefaultWaitNs = 2000000000ull;  // a wait gives up after two seconds
constexpr uint32_t kPollsPerClockRead = 32;         // try_wait polls between two looks at the clock
// Per translation unit: a non-zero value (microseconds) replaces the default deadline.  Only the wait
// self-test sets it (to make a wait run out quickly); product kernels run with the default.
static __device__ unsigned int g_wait_limit_us = 0;

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint64_t wait_limit_ns() {
  const unsigned int us = *(volatile unsigned int*)&g_wait_limit_us;
  return us != 0 ? (uint64_t)us * 1000ull : kDefaultWaitNs;
}
__device__ __forceinline__ void record_giveup(int* status, int code) {
  if (status != nullptr) {
    atomicCAS(status, 0, code);
    status[(code % 100) & 63] = code;  // every wait that gave up, for diagnosis (the first word keeps the first)
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------- mbarrier -----------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  On time-out stores `code` to *status (first writer wins) and returns false.
// A phase that has already completed is caught by the non-suspending test first; the clock is
// only consulted once a first batch of polls has failed, so a short wait never reads it.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
  if (mbar_test_wait(bar, parity)) return true;
  for (uint32_t i = 0; i < kPollsPerClockRead; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  const uint64_t t0 = global_timer_ns(), limit = wait_limit_ns();
  do {
    for (uint32_t i = 0; i < kPollsPerClockRead; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
  } while (global_timer_ns() - t0 < limit);
  record_giveup(status, code);
  return false;
}

// Variants on a shared-space address (the MMA-issuing warp keeps barrier addresses as integers
// so that no generic-to-shared conversion sits in its instruction stream).
__device__ __forceinline__ bool mbar_test_wait_a(uint32_t bar, uint32_t parity) {
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
__device__ __forceinline__ bool mbar_try_wait_a(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_a(uint32_t bar, uint32_t parity, int* status, int code) {
  if (mbar_test_wait_a(bar, parity)) return true;
  for (uint32_t i = 0; i < kPollsPerClockRead; ++i) {
    if (mbar_try_wait_a(bar, parity)) return true;
  }
  const uint64_t t0 = global_timer_ns(), limit = wait_limit_ns();
  do {
    for (uint32_t i = 0; i < kPollsPerClockRead; ++i) {
      if (mbar_try_wait_a(bar, parity)) return true;
    }
  } while (global_timer_ns() - t0 < limit);
  record_giveup(status, code);
  return false;
}
// --------------------------------- TMA --------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 3-D tiled load (x = innermost).  x must keep the 16-byte rule: x * sizeof(elem) % 16 == 0.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
      "%5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x,
                                            int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
      "%5, %6}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x,
                                            int y, int z, int w, int v) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
      "%5, %6, %7}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(v)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* smem_src, int x, int y,
                                             int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
// 5-D tiled store; elements outside the tensor are not written.  Coordinates must not be negative.
__device__ __forceinline__ void tma_store_5d(const CUtensorMap* m, const void* smem_src, int x, int y,
                                             int z, int w, int v) {
  asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(v)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
// Generic-proxy writes to shared memory -> visible to the async proxy (TMA store, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------- tcgen05 ------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {  // one full warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // one full warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// TMEM -> registers: each thread of a warp reads its own lane (row), N consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
      "%15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld1(uint32_t taddr, uint32_t& r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st1(uint32_t taddr, uint32_t r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(r) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
      "%15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
      "%15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ------------------------------ descriptors ---------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 version field = 1.
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) version = 1     bits [61,64) layout = 2 (SW128)
// K-major operand  (rows of 64 bf16 = 128 B, 8-row groups of 1024 B): SBO = 1024, LBO unused (1).
// MN-major operand (MN contiguous, 64 per 128-B row; one row per K index): SBO = 1024 between
//   groups of 8 K-rows, LBO = byte distance between 64-wide MN chunks.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// The same descriptor split into 32-bit halves: the low word carries the start address (and LBO),
// so stepping through a tile is one 32-bit add per MMA instead of rebuilding 64 bits.
struct DescHalves {
  uint32_t lo, hi;
};
__device__ __forceinline__ DescHalves make_desc_halves_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                             uint32_t sbo_bytes) {
  DescHalves d;
  d.lo = ((smem_addr >> 4) & 0x3FFF) | (((lbo_bytes >> 4) & 0x3FFF) << 16);
  d.hi = ((sbo_bytes >> 4) & 0x3FFF) | (1u << 14) | (2u << 29);
  return d;
}
// ---------------------- warp-convergent issue (elected lane) ----------------------
// The tcgen05 instructions take their descriptors and addresses from warp-uniform registers.  Issued
// from a branch only one lane enters, each MMA costs that lane 80-160 cycles (more when the other warps
// of the SM are busy); issued by the whole warp in convergent code, with only the instruction itself
// guarded by the elected lane's predicate, the same stream runs at the tensor pipe's own rate (64 cycles
// for M128 N128 K16).  These variants take that predicate (`el`, 1 on the elected lane, 0 elsewhere);
// every lane of the warp must call them together with identical arguments.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred;
}
__device__ __forceinline__ void mma_commit_w(uint32_t el, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred pe;\n\tsetp.ne.b32 pe, %1, 0;\n\t"
      "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar),
      "r"(el)
      : "memory");
}
__device__ __forceinline__ void mma_ss_w(uint32_t el, uint32_t d_tmem, DescHalves a, uint32_t a_off_bytes,
                                         DescHalves b, uint32_t b_off_bytes, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, pe;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "setp.ne.b32 pe, %7, 0;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
      "r"(a.lo + (a_off_bytes >> 4)), "r"(a.hi), "r"(b.lo + (b_off_bytes >> 4)), "r"(b.hi), "r"(idesc),
      "r"(accumulate), "r"(el)
      : "memory");
}
__device__ __forceinline__ void mma_ts_w(uint32_t el, uint32_t d_tmem, uint32_t a_tmem, DescHalves b,
                                         uint32_t b_off_bytes, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, pe;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.ne.b32 pe, %6, 0;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b.lo + (b_off_bytes >> 4)), "r"(b.hi), "r"(idesc), "r"(accumulate), "r"(el)
      : "memory");
}
// Four consecutive K-steps of  D[tmem] (+)= A[tmem] * B[smem]  (A: 16 keys = 8 packed columns per
// step; B: MN-major, `b_step16` 16-byte descriptor units per step from low word `b_lo`).
__device__ __forceinline__ void mma_ts_x4_w(uint32_t el, uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                            uint32_t b_hi, uint32_t b_step16, uint32_t idesc,
                                            uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p0, p1, pe;\n\t.reg .b64 db;\n\t.reg .b32 lo;\n\t"
      "setp.ne.b32 p0, %6, 0;\n\t"
      "setp.ne.b32 pe, %7, 0;\n\t"
      "setp.eq.b32 p1, 0, 0;\n\t"
      "mov.b32 lo, %2;\n\t"
      "mov.b64 db, {lo, %3};\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %5, p0;\n\t"
      "add.u32 lo, lo, %4;\n\t mov.b64 db, {lo, %3};\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1 + 8], db, %5, p1;\n\t"
      "add.u32 lo, lo, %4;\n\t mov.b64 db, {lo, %3};\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1 + 16], db, %5, p1;\n\t"
      "add.u32 lo, lo, %4;\n\t mov.b64 db, {lo, %3};\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1 + 24], db, %5, p1;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(b_step16), "r"(idesc), "r"(accumulate_first), "r"(el)
      : "memory");
}

// Instruction descriptor for kind::f16 with bf16 A/B and fp32 accumulation.
//   [4,6) D fmt = 1 (f32)  [7,10) A fmt = 1 (bf16)  [10,13) B fmt = 1 (bf16)
//   [15] A major (0 = K)   [16] B major (0 = K, 1 = MN)   [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

// Same with both operand majors selectable (bit 15: A is MN-major, bit 16: B is MN-major).
__host__ __device__ constexpr uint32_t make_idesc_bf16_ab(int M, int N, int a_mn_major, int b_mn_major) {
  return make_idesc_bf16(M, N, b_mn_major) | ((uint32_t)a_mn_major << 15);
}

// Byte offset of element (row, col) of a [rows x 64] bf16 tile stored with the 128-byte swizzle
// TMA and tcgen05 agree on: 16-byte chunk index XOR (row mod 8).  Tile base must be 1024-aligned.
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
  const int chunk = (col >> 3) ^ (row & 7);
  return (uint32_t)(row * 128 + chunk * 16 + (col & 7) * 2);
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace ptx
}  // namespace mvpa
