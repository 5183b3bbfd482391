// tcgen05 / TMEM / mbarrier primitives for sm_100a, as thin inline-PTX wrappers.
//
// Conventions used by the KDA kernels:
//   * cta_group::1 only; one elected lane issues tcgen05.mma and tcgen05.commit, predicated inside a warp-convergent loop.
//   * Shared-memory operands use the canonical swizzled layouts of the 5th-generation tensor core:
//       K-major  SW128: rows (M or N index) of 128 bytes of K, 8-row groups 1024 B apart (SBO), 16-byte chunks of a
//                       row XOR-swizzled with (row % 8); a K slice of one instruction is 32 bytes and is selected by
//                       advancing the descriptor's start address inside the 128-byte row.
//       MN-major SW128: rows are K indices holding 128 bytes of M/N-contiguous data, 8 K-rows form a 1024-byte atom;
//                       LBO = byte distance between atoms along M/N, SBO = byte distance between 8-row K groups.
//                       (16-bit operands; 32-bit MN-major operands need the 32-byte-base variant, see
//                       mnmajor_f32_off.)
//     Tiles are 1024-byte aligned so that the address-bit swizzle of the hardware equals the (row % 8) rule above.
//   * Every wait on an mbarrier is bounded: after `limit_ns` of wall time (kWaitLimitNs unless the launch overrides it)
//     the waiter raises the CTA's abort flag and carries on as if the wait had succeeded, so control flow (and every
//     barrier count) stays intact, the kernel drains, frees its tensor memory and returns; the host reads the error
//     code from the status word.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace kda {
namespace umma {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // a wait is abandoned after about two seconds

// ---------------------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}\n" :: "r"(bar) : "memory");
}
// Potentially blocking test: the hardware may suspend the thread until the phase completes or a time limit of its own
// passes, so a waiting warp does not take issue slots from the warps it is waiting for.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity), "r"(4000u) : "memory");
  return ok != 0;
}
// non-blocking test of a phase (never suspends the thread)
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
// Bounded wait of ONE thread.  `abort_flag` is a shared-memory int; returns false when the wait was abandoned
// (after kWaitLimitNs of wall time, or as soon as another thread of the CTA has given up).  `sleep_ns` > 0 makes the
// waiter sleep between polls so that it does not take issue slots from the warps it is waiting for.
// The polling loop is kept out of line: it is instantiated at dozens of wait sites, and instruction-cache footprint is
// what limits the role-specialised kernels.
// `abort_flag` points at the CTA's control words in shared memory: [0] abort code, [2..3] the wait limit in ns (64 bit).
__device__ __forceinline__ unsigned long long wait_limit_of(volatile int* abort_flag) {
  return *reinterpret_cast<volatile unsigned long long*>(abort_flag + 2);
}
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, unsigned sleep_ns) {
  const unsigned long long limit_ns = wait_limit_of(abort_flag);
  unsigned long long t0 = 0;
  uint32_t n = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (sleep_ns) __nanosleep(sleep_ns);
    if (*abort_flag != 0) return false;
    if ((++n & 63u) == 0) {
      const unsigned long long now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) {
        atomicCAS(const_cast<int*>(abort_flag), 0, code);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, unsigned sleep_ns = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, code, sleep_ns);
}
// Bounded wait that does NOT return early when the CTA has already given up elsewhere: used before a CTA leaves, for
// asynchronous work (bulk copies, tensor-core instructions) that must not be left in flight.  Returns false when the
// limit ran out (the caller records the code; nothing more can be done).
__device__ __noinline__ bool mbar_wait_drain(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const unsigned long long limit_ns = wait_limit_of(abort_flag);
  unsigned long long t0 = 0;
  uint32_t n = 0;
  while (!mbar_try_wait(bar, parity)) {
    __nanosleep(64);
    if ((++n & 63u) == 0) {
      const unsigned long long now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) return false;
    }
  }
  return true;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
// generic-proxy writes to shared memory -> visible to the async proxy (tcgen05.mma operand reads)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" :: "r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {    // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" :: "r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets row (lane base + i), registers = columns
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
// 32 lanes x 16 columns
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
      :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
         "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
         "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
         "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
         "r"(r[30]), "r"(r[31])
      : "memory");
}

// ---------------------------------------------------------------------------------------------- descriptors
constexpr uint32_t FMT_BF16 = 1, FMT_TF32 = 2;

// Instruction descriptor of kind::f16 / kind::tf32 with fp32 accumulation: D format bits [4,6) = 1 (F32), A format
// [7,10), B format [10,13), negate A bit 13, negate B bit 14, A major bit 15, B major bit 16 (0 = K-major,
// 1 = MN-major), N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, int M, int N, int a_mn_major, int b_mn_major, int neg_b) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)neg_b << 14) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Shared-memory matrix descriptor: start address >> 4 in [0,14), LBO >> 4 in [16,30), SBO >> 4 in [32,46),
// version 1 in [46,48), layout type in [61,64) (2 = 128-byte swizzle, 4 = 64-byte swizzle).
constexpr uint64_t LAYOUT_SW128_BASE32B = 1, LAYOUT_SW128 = 2, LAYOUT_SW64 = 4;
__device__ __forceinline__ uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t layout) {
  return (uint64_t)((smem_addr & 0x3ffffu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
         (1ull << 46) | (layout << 61);
}

// ---------------------------------------------------------------------------------------------- MMA issue
// Warp-convergent issue.  The tensor-core instructions take their descriptors and addresses from warp-uniform
// registers.  When the issuing code sits inside a one-lane branch the compiler has to move every operand from a
// vector register into a uniform one right before each instruction, which serialises at roughly 50 cycles per
// MMA; when the WHOLE warp runs the issuing code with warp-uniform operands and only the instruction itself is
// predicated on the elected lane, the operands are computed in uniform registers and an MMA issues in under 20
// cycles.  `go` is the result of elect_one() taken once: the same lane must issue the MMAs and their commits.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred;
}
// D (tensor memory) (+)= A (shared memory) * B (shared memory), bf16 operands
__device__ __forceinline__ void mma_ss_f16_pred(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate, uint32_t go) {
  asm volatile("{\n .reg .pred p, q;\n setp.ne.b32 p, %4, 0;\n setp.ne.b32 q, %5, 0;\n"
               " @q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(go) : "memory");
}
// D (tensor memory) (+)= A (tensor memory, fp32 columns read as tf32) * B (shared memory, tf32)
__device__ __forceinline__ void mma_ts_tf32_pred(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate, uint32_t go) {
  asm volatile("{\n .reg .pred p, q;\n setp.ne.b32 p, %4, 0;\n setp.ne.b32 q, %5, 0;\n"
               " @q tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n}\n"
               :: "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(go) : "memory");
}
// the mbarrier receives one arrival once every tcgen05.mma issued so far by the elected lane has completed
__device__ __forceinline__ void mma_commit_pred(uint32_t bar, uint32_t go) {
  asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %1, 0;\n"
               " @q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n" :: "r"(bar), "r"(go) : "memory");
}

// ---------------------------------------------------------------------------------------------- tile addressing
// K-major SW128 tile of 32-bit elements, rows of 128 bytes (32 elements), K blocks `kblock_bytes` apart:
// byte offset of element (row, k).
__device__ __forceinline__ uint32_t kmajor_f32_off(int row, int k, uint32_t kblock_bytes) {
  return (uint32_t)(k >> 5) * kblock_bytes + (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u +
         (uint32_t)((((k & 31) >> 2) ^ (row & 7)) << 4) + (uint32_t)(k & 3) * 4u;
}
// MN-major tile of 32-bit elements in the 128-byte swizzle with 32-byte base (layout type 1, the only MN-major form
// the tensor core accepts for tf32): K rows of 128 bytes (32 M/N elements), 4 K-rows form a 512-byte atom whose
// 32-byte pieces are XOR-ed with (k % 4); atom (mn block, k group of 4) at mn_block * lbo + k_group * sbo.
__device__ __forceinline__ uint32_t mnmajor_f32_off(int mn, int k, uint32_t lbo, uint32_t sbo) {
  return (uint32_t)(mn >> 5) * lbo + (uint32_t)(k >> 2) * sbo + (uint32_t)(k & 3) * 128u +
         (uint32_t)((((mn & 31) >> 3) ^ (k & 3)) << 5) + (uint32_t)(mn & 7) * 4u;
}
// MN-major SW128 tile of 16-bit elements (64 M/N elements per 128-byte row).
__device__ __forceinline__ uint32_t mnmajor_b16_off(int mn, int k, uint32_t lbo, uint32_t sbo) {
  return (uint32_t)(mn >> 6) * lbo + (uint32_t)(k >> 3) * sbo + (uint32_t)(k & 7) * 128u +
         (uint32_t)((((mn & 63) >> 3) ^ (k & 7)) << 4) + (uint32_t)(mn & 7) * 2u;
}
// K-major SW64 tile of 16-bit elements: rows of 64 bytes (32 elements), 8-row groups 512 B apart; the 16-byte chunk
// index is XOR-ed with address bits [7,9) = (row / 2) % 4.
__device__ __forceinline__ uint32_t kmajor_b16_sw64_off(int row, int k) {
  return (uint32_t)row * 64u + (uint32_t)((((k >> 3) ^ ((row >> 1) & 3)) & 3) << 4) + (uint32_t)(k & 7) * 2u;
}

}  // namespace umma
}  // namespace kda
