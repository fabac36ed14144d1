// Thin inline-PTX wrappers for the Blackwell (sm_100a) tensor-core path:
// tensor memory (TMEM) allocation and access, tcgen05.mma with the A operand in TMEM,
// mbarriers with BOUNDED waits, and the shared-memory / instruction descriptors.
//
// Every wait in this file gives up after a fixed number of polls, records why in a
// device status word and raises a block-wide abort flag; callers then fall through to
// their teardown (TMEM is always freed) instead of hanging the GPU.
#pragma once

#include <cstdint>

namespace b200lut {
namespace tc {

// ---- device status (read by the host through b200lut_device_status) ---------------
enum : int {
  kStatusOk = 0,
  kStatusWaitFull = 1,    // MMA issuer gave up waiting for dequantised operands
  kStatusWaitEmpty = 2,   // a dequant warp gave up waiting for a free operand stage
  kStatusWaitDone = 3,    // the epilogue gave up waiting for the last MMA
  kStatusWaitLoad = 4     // a consumer gave up waiting for a bulk (TMA) load
};

constexpr long long kWaitCycles = 20000000;   // ~10 ms at 2 GHz: far beyond any healthy wait

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -----------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Non-blocking phase test.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
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

// Bounded wait. `abort_flag` is a shared-memory word: once any waiter in the block has
// timed out it is set, and every later wait returns at once, so a block that lost a
// signal drains in microseconds. The deadline is in SM clock cycles. Returns false on
// abort.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int why, long long limit = kWaitCycles) {
  if (mbar_test(bar, parity)) return true;
  if (*abort_flag) return false;
  const long long t0 = clock64();
  for (uint32_t i = 1;; ++i) {
    if (mbar_test(bar, parity)) return true;
    if ((i & 15u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) break;
    }
  }
  *abort_flag = 1;
  if (status) atomicCAS(status, kStatusOk, why);
  return false;
}

// ---- TMEM ---------------------------------------------------------------------------
// All of one warp must execute alloc / dealloc. ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// generic-proxy writes to shared memory -> visible to the async proxy (tcgen05.mma, TMA)
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Store a 16-row x 32-column (64 bf16 of K) operand block: the warp's lane (g = lane/4,
// t = lane%4) passes, for each of the four 8-column repetitions i, the registers
// (row g, col 8i+2t), (row g, col 8i+2t+1), (row g+8, col 8i+2t), (row g+8, col 8i+2t+1).
__device__ __forceinline__ void tmem_st_16x256b_x4(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}

// Load 16 consecutive 32-bit columns of the thread's own TMEM lane (lane = 32*(warp%4)+tid).
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// ---- descriptors --------------------------------------------------------------------
// Shared-memory matrix descriptor, K-major operand. Addresses and offsets in bytes.
//   layout 0: no swizzle — core matrices of 8 rows x 16 bytes, `lbo` between the two
//             8-element K halves of a K=16 step, `sbo` between 8-row groups;
//   layout 2: 128-byte swizzle — rows of 128 bytes, `sbo` between 8-row groups (1024).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo,
                                              uint32_t layout) {
  uint64_t d = 0;
  d |= uint64_t((addr >> 4) & 0x3FFFu);
  d |= uint64_t((lbo >> 4) & 0x3FFFu) << 16;
  d |= uint64_t((sbo >> 4) & 0x3FFFu) << 32;
  d |= uint64_t(1) << 46;                 // descriptor version of sm_100
  d |= uint64_t(layout & 7u) << 61;
  return d;
}

// Instruction descriptor of tcgen05.mma kind::f16: fp32 accumulate, A and B K-major.
// fmt: 0 = f16, 1 = bf16. M in {64, 128}; N a multiple of 16 (M = 128) up to 256.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt, uint32_t M, uint32_t N) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// D[tmem_d] (+)= A[tmem_a] * B[desc_b]; one thread issues. accumulate == 0 overwrites D.
__device__ __forceinline__ void mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// The four K = 16 steps of one 64-wide k-block in one instruction group: D (+)= A[a0 + 8 j] *
// B[desc + 32 j bytes], j = 0..3. The descriptor is passed as its two words (only the low
// one, which holds the start address in 16-byte units, changes between steps); the first
// step overwrites D when accumulate == 0. One thread issues.
__device__ __forceinline__ void mma_ts_kblock(uint32_t tmem_d, uint32_t a0, uint32_t desc_lo,
                                              uint32_t desc_hi, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 b0, b1, b2, b3;\n\t.reg .b32 l1, l2, l3, a1, a2, a3;\n\t"
      "setp.ne.b32 p, %5, 0;\n\tsetp.eq.b32 q, %6, %6;\n\t"
      "add.u32 l1, %2, 2;\n\tadd.u32 l2, %2, 4;\n\tadd.u32 l3, %2, 6;\n\t"
      "add.u32 a1, %1, 8;\n\tadd.u32 a2, %1, 16;\n\tadd.u32 a3, %1, 24;\n\t"
      "mov.b64 b0, {%2, %3};\n\tmov.b64 b1, {l1, %3};\n\tmov.b64 b2, {l2, %3};\n\tmov.b64 b3, {l3, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], b0, %4, {%6, %6, %6, %6}, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %4, {%6, %6, %6, %6}, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %4, {%6, %6, %6, %6}, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %4, {%6, %6, %6, %6}, q;\n\t}"
      :
      : "r"(tmem_d), "r"(a0), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// All MMAs issued so far by this thread arrive on `bar` when they complete.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// ---- CTA pairs (cta_group::2) ---------------------------------------------------------------------
// Two CTAs of a cluster work as one MMA unit: each keeps its 128 rows of the A operand in its own
// tensor memory and HALF of the B tile in its own shared memory; one thread of the leader (cluster
// rank 0) issues the MMAs, the tensor cores of both CTAs run them, each into its own accumulator.
// Shared-state addresses carry the CTA's rank in bit 24: clearing it names the leader's copy of a
// barrier, which is how the peer's arrivals and its bulk loads report to the leader. No load here
// is a multicast load.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on a barrier of any CTA of the cluster (shared::cluster address).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One warp of EACH CTA of the pair executes alloc / dealloc (same warp index, same dst offset).
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// The four K = 16 steps of one k-block on a CTA pair: D (256 rows over the two CTAs) (+)=
// A[a0 + 8 j in each CTA's tensor memory] * B[desc + 32 j bytes, half of its N rows in each CTA].
__device__ __forceinline__ void mma_ts_kblock_pair(uint32_t tmem_d, uint32_t a0, uint32_t desc_lo,
                                                   uint32_t desc_hi, uint32_t idesc,
                                                   uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 b0, b1, b2, b3;\n\t.reg .b32 l1, l2, l3, a1, a2, a3;\n\t"
      "setp.ne.b32 p, %5, 0;\n\tsetp.eq.b32 q, %6, %6;\n\t"
      "add.u32 l1, %2, 2;\n\tadd.u32 l2, %2, 4;\n\tadd.u32 l3, %2, 6;\n\t"
      "add.u32 a1, %1, 8;\n\tadd.u32 a2, %1, 16;\n\tadd.u32 a3, %1, 24;\n\t"
      "mov.b64 b0, {%2, %3};\n\tmov.b64 b1, {l1, %3};\n\tmov.b64 b2, {l2, %3};\n\tmov.b64 b3, {l3, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], b0, %4, {%6, %6, %6, %6, %6, %6, %6, %6}, p;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [a1], b1, %4, {%6, %6, %6, %6, %6, %6, %6, %6}, q;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [a2], b2, %4, {%6, %6, %6, %6, %6, %6, %6, %6}, q;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [a3], b3, %4, {%6, %6, %6, %6, %6, %6, %6, %6}, q;\n\t}"
      :
      : "r"(tmem_d), "r"(a0), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// All MMAs issued so far by this thread arrive, when complete, on the barrier at the same offset
// in both CTAs of the pair.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(uint16_t(3))
      : "memory");
}

}  // namespace tc
}  // namespace b200lut
