// Thin inline-PTX wrappers for the sm_100a features the GEMM uses: mbarrier, TMA tiled loads,
// tensor memory (TMEM) allocation, tcgen05.mma / commit / ld, and the matching fences.
// Every blocking wait is bounded: it gives up after a spin budget and reports failure so that
// a broken pipeline ends the kernel with a status word instead of hanging the device.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace qlin {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Budget of a bounded wait.  The first polls spin; after that every miss sleeps 64 ns and checks
// the CTA's abort flag and the wall clock (%globaltimer, nanoseconds).
constexpr uint32_t kSpinFast = 2048;
constexpr uint64_t kWaitBudgetNs = 2000000000ull;   // 2 s
constexpr uint64_t kDrainBudgetNs = 200000000ull;   // 0.2 s

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Waits for the phase with the given parity.  Returns false when the budget ran out or another
// thread of the CTA already raised `*abort_flag`.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinFast; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(64);
    if (*abort_flag) return false;
    if (global_timer_ns() - t0 > kWaitBudgetNs) return false;
  }
}

// Warp-level forms: mbarrier operations on one address are processed lane by lane, so a whole warp
// polling costs ~32x the latency of a single lane.  One lane polls, the result is broadcast; the
// warp is converged again when these return.
__device__ __forceinline__ bool warp_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  uint32_t ok = 0;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1u : 0u;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// Split form of a non-blocking poll: `begin` issues the test in lane 0 and returns a per-lane token
// without consuming the result, `end` broadcasts it.  Work placed between the two overlaps the
// barrier round trip (the warp issues in order and only stalls where the result is first read).
__device__ __forceinline__ uint32_t warp_mbar_test_begin(uint64_t* bar, uint32_t parity) {
  uint32_t ok = 0;
  if ((threadIdx.x & 31) == 0) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
  }
  return ok;
}
__device__ __forceinline__ bool warp_mbar_test_end(uint32_t token) {
  return __shfl_sync(0xffffffffu, token, 0) != 0;
}

// Bounded wait used while winding down: ignores the abort flag and uses a shorter budget.
__device__ __forceinline__ bool mbar_wait_drain(uint64_t* bar, uint32_t parity) {
  const uint64_t t0 = global_timer_ns();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(64);
    if (global_timer_ns() - t0 > kDrainBudgetNs) return false;
  }
}

// ---------------------------------------------------------------- TMA
// 2-D tiled load global -> shared, completion counted in bytes on `bar`.  x is the innermost
// (contiguous) coordinate and must keep x * element_size a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int32_t x,
                                            int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// ---------------------------------------------------------------- TMEM
// Whole-warp (.sync.aligned) operations: call with all 32 lanes converged.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive once on `bar` when every tcgen05 operation issued so far by this thread has finished.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle TMA writes (8-row x 128-byte atoms, 1024 bytes apart).  Stepping along K inside
// the 128-byte row is done by adding the byte offset (>> 4) to the low word.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                       // leading byte offset (unused when swizzled)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;               // stride byte offset: next 8-row group
  d |= static_cast<uint64_t>(1) << 46;                       // descriptor version of sm_100
  d |= static_cast<uint64_t>(2) << 61;                       // 128-byte swizzle
  return d;
}

// Instruction descriptor: dense, no negate, both operands K-major.
//   c_format: 1 = f32, 2 = s32;  ab_format: kind::i8 1 = signed 8-bit; kind::f8f6f4 0 = e4m3.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t c_format, uint32_t ab_format, uint32_t m, uint32_t n) {
  return (c_format << 4) | (ab_format << 7) | (ab_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] . B[smem]^T, issued by one thread.
template <int KIND_F8>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  if (KIND_F8) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// The issue helpers below are executed by a whole converged warp; one elected lane issues (guard
// predicate from elect.sync), so the surrounding loop stays free of divergent branches and its
// operands stay warp-uniform.

// One stage of the TMA producer: arm the barrier with the byte count, then load the A and B boxes.
__device__ __forceinline__ void tma_issue_stage(uint64_t* full_bar, uint32_t bytes, void* smem_a, const void* tmap_a,
                                                int32_t ya, void* smem_b, const void* tmap_b, int32_t yb, int32_t x) {
  asm volatile(
      "{\n\t"
      ".reg .pred pe;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "@pe mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t"
      "@pe cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%2], [%3, {%8, %4}], [%0];\n\t"
      "@pe cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%5], [%6, {%8, %7}], [%0];\n\t"
      "}" ::"r"(smem_u32(full_bar)),
      "r"(bytes), "r"(smem_u32(smem_a)), "l"(reinterpret_cast<uint64_t>(tmap_a)), "r"(ya), "r"(smem_u32(smem_b)),
      "l"(reinterpret_cast<uint64_t>(tmap_b)), "r"(yb), "r"(x)
      : "memory");
}

// One full 128-byte K block: four K=32-byte MMAs into the same accumulator (the first one
// overwrites it when `accumulate` is 0), then release the shared-memory stage through `empty_bar`.
template <int KIND_F8>
__device__ __forceinline__ void tc_mma4_release(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate, uint64_t* empty_bar) {
#define QLIN_MMA4(KIND)                                                                         \
  asm volatile(                                                                                 \
      "{\n\t"                                                                                   \
      ".reg .pred pe, pa, pt;\n\t"                                                              \
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"                                                   \
      "elect.sync _|pe, 0xffffffff;\n\t"                                                        \
      "setp.ne.b32 pa, %4, 0;\n\t"                                                              \
      "setp.ne.b32 pt, %3, 0;\n\t"                                                              \
      "add.s64 a1, %1, 2;\n\t"                                                                  \
      "add.s64 b1, %2, 2;\n\t"                                                                  \
      "add.s64 a2, %1, 4;\n\t"                                                                  \
      "add.s64 b2, %2, 4;\n\t"                                                                  \
      "add.s64 a3, %1, 6;\n\t"                                                                  \
      "add.s64 b3, %2, 6;\n\t"                                                                  \
      "@pe tcgen05.mma.cta_group::1.kind::" KIND " [%0], %1, %2, %3, pa;\n\t"                   \
      "@pe tcgen05.mma.cta_group::1.kind::" KIND " [%0], a1, b1, %3, pt;\n\t"                   \
      "@pe tcgen05.mma.cta_group::1.kind::" KIND " [%0], a2, b2, %3, pt;\n\t"                   \
      "@pe tcgen05.mma.cta_group::1.kind::" KIND " [%0], a3, b3, %3, pt;\n\t"                   \
      "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%5];\n\t"     \
      "}" ::"r"(d_tmem),                                                                        \
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(smem_u32(empty_bar))             \
      : "memory")
  if (KIND_F8) {
    QLIN_MMA4("f8f6f4");
  } else {
    QLIN_MMA4("i8");
  }
#undef QLIN_MMA4
}

// One accumulation chunk of NMMA (1, 2 or 4) K=32-byte MMAs into a fresh accumulator (the first MMA
// overwrites it), then the "accumulator full" commit on `tfull_bar`.
template <int KIND_F8, int NMMA>
__device__ __forceinline__ void tc_mma_chunk(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint64_t* tfull_bar) {
#define QLIN_CHUNK_HEAD                                   \
  "{\n\t"                                                 \
  ".reg .pred pe, pf, pt;\n\t"                            \
  ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"                 \
  "elect.sync _|pe, 0xffffffff;\n\t"                      \
  "setp.ne.b32 pt, %3, 0;\n\t"                            \
  "setp.eq.b32 pf, %3, 0;\n\t"                            \
  "add.s64 a1, %1, 2;\n\t"                                \
  "add.s64 b1, %2, 2;\n\t"                                \
  "add.s64 a2, %1, 4;\n\t"                                \
  "add.s64 b2, %2, 4;\n\t"                                \
  "add.s64 a3, %1, 6;\n\t"                                \
  "add.s64 b3, %2, 6;\n\t"
#define QLIN_CHUNK_TAIL                                                                        \
  "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%4];\n\t"        \
  "}" ::"r"(d_tmem),                                                                           \
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(smem_u32(tfull_bar))                             \
      : "memory"
#define QLIN_M(KIND, A, B, P) "@pe tcgen05.mma.cta_group::1.kind::" KIND " [%0], " A ", " B ", %3, " P ";\n\t"
#define QLIN_CHUNK(KIND)                                                                                         \
  if (NMMA == 1) {                                                                                               \
    asm volatile(QLIN_CHUNK_HEAD QLIN_M(KIND, "%1", "%2", "pf") QLIN_CHUNK_TAIL);                                \
  } else if (NMMA == 2) {                                                                                        \
    asm volatile(QLIN_CHUNK_HEAD QLIN_M(KIND, "%1", "%2", "pf") QLIN_M(KIND, "a1", "b1", "pt") QLIN_CHUNK_TAIL); \
  } else {                                                                                                       \
    asm volatile(QLIN_CHUNK_HEAD QLIN_M(KIND, "%1", "%2", "pf") QLIN_M(KIND, "a1", "b1", "pt")                   \
                     QLIN_M(KIND, "a2", "b2", "pt") QLIN_M(KIND, "a3", "b3", "pt") QLIN_CHUNK_TAIL);             \
  }
  if (KIND_F8) {
    QLIN_CHUNK("f8f6f4")
  } else {
    QLIN_CHUNK("i8")
  }
#undef QLIN_CHUNK
#undef QLIN_M
#undef QLIN_CHUNK_TAIL
#undef QLIN_CHUNK_HEAD
}

// One accumulation chunk of NMMA (1, 2 or 4) K=32-byte int8 MMAs issued twice: into a running total accumulator
// (`accumulate_total` = 0 makes the first MMA overwrite it) and into a fresh per-chunk accumulator, then the
// "accumulator full" commit on `tfull_bar` (it covers both).
template <int NMMA>
__device__ __forceinline__ void tc_mma_chunk_and_total_i8(uint32_t d_chunk, uint32_t d_total, uint64_t adesc, uint64_t bdesc,
                                                          uint32_t idesc, uint32_t accumulate_total, uint64_t* tfull_bar) {
#define QLIN_CT_HEAD                                      \
  "{\n\t"                                                 \
  ".reg .pred pe, pf, pt, pa;\n\t"                        \
  ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"                 \
  "elect.sync _|pe, 0xffffffff;\n\t"                      \
  "setp.ne.b32 pt, %3, 0;\n\t"                            \
  "setp.eq.b32 pf, %3, 0;\n\t"                            \
  "setp.ne.b32 pa, %6, 0;\n\t"                            \
  "add.s64 a1, %1, 2;\n\t"                                \
  "add.s64 b1, %2, 2;\n\t"                                \
  "add.s64 a2, %1, 4;\n\t"                                \
  "add.s64 b2, %2, 4;\n\t"                                \
  "add.s64 a3, %1, 6;\n\t"                                \
  "add.s64 b3, %2, 6;\n\t"
#define QLIN_CT_TAIL                                                                           \
  "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%4];\n\t"        \
  "}" ::"r"(d_chunk),                                                                          \
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(smem_u32(tfull_bar)), "r"(d_total), "r"(accumulate_total) \
      : "memory"
#define QLIN_MC(A, B, P) "@pe tcgen05.mma.cta_group::1.kind::i8 [%0], " A ", " B ", %3, " P ";\n\t"
#define QLIN_MT(A, B, P) "@pe tcgen05.mma.cta_group::1.kind::i8 [%5], " A ", " B ", %3, " P ";\n\t"
  if (NMMA == 1) {
    asm volatile(QLIN_CT_HEAD QLIN_MT("%1", "%2", "pa") QLIN_MC("%1", "%2", "pf") QLIN_CT_TAIL);
  } else if (NMMA == 2) {
    asm volatile(QLIN_CT_HEAD QLIN_MT("%1", "%2", "pa") QLIN_MC("%1", "%2", "pf") QLIN_MT("a1", "b1", "pt") QLIN_MC("a1", "b1", "pt") QLIN_CT_TAIL);
  } else {
    asm volatile(QLIN_CT_HEAD QLIN_MT("%1", "%2", "pa") QLIN_MC("%1", "%2", "pf") QLIN_MT("a1", "b1", "pt") QLIN_MC("a1", "b1", "pt")
                     QLIN_MT("a2", "b2", "pt") QLIN_MC("a2", "b2", "pt") QLIN_MT("a3", "b3", "pt") QLIN_MC("a3", "b3", "pt") QLIN_CT_TAIL);
  }
#undef QLIN_MT
#undef QLIN_MC
#undef QLIN_CT_TAIL
#undef QLIN_CT_HEAD
}

// A single K=32-byte MMA, elected-lane form.
template <int KIND_F8>
__device__ __forceinline__ void tc_mma1(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
#define QLIN_MMA1(KIND)                                                               \
  asm volatile(                                                                       \
      "{\n\t"                                                                         \
      ".reg .pred pe, pa;\n\t"                                                        \
      "elect.sync _|pe, 0xffffffff;\n\t"                                              \
      "setp.ne.b32 pa, %4, 0;\n\t"                                                    \
      "@pe tcgen05.mma.cta_group::1.kind::" KIND " [%0], %1, %2, %3, pa;\n\t"         \
      "}" ::"r"(d_tmem),                                                              \
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)                             \
      : "memory")
  if (KIND_F8) {
    QLIN_MMA1("f8f6f4");
  } else {
    QLIN_MMA1("i8");
  }
#undef QLIN_MMA1
}

// tcgen05.commit, elected-lane form.
__device__ __forceinline__ void tc_commit_elect(uint64_t* bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred pe;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}" ::"r"(smem_u32(bar))
      : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster of two share one MMA: the even CTA (the leader) issues tcgen05.mma for a
// 256-row tile, each CTA holds its 128 rows of A, its half of B's rows and its 128 accumulator rows.
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive_wait() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (an address in this CTA's shared memory) as seen in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
  return a;
}
// 32-bit load from a shared::cluster address (another CTA's shared memory, or this one's).
__device__ __forceinline__ uint32_t ld_cluster_u32(uint32_t cluster_addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
  return v;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// One stage of a CTA pair: both CTAs load their own two boxes into their own shared memory; the
// bytes are counted on the leader's barrier (`leader_bar`, a shared::cluster address), on which only
// the leader posts the expected total.  No multicast: each CTA fetches what it needs itself.
__device__ __forceinline__ void tma_issue_stage_pair(uint32_t leader_bar, bool is_leader, uint32_t total_bytes, void* dst_a,
                                                     const void* tmap_a, int32_t ya, void* dst_b, const void* tmap_b,
                                                     int32_t yb, int32_t x) {
  asm volatile(
      "{\n\t"
      ".reg .pred pe, pl;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.ne.b32 pl, %9, 0;\n\t"
      "and.pred pl, pl, pe;\n\t"
      "@pl mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;\n\t"
      "@pe cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%2], [%3, {%4, %5}], [%0];\n\t"
      "@pe cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%6], [%7, {%4, %8}], [%0];\n\t"
      "}" ::"r"(leader_bar),
      "r"(total_bytes), "r"(smem_u32(dst_a)), "l"(reinterpret_cast<uint64_t>(tmap_a)), "r"(x), "r"(ya), "r"(smem_u32(dst_b)),
      "l"(reinterpret_cast<uint64_t>(tmap_b)), "r"(yb), "r"(is_leader ? 1u : 0u)
      : "memory");
}
// Leader only.  Four K=32-byte MMAs of the pair into one accumulator, then the stage is released in
// both CTAs (commit with a two-CTA mask on the barrier at this offset in each of them).
template <int KIND_F8>
__device__ __forceinline__ void tc_mma4_release_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                     uint32_t accumulate, uint64_t* empty_bar) {
#define QLIN_MMA4P(KIND)                                                                                              \
  asm volatile(                                                                                                       \
      "{\n\t"                                                                                                         \
      ".reg .pred pe, pa, pt;\n\t"                                                                                    \
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"                                                                         \
      ".reg .b16 mask;\n\t"                                                                                           \
      "elect.sync _|pe, 0xffffffff;\n\t"                                                                              \
      "setp.ne.b32 pa, %4, 0;\n\t"                                                                                    \
      "setp.ne.b32 pt, %3, 0;\n\t"                                                                                    \
      "mov.b16 mask, 3;\n\t"                                                                                          \
      "add.s64 a1, %1, 2;\n\t"                                                                                        \
      "add.s64 b1, %2, 2;\n\t"                                                                                        \
      "add.s64 a2, %1, 4;\n\t"                                                                                        \
      "add.s64 b2, %2, 4;\n\t"                                                                                        \
      "add.s64 a3, %1, 6;\n\t"                                                                                        \
      "add.s64 b3, %2, 6;\n\t"                                                                                        \
      "@pe tcgen05.mma.cta_group::2.kind::" KIND " [%0], %1, %2, %3, pa;\n\t"                                         \
      "@pe tcgen05.mma.cta_group::2.kind::" KIND " [%0], a1, b1, %3, pt;\n\t"                                         \
      "@pe tcgen05.mma.cta_group::2.kind::" KIND " [%0], a2, b2, %3, pt;\n\t"                                         \
      "@pe tcgen05.mma.cta_group::2.kind::" KIND " [%0], a3, b3, %3, pt;\n\t"                                         \
      "@pe tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%5], mask;\n\t"  \
      "}" ::"r"(d_tmem),                                                                                              \
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(smem_u32(empty_bar))                                   \
      : "memory")
  if (KIND_F8) {
    QLIN_MMA4P("f8f6f4");
  } else {
    QLIN_MMA4P("i8");
  }
#undef QLIN_MMA4P
}
// Leader only.  One K=32-byte MMA of the pair (ragged K tail).
template <int KIND_F8>
__device__ __forceinline__ void tc_mma1_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
#define QLIN_MMA1P(KIND)                                                       \
  asm volatile(                                                                \
      "{\n\t"                                                                  \
      ".reg .pred pe, pa;\n\t"                                                 \
      "elect.sync _|pe, 0xffffffff;\n\t"                                       \
      "setp.ne.b32 pa, %4, 0;\n\t"                                             \
      "@pe tcgen05.mma.cta_group::2.kind::" KIND " [%0], %1, %2, %3, pa;\n\t"  \
      "}" ::"r"(d_tmem),                                                       \
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)                      \
      : "memory")
  if (KIND_F8) {
    QLIN_MMA1P("f8f6f4");
  } else {
    QLIN_MMA1P("i8");
  }
#undef QLIN_MMA1P
}
// Leader only.  Arrive on the barrier at this offset in both CTAs once the pair's MMAs so far are done.
__device__ __forceinline__ void tc_commit_pair_elect(uint64_t* bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred pe;\n\t"
      ".reg .b16 mask;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "mov.b16 mask, 3;\n\t"
      "@pe tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], mask;\n\t"
      "}" ::"r"(smem_u32(bar))
      : "memory");
}

// Reads 32 consecutive 32-bit columns of this warp's 32 TMEM lanes (lane i of the warp gets TMEM
// lane base+i) and waits for the data; the registers are valid when the call returns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// The low 16 bits of 32 consecutive 32-bit columns, two columns per register (column 2i in the low half of r[i],
// column 2i + 1 in the high half): half the register traffic of tmem_ld32 for callers that only need the low bits.
__device__ __forceinline__ void tmem_ld32_low16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.pack::16b.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Two back-to-back 32-column reads (64 columns) with a single wait.
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
        "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
        "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
        "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
        "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
}

}  // namespace qlin
