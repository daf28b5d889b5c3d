// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (bulk tensor and flat bulk copies, never multicast),
// tcgen05 (TMEM allocation, block-scaled FP4 MMA, scale-factor copy, accumulator loads) and programmatic
// dependent launch. Every wait is bounded: a wait that runs out records a code in a status word and lets the
// kernel unwind instead of spinning forever.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace q27b {

// Status codes a kernel may leave in its status word (0 = fine).
enum : uint32_t {
  kStatusOk = 0,
  kStatusFullWaitTimeout = 1,    // consumer never saw a TMA stage arrive
  kStatusEmptyWaitTimeout = 2,   // producer never saw a stage released
  kStatusAccumWaitTimeout = 3,   // epilogue never saw the MMAs of a tile complete
  kStatusAccumFreeTimeout = 4,   // MMA issuer never saw an accumulator buffer drained
  kStatusDrainTimeout = 5,       // a copy in flight did not land during unwinding
  kStatusProbeTimeout = 6,       // the self-test's wait on a barrier nothing arrives at ran out, as it must
  kStatusTileWaitTimeout = 7,    // grouped launch: the pieces of a cut tile never all arrived
  kStatusPeerWaitTimeout = 8,    // fused gather: a peer GPU never reported its block of the outputs
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------------------------------------ mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  // makes the initialised barriers visible to the async proxy (TMA, tcgen05.commit)
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
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// The same with cluster scope: the arrivals may come from the partner CTA of a pair.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Budget of a bounded wait in SM clock cycles (about two seconds at 2 GHz) and in polls (each poll may itself
// block for a hardware-defined slice of time; the cycle budget is what normally ends a wait that cannot succeed).
constexpr long long kMaxWaitCycles = 4000000000ll;
constexpr uint32_t kMaxPolls = 1u << 28;

// Waits for the phase with the given parity; gives up when `abort_flag` (shared memory) is raised by another
// role or when the budget is spent, in which case it raises the flag itself and records `code`.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                  uint32_t* status, uint32_t code, uint32_t sleep_ns = 0,
                                                  bool cluster = false, long long max_cycles = kMaxWaitCycles) {
  if (cluster ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 1; i < kMaxPolls; i++) {
    if (sleep_ns) __nanosleep(sleep_ns);  // long waits back off: polls go through the shared-memory pipe
    if (cluster ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > max_cycles) break;
    }
  }
  *abort_flag = 1u;
  if (status) atomicCAS(status, 0u, code);
  return false;
}

// The same for a whole (converged) warp: one lane polls, then every lane observes the completed phase itself.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* status, uint32_t code, uint32_t sleep_ns) {
  uint32_t ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait_bounded(bar, parity, abort_flag, status, code, sleep_ns);
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (ok) ok = mbar_wait_bounded(bar, parity, abort_flag, status, code);
  return __all_sync(0xffffffffu, ok) != 0;
}

// ------------------------------------------------------------------------------------------------ TMA

constexpr uint64_t kEvictNormal = 0x1000000000000000ull;
constexpr uint64_t kEvictFirst = 0x12F0000000000000ull;
constexpr uint64_t kEvictLast = 0x14F0000000000000ull;

// 2-D tiled load: box starting at element (x = innermost coordinate, y = row) into shared memory.
// x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const void* tmap, int x, int y, uint32_t bar,
                                            uint64_t hint) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_dst), "l"(tmap), "r"(bar), "r"(x), "r"(y), "l"(hint)
      : "memory");
}
// Flat copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar,
                                          uint64_t hint) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar), "l"(hint)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------------------------------------ PDL

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ tcgen05

__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {  // whole warp
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are 128 bytes apart and stored with the
// 128-byte TMA swizzle (tile base 1024-byte aligned): groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= uint64_t(1) << 16;                      // leading byte offset (unused for swizzled K-major)
  d |= uint64_t(1024 >> 4) << 32;              // stride byte offset: 8 rows x 128 B
  d |= uint64_t(1) << 46;                      // descriptor version of this architecture
  d |= uint64_t(2) << 61;                      // layout: 128-byte swizzle
  return d;
}
// Descriptor of a 512-byte scale-factor atom (32 lines of 16 bytes, no swizzle) for tcgen05.cp 32x128b.
__device__ __forceinline__ uint64_t umma_desc_sf_atom(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFFu) >> 4);
  d |= uint64_t(128 >> 4) << 32;  // 8 lines x 16 B between line groups
  d |= uint64_t(1) << 46;
  return d;
}

// Instruction descriptor of kind::mxf4nvf4 (E2M1 x E2M1, UE4M3 scales per 16, fp32 accumulate), both operands
// K-major, MMA shape 128 x n x 64.
__host__ __device__ constexpr uint32_t umma_idesc_nvfp4(uint32_t n) {
  return (1u << 7)          // A format E2M1
         | (1u << 10)       // B format E2M1
         | ((n >> 3) << 17) // N / 8
         | (0u << 23)       // scale format UE4M3
         | ((128u >> 4) << 24);  // M / 16
}

// D[tmem] (+)= A[smem] . B[smem]^T with per-16 scales read from tensor memory. One thread issues.
__device__ __forceinline__ void umma_nvfp4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// Arrives on the barrier once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// One 512-byte scale atom -> 4 tensor-memory columns (lanes 0..31, replicated to the four lane quarters).
__device__ __forceinline__ void tmem_cp_sf_atom(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// 32 lanes x 8 / 16 consecutive fp32 columns: thread t of the warp receives lane (base lane + t).
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float* v) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 lanes x 16 consecutive 32-bit columns from registers: thread t of the warp writes lane (base lane + t);
// v = four 16-byte vectors, in column order.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint4 (&v)[4]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0].x), "r"(v[0].y), "r"(v[0].z), "r"(v[0].w), "r"(v[1].x), "r"(v[1].y), "r"(v[1].z),
        "r"(v[1].w), "r"(v[2].x), "r"(v[2].y), "r"(v[2].z), "r"(v[2].w), "r"(v[3].x), "r"(v[3].y), "r"(v[3].z),
        "r"(v[3].w)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }


// ------------------------------------------------------------------------------------------------ CTA pairs
// (clusters of two CTAs on neighbouring SMs driving one tcgen05.mma.cta_group::2; no multicast loads anywhere)

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Every thread of both CTAs arrives and waits: used once at start-up and once before exit, unconditionally.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t rank) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}"
      ::"r"(bar), "r"(rank)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_2sm(uint32_t smem_result, uint32_t ncols) {  // one warp in each CTA
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2sm() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2sm(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Instruction descriptor for the pair: 256 x n x 64 (each CTA holds 128 of the 256 rows).
__host__ __device__ constexpr uint32_t umma_idesc_nvfp4_2sm(uint32_t n) {
  return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}
// Issued by the leader CTA only; runs on both SMs. A: each CTA's own 128 rows, B: each CTA holds n / 2 rows.
__device__ __forceinline__ void umma_nvfp4_2sm(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// The same with the accumulate flag fixed at compile time (no predicate to evaluate between two MMAs).
template <bool kAccumulate>
__device__ __forceinline__ void umma_nvfp4_2sm_imm(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                   uint32_t sfa_tmem, uint32_t sfb_tmem) {
  if constexpr (kAccumulate)
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}
// One 512-byte scale atom of EACH CTA of the pair (same shared-memory offset) -> 4 columns of that CTA's own tensor memory
// (lanes 0..31, replicated to the four lane quarters). Issued by one thread of the leader CTA. (Measured: the partner's
// tensor memory receives the partner's own shared memory, not the leader's.)
__device__ __forceinline__ void tmem_cp_sf_atom_2sm(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// Arrives on the issuing CTA's barrier once this thread's tcgen05 operations so far have completed in both CTAs.
__device__ __forceinline__ void umma_commit_2sm_local(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Arrives on the barrier at this offset in both CTAs once the leader's tcgen05 operations so far have completed.
__device__ __forceinline__ void umma_commit_2sm(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(uint16_t(3))
      : "memory");
}

}  // namespace q27b
