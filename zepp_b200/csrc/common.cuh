// Shared device helpers: status words, bounded waits, PTX wrappers for sm_100a
// (mbarrier, TMA, tcgen05/TMEM).  Everything here is header-only and internal.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace zepp {

// ---------------------------------------------------------------------------------------
// Status block (one per layer, device memory, read by the host after a step).
// Every wait in every kernel is bounded; a wait that gives up records what it waited
// for here and the kernel returns, so the CUDA context stays usable.
// ---------------------------------------------------------------------------------------
enum StatusWord : int {
  ST_ERROR = 0,        // OR of ErrorBit
  ST_WAIT_WHAT = 1,    // which wait gave up (WaitId)
  ST_WAIT_PEER = 2,    // peer / item index of the wait that gave up
  ST_WAIT_EPOCH = 3,   // epoch it waited for
  ST_VIOLATION = 4,    // capacity violation mask of the step (demands kernel)
  // device timeline of the last step (globaltimer ns), written by block 0 / the last block of each kernel
  TR_ROUTE = 8, TR_PASS1 = 9, TR_PASS1_GO = 10, TR_PASS2 = 11, TR_GEMM1 = 12, TR_GEMM1_X = 13, TR_GEMM1_END = 14,
  TR_GEMM2 = 15, TR_GEMM2_END = 16, TR_REDUCE = 17, TR_REDUCE_GO = 18, TR_REDUCE_END = 19,
  // inside the scan block of the first metadata kernel
  TR_SCAN = 20, TR_SCAN_COUNTS = 21, TR_SCAN_BASES = 22, TR_SCAN_DEMANDS = 23, TR_SCAN_SCHED = 24, TR_SCAN_END = 25,
  // cycle sums of a -DZEPP_GEMM_PROFILE build (not time stamps): MMA thread waiting for operand stages / for a free
  // accumulator, epilogue warp working / waiting
  TR_PROF_MMA_DATA = 26, TR_PROF_MMA_ACC = 27, TR_PROF_EPI_BUSY = 28, TR_PROF_EPI_WAIT = 29,
  // the same four words in a normal build: stamps of the swap kernels that run before the routing
  TR_LOADS = 26, TR_DECIDE = 27, TR_DECIDE_GO = 28, TR_DECIDE_END = 29,
  TR_GATHER_END = 30,  // dispatch GEMM: the last gather warp finished (max over warps)
  TR_FIRST_ITEMS = 31, // dispatch GEMM: latest start of a CTA's first item (max over CTAs)
  TR_RING = 32,        // start stamps of the last 16 steps (slot = epoch % 16), then their end stamps
  ST_WORDS = 64
};
enum ErrorBit : unsigned long long {
  ERR_TIMEOUT = 1ull,        // a bounded wait ran out
  ERR_CAPACITY = 2ull,       // the step's demands exceed the buffers; GEMMs skipped
  ERR_BAD_INDEX = 4ull,      // an index table entry was out of range (clamped, skipped)
  ERR_ROUTE = 8ull           // router: stranded demand / ordinal beyond the tables
};
enum WaitId : int {
  WAIT_LOADS = 1, WAIT_ROUTING = 2, WAIT_X = 3, WAIT_COMBINE = 4, WAIT_MBAR_FULL = 5,
  WAIT_MBAR_EMPTY = 6, WAIT_TMEM_FULL = 7, WAIT_TMEM_EMPTY = 8, WAIT_TILE_READY = 9,
  WAIT_BARRIER = 10, WAIT_TEST = 11, WAIT_WEIGHTS = 12
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void trace_mark(unsigned long long* status, int slot) {
  if (status != nullptr) status[slot] = globaltimer_ns();
}
// Stamps inside a kernel's serial sections (each costs the stamping thread a globaltimer read that the block then
// waits for at its next barrier): compiled in only with -DZEPP_FINE_TRACE.
#ifdef ZEPP_FINE_TRACE
#define ZEPP_FINE_MARK(status, slot) trace_mark(status, slot)
#else
#define ZEPP_FINE_MARK(status, slot) ((void)0)
#endif
__device__ __forceinline__ void trace_mark_max(unsigned long long* status, int slot) {
  if (status != nullptr) atomicMax(status + slot, globaltimer_ns());
}

__device__ __forceinline__ void record_timeout(unsigned long long* status, int what, long long peer,
                                               long long epoch) {
  if (status == nullptr) return;
  unsigned long long old = atomicOr(status + ST_ERROR, (unsigned long long)ERR_TIMEOUT);
  if ((old & ERR_TIMEOUT) == 0) {
    status[ST_WAIT_WHAT] = (unsigned long long)what;
    status[ST_WAIT_PEER] = (unsigned long long)peer;
    status[ST_WAIT_EPOCH] = (unsigned long long)epoch;
  }
}

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// epoch word store after the caller's own system-scope fence (one fence, then one store per peer)
__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded acquire-spin on a monotone epoch word written by another GPU (or another kernel
// that already ran).  Returns true when *flag >= epoch, false when `limit_ns` ran out.
__device__ __forceinline__ bool wait_epoch_geq(const unsigned long long* flag, unsigned long long epoch,
                                               unsigned long long limit_ns) {
  if (ld_acquire_sys(flag) >= epoch) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned int backoff = 32;
  while (true) {
    if (ld_acquire_sys(flag) >= epoch) return true;
    if (globaltimer_ns() - t0 > limit_ns) return false;
    __nanosleep(backoff);
    if (backoff < 1024) backoff <<= 1;
  }
}

// ---------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
// Bounded wait: gives up `limit_ns` of wall time after its first failed poll burst, or as soon as the
// CTA-wide abort flag is raised by another role.  The clock is read once per 64 polls.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                  unsigned long long limit_ns) {
  for (int it = 0; it < 64; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  while (true) {
    for (int it = 0; it < 64; ++it)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > limit_ns) return false;
  }
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// one 32-byte store (a whole sector): sm_100 has 256-bit global stores; the address is 32-byte aligned
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t (&w)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]),
               "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

// ---------------------------------------------------------------------------------------
// TMA (tiled 2D loads, each into the issuing CTA's own shared memory only)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------------------------------
// tcgen05 / TMEM
// ---------------------------------------------------------------------------------------
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
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 x bf16 -> fp32, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// mbarrier arrives once every tcgen05 op issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread (thread i <-> lane base+i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major bf16 tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA box of 64 bf16 columns with CU_TENSOR_MAP_SWIZZLE_128B
// writes): 8-row groups are 1024 bytes apart.  Tile bases are 1024-byte aligned; a K step of
// 16 elements advances the start address by 32 bytes inside the swizzle atom.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                         // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                         // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                         // layout type: 128-byte swizzle
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M = 128 (one CTA) or 256 (a CTA pair),
// N multiple of 16.
__device__ __forceinline__ uint32_t make_idesc_bf16(uint32_t m, uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ uint32_t make_idesc_bf16_m128(uint32_t n) { return make_idesc_bf16(128u, n); }

// ---------------------------------------------------------------------------------------
// CTA pairs (cluster of two CTAs on neighbouring SMs driving one tcgen05.mma.cta_group::2).
// Shared-memory addresses below are 32-bit shared::cluster window addresses; a CTA's own
// shared::cta address is valid there and names the CTA itself.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// address of the same shared-memory object in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// every thread of both CTAs (a hardware barrier: reached on every path, aborted ones included)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t bar_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.relaxed.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(bar_addr), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// Tiled 2D load into this CTA's shared memory whose completion bytes are credited to an mbarrier of the pair's
// leader CTA (no multicast: each CTA of the pair loads its own half of the operands).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t leader_bar_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(leader_bar_addr), "r"(c0), "r"(c1)
      : "memory");
}
// TMEM of both CTAs of a pair: one warp of EACH CTA allocates / frees (the columns are the same in both)
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A * B over the pair: each CTA holds its 128 rows of A and its half of B's rows at the
// same shared-memory offsets; issued by one thread of the leader CTA.
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the mbarrier at this offset in BOTH CTAs of the pair arrives once every tcgen05 op issued so far has completed
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(both)
               : "memory");
}

}  // namespace zepp
