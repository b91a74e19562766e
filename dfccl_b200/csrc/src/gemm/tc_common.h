// sm_100a building blocks for the tensor-core kernels of this library, as inline PTX:
// mbarriers, TMA tile loads (never with cluster multicast), tcgen05 tensor-memory allocation,
// UMMA descriptors, tcgen05.mma / commit / ld.  Every wait is bounded: a wait that runs out
// returns false and the caller leaves through its clean-up path (drain its own copies, free
// tensor memory, set an error word) instead of hanging the GPU.
//
// The reference has no tensor-core code (it is a collective library); these kernels exist for
// the fused compute + collective operators of the tensor-parallel workloads.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dfccl {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
// Bounded wait: false when the time limit ran out or another role already gave up.  The limit is
// generous because a role may legitimately wait as long as the slowest peer GPU is late; the waits on
// peers carry the caller's own (shorter) limit and raise giveUp first.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* giveUp, uint64_t limitNs = 120000000000ull) {
  uint64_t t0 = 0;
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023) == 1023) {
      if (*giveUp) return false;
      uint64_t t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (t0 == 0) t0 = t;
      else if (t - t0 > limitNs) break;
    }
  }
  *giveUp = 1;
  return false;
}

// ---- TMA: 2-D tile load global -> shared, completion on an mbarrier.  x is the innermost
// coordinate in elements and must keep x * sizeof(element) a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smemDst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smemDst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t* smemResult, uint32_t ncols) {      // one full warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smemResult)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {          // the same warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- UMMA descriptors
// Shared-memory operand, K-major, 128-byte swizzle: rows of 64 bf16 (128 bytes), groups of 8 rows
// 1024 bytes apart, the layout a TMA tile load with CU_TENSOR_MAP_SWIZZLE_128B produces.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(const void* smem) {
  const uint64_t addr = (uint64_t)(smem_u32(smem) & 0x3FFFFu) >> 4;
  return addr                               // start address              bits [0,14)
         | ((uint64_t)1 << 16)              // leading byte offset (unused with this swizzle)   bits [16,30)
         | ((uint64_t)(1024 >> 4) << 32)    // stride byte offset: 8 rows x 128 bytes           bits [32,46)
         | ((uint64_t)1 << 46)              // descriptor version of sm_100                    bits [46,48)
         | ((uint64_t)2 << 61);             // layout: 128-byte swizzle                        bits [61,64)
}
// Shared-memory operand, MN-major (the contraction index is the slow one: the operand is stored transposed),
// 128-byte swizzle.  The tile is a row of blocks of 64 MN-elements; a block is [K rows] x 128 bytes, exactly what a
// TMA tile load of 64 columns x K rows with CU_TENSOR_MAP_SWIZZLE_128B produces.  Groups of 8 K-rows are 1024 bytes
// apart (stride byte offset), the blocks `blockBytes` apart (leading byte offset).
__device__ __forceinline__ uint64_t umma_smem_desc_mn_sw128(const void* smem, uint32_t blockBytes) {
  const uint64_t addr = (uint64_t)(smem_u32(smem) & 0x3FFFFu) >> 4;
  return addr
         | ((uint64_t)(blockBytes >> 4) << 16)   // leading byte offset: next block of 64 MN-elements
         | ((uint64_t)(1024 >> 4) << 32)         // stride byte offset: next group of 8 K-rows
         | ((uint64_t)1 << 46)
         | ((uint64_t)2 << 61);
}
// Instruction descriptor: bf16 x bf16 -> fp32, dense; each operand K-major (0) or MN-major (1).
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n, int aMnMajor = 0, int bMnMajor = 0) {
  return (1u << 4)                          // accumulator format: fp32
         | (1u << 7) | (1u << 10)           // A and B format: bf16
         | ((uint32_t)(aMnMajor & 1) << 15) | ((uint32_t)(bMnMajor & 1) << 16)
         | ((uint32_t)(n >> 3) << 17)       // N / 8
         | ((uint32_t)(m >> 4) << 24);      // M / 16
}

// D[tmem] (+)= A[smem] x B[smem]^T, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier when all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster work on one tile.  Each holds half of the rows of A and half
// of the rows of B in its own shared memory and half of the accumulator rows in its own tensor memory; one thread
// of the leader (cluster rank 0) issues the MMAs for both.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {          // every thread of every CTA of the cluster
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t mapa_u32(uint32_t smemAddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smemAddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t clusterAddr) {     // arrive on a barrier of another CTA of the cluster
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
// TMA tile load into THIS CTA's shared memory whose completion is counted on a barrier that may live in the peer CTA
// of the pair (no cluster multicast: the tile goes to one CTA).
__device__ __forceinline__ void tma_load_2d_pair(void* smemDst, const CUtensorMap* map, int x, int y, uint32_t barClusterAddr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smemDst)), "l"(map), "r"(barClusterAddr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smemResult, uint32_t ncols) {       // one full warp in EACH CTA of the pair
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smemResult)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in both CTAs of the pair when the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

// 32 consecutive fp32 columns of this thread's lane (row) of tensor memory.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Tile visiting order of a persistent GEMM: groups of `groupM` row tiles, row index fastest inside a group.  The
// CTAs that work at the same time then share a block of about groupM row tiles x (CTAs / groupM) column tiles, whose
// operands fit in L2, instead of a couple of row tiles times EVERY column tile (all of B per wave).
__device__ __forceinline__ void raster_tile(int t, int mTiles, int nTiles, int groupM, int& mt, int& nt) {
  const int perGroup = groupM * nTiles;
  const int grp = t / perGroup, first = grp * groupM;
  const int gsz = min(groupM, mTiles - first);
  const int r = t - grp * perGroup;
  mt = first + r % gsz;
  nt = r / gsz;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

}  // namespace tc
}  // namespace dfccl
