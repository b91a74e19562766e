// bf16 GEMM on the 5th-generation tensor cores, hand-written for sm_100a:
//     C[M,N] = A[M,K] * B[N,K]^T        (both operands K-major: y = x W^T of a linear layer)
// and its two communication-fused forms for tensor parallelism over NVLink peer memory:
//   * all-gather -> GEMM : A is row-sharded over the ranks.  Extra warps of the SAME kernel pull
//     the peers' row blocks into the local A buffer (plain peer loads) and publish one flag per
//     128-row block; the TMA producer waits for the flag of the block it is about to load, so the
//     transfer of block i+1.. overlaps the tensor-core work on block i.
//   * GEMM -> reduce-scatter : C is a partial sum whose row blocks belong to different ranks.  The
//     epilogue stores each finished tile straight into its owner's receive slot (peer stores) and
//     publishes a per-tile flag there; the owner sums the n slots of a tile as soon as all have
//     arrived, in the same kernel, while other CTAs are still on the tensor cores.
// Structure of a CTA (persistent, one per SM): warp 0 = TMA producer (one elected thread), warp 1 =
// tensor-memory owner and MMA issuer (one elected thread, tcgen05.mma, 128 x 256 x 16 per
// instruction), warps 2-5 = epilogue (tcgen05.ld from a double-buffered 2 x 256-column accumulator),
// warps 6-9 = communication.  4 shared-memory stages of 48 KB (A 128x64, B 256x64, 128-byte swizzle)
// filled by TMA (no cluster multicast anywhere), full/empty mbarriers, tcgen05.commit to release
// stages and to hand accumulators over.  Every wait is bounded and ends in an error word.
#include "tc_common.h"
#include "gemm.h"
#include "../common/param.h"
#include "dfccl.h"
#include "../common/log.h"
#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>
#include <tuple>

namespace dfccl {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int MN_BLOCK_BYTES = 64 * BK * 2;          // MN-major operand: one block of 64 MN-columns x BK K-rows
static_assert(BM == GEMM_BM && BN == GEMM_BN && BK == GEMM_BK, "tile constants of gemm.h");
constexpr int TMEM_COLS = 512;                       // two accumulators of BN fp32 columns
constexpr int NUM_THREADS = 320;                     // 10 warps
constexpr int GATHER_PIECES = 8;                     // pieces a 128-row block is pulled in (all-gather -> GEMM)
constexpr int EPI_ROW_BYTES = 64 * 2 + 16;            // one staged row: 64 bf16 columns + 16 bytes so that rows start in different banks
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_BYTES;   // 32 rows per epilogue warp
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 4 * EPI_WARP_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct GemmArgs {
  __nv_bfloat16* C;
  int M, N, K, ldc;
  int groupM;                       // plain GEMM: row tiles per rasterisation group (0 = row-major tile order, the fused forms)
  int aMn, bMn;                     // operand stored with the contraction index slow: A as [K, M], B as [K, N] (row-major)
  uint32_t* err;                    // device word: non-zero = a bounded wait ran out (later launches return at once)
  uint64_t waitNs;                  // limit of every wait on a word another GPU or CTA writes
  uint32_t* errHost;                // the same verdict in pinned host memory, read by the host without a synchronisation
  FusedArgs f;
};

__device__ __forceinline__ uint64_t ld_acq_sys(const volatile uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acq_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acq_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_rel_sys(volatile uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_rel_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_rel_gpu_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_peer16(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Bounded spin on a 64-bit flag in local memory written by a peer.
// Waits on words that another GPU (or another CTA) writes are bounded by time, not by polls: a peer may
// legitimately be seconds late (its host was slow to launch), but never forever.
__device__ __forceinline__ uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool wait_flag64(const volatile uint64_t* p, uint64_t want, volatile uint32_t* giveUp, uint64_t limitNs) {
  const uint64_t t0 = now_ns();
  for (uint32_t i = 0;; ++i) {
    if (ld_acq_sys(p) >= want) return true;
    if ((i & 255) == 255) {
      if (*giveUp) return false;
      if (now_ns() - t0 > limitNs) break;
    }
  }
  *giveUp = 1;
  return false;
}
__device__ __forceinline__ bool wait_flag32(const uint32_t* p, uint32_t want, volatile uint32_t* giveUp, bool sys, uint64_t limitNs) {
  const uint64_t t0 = now_ns();
  for (uint32_t i = 0;; ++i) {
    if ((sys ? ld_acq_sys_u32(p) : ld_acq_gpu_u32(p)) >= want) return true;
    if ((i & 255) == 255) {
      if (*giveUp) return false;
      if (now_ns() - t0 > limitNs) break;
    }
  }
  *giveUp = 1;
  return false;
}

// m-tile visiting order: own row blocks first, then the peers' in ring order, so that the
// tensor cores start on data that is already here while the rest is in flight.
__device__ __forceinline__ int orderedMTile(const FusedArgs& f, int i, int mTiles) {
  if (f.nranks <= 1 || f.mode == 0) return i;
  const int per = mTiles / f.nranks;
  const int owner = (f.rank + (f.mode == 2 ? 1 : 0) + i / per) % f.nranks;   // reduce-scatter: other ranks' rows first, mine last
  return owner * per + i % per;
}

__device__ __forceinline__ void tileCoord(const GemmArgs& g, int t, int mTiles, int nTiles, int& mt, int& nt) {
  if (g.groupM > 0) { raster_tile(t, mTiles, nTiles, g.groupM, mt, nt); return; }
  mt = orderedMTile(g.f, t / nTiles, mTiles);
  nt = t % nTiles;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
dfcclGemmKernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const GemmArgs g) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
  uint8_t* epiSmem = smem + STAGES * STAGE_BYTES;
  uint64_t* fullBar = (uint64_t*)(epiSmem + 4 * EPI_WARP_BYTES);
  uint64_t* emptyBar = fullBar + STAGES;
  uint64_t* accFull = emptyBar + STAGES;            // [2]
  uint64_t* accEmpty = accFull + 2;                 // [2]
  uint32_t* tmemBaseSlot = (uint32_t*)(accEmpty + 2);
  volatile uint32_t* giveUp = tmemBaseSlot + 1;
  uint64_t* epochSlot = (uint64_t*)(tmemBaseSlot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mTiles = g.M / BM, nTiles = g.N / BN, kBlocks = g.K / BK;
  const int numTiles = mTiles * nTiles;
  const FusedArgs& f = g.f;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&fullBar[s], 1); mbar_init(&emptyBar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&accFull[a], 1); mbar_init(&accEmpty[a], 4); }
    *giveUp = *(volatile uint32_t*)g.err;          // an earlier launch gave up: its flags and counters are stale, do nothing
    *epochSlot = g.f.epochCounter ? *(volatile uint64_t*)g.f.epochCounter + 1 : g.f.epoch;
    mbar_fence_init();
    tma_prefetch_desc(&mapA);
    tma_prefetch_desc(&mapB);
  }
  if (warp == 1) tmem_alloc(tmemBaseSlot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmemBase = *tmemBaseSlot;
  const bool dead = *giveUp != 0;
  const uint64_t epoch = *epochSlot;
  if (!dead && f.mode == 2 && f.nranks > 1) {
    // the owners must have finished reducing the previous call before this one overwrites their slots
    if (warp == 2 && lane < f.nranks && lane != f.rank) wait_flag64(&f.done[lane], epoch - 1, giveUp, g.waitNs);
    __syncthreads();
  }

  if (dead) {
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
        int mt, nt;
        tileCoord(g, t, mTiles, nTiles, mt, nt);
        if (f.mode == 1 && f.nranks > 1 && mt / (f.rowsPerRank / BM) != f.rank) {
          // this row block comes from a peer: wait until the communication warps have placed it
          ok = wait_flag32(&f.blockReady[mt], (uint32_t)epoch * GATHER_PIECES, giveUp, false, g.waitNs);
          asm volatile("fence.proxy.async.global;" ::: "memory");   // their generic-proxy stores before my async-proxy loads
          if (!ok) break;
        }
        for (int kb = 0; kb < kBlocks; ++kb) {
          if (!mbar_wait(&emptyBar[stage], phase ^ 1, giveUp)) { ok = false; break; }
          mbar_expect_tx(&fullBar[stage], STAGE_BYTES);
          uint8_t* sa = smem + stage * STAGE_BYTES;
          // K-major operand: one box of [tile rows] x 64 K-columns.  MN-major operand: the tile is a row of blocks
          // of 64 MN-columns x 64 K-rows (8 KB each), one box per block.
          if (!g.aMn) tma_load_2d(sa, &mapA, kb * BK, mt * BM, &fullBar[stage]);
          else for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * MN_BLOCK_BYTES, &mapA, mt * BM + 64 * i, kb * BK, &fullBar[stage]);
          if (!g.bMn) tma_load_2d(sa + A_BYTES, &mapB, kb * BK, nt * BN, &fullBar[stage]);
          else for (int i = 0; i < BN / 64; ++i) tma_load_2d(sa + A_BYTES + i * MN_BLOCK_BYTES, &mapB, nt * BN + 64 * i, kb * BK, &fullBar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // let the copies already issued land before the block goes away (bounded)
        for (int i = 0; i < 20000; ++i) __nanosleep(200);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_bf16(BM, BN, g.aMn, g.bMn);
      // one instruction consumes 16 K-elements: 32 bytes along a K-major row (+2 in the 16-byte address field), two
      // groups of 8 K-rows of an MN-major block (2048 bytes, +128)
      const uint32_t stepA = g.aMn ? 128u : 2u, stepB = g.bMn ? 128u : 2u;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x, ++it) {
        const int ab = it & 1;
        if (!mbar_wait(&accEmpty[ab], ((it >> 1) & 1) ^ 1, giveUp)) break;
        tc_fence_after();
        const uint32_t d = tmemBase + ab * BN;
        for (int kb = 0; kb < kBlocks; ++kb) {
          if (!mbar_wait(&fullBar[stage], phase, giveUp)) { ok = false; break; }
          tc_fence_after();
          const uint8_t* pa = smem + stage * STAGE_BYTES;
          const uint64_t da = g.aMn ? umma_smem_desc_mn_sw128(pa, MN_BLOCK_BYTES) : umma_smem_desc_sw128(pa);
          const uint64_t db = g.bMn ? umma_smem_desc_mn_sw128(pa + A_BYTES, MN_BLOCK_BYTES) : umma_smem_desc_sw128(pa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(d, da + stepA * k, db + stepB * k, idesc, (kb | k) != 0);
          umma_commit(&emptyBar[stage]);              // the stage is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&accFull[ab]);            // accumulator complete
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue: TMEM -> bf16 -> global (local or peer)
    const int quarter = warp & 3;                     // the 32 TMEM lanes this warp may read
    int it = 0;
    for (int t = blockIdx.x; t < numTiles; t += gridDim.x, ++it) {
      int mt, nt;
      tileCoord(g, t, mTiles, nTiles, mt, nt);
      const int ab = it & 1;
      if (!mbar_wait(&accFull[ab], (it >> 1) & 1, giveUp)) break;
      tc_fence_after();
      const int row = mt * BM + quarter * 32 + lane;
      __nv_bfloat16* crow;
      int owner = 0, tileInOwner = 0;
      if (f.mode == 2 && f.nranks > 1) {
        owner = row / f.rowsPerRank;
        tileInOwner = ((mt * BM - owner * f.rowsPerRank) / BM) * nTiles + nt;
        crow = f.slot[owner] + (size_t)(row - owner * f.rowsPerRank) * g.N + nt * BN;
      } else {
        crow = g.C + (size_t)row * g.ldc + nt * BN;
      }
      // 64 columns at a time: registers -> this warp's staging rows in shared memory -> global, so that
      // every store instruction writes whole 128-byte row segments (what NVLink and DRAM both want)
      // instead of 32 scattered 16-byte pieces
      uint8_t* stage = epiSmem + (warp - 2) * EPI_WARP_BYTES;
      __nv_bfloat16* cbase = crow - (size_t)lane * (f.mode == 2 && f.nranks > 1 ? g.N : g.ldc);    // row 0 of this warp's 32 rows
      const size_t rowStride = (f.mode == 2 && f.nranks > 1) ? (size_t)g.N : (size_t)g.ldc;
#pragma unroll 1
      for (int c4 = 0; c4 < BN / 64; ++c4) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld32(tmemBase + ((uint32_t)(quarter * 32) << 16) + ab * BN + c4 * 64 + h * 32, r);
          tmem_ld_wait();
          uint4* srow = (uint4*)(stage + lane * EPI_ROW_BYTES + h * 64);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
            srow[v] = o;
          }
        }
        __syncwarp();
#pragma unroll
        for (int t = 0; t < 8; ++t) {                 // 32 rows x 8 chunks of 16 bytes; 8 lanes cover one row segment
          const int chunk = t * 32 + lane, rr = chunk >> 3, cc = chunk & 7;
          const uint4 o = *(const uint4*)(stage + rr * EPI_ROW_BYTES + cc * 16);
          st_peer16(cbase + (size_t)rr * rowStride + c4 * 64 + cc * 8, o);
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&accEmpty[ab]);      // 4 epilogue warps release the accumulator
      if (f.mode == 2 && f.nranks > 1) {
        // publish the tile in its owner's memory once all four warps have stored their rows
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          __threadfence_system();
          st_rel_sys_u32(f.tileFlag[owner] + (size_t)f.rank * (f.rowsPerRank / BM) * nTiles + tileInOwner, (uint32_t)epoch);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ communication warps (6..9)
    const int ct = threadIdx.x - 6 * 32;              // 0..127
    if (f.mode == 1 && f.nranks > 1) {
      const int blocksPerRank = f.rowsPerRank / BM;
      const size_t blockBytes = (size_t)BM * g.K * 2;
      if (blockIdx.x == 0 && ct < f.nranks && ct != f.rank) st_rel_sys(f.peerArrive[ct], epoch);   // my shard is ready
      // remote row blocks in the order the tiles will need them, each cut into PIECES so that every CTA
      // has loads in flight (one CTA alone moves a few GB/s); a block is ready when all its pieces are
      const int remote = (f.nranks - 1) * blocksPerRank * GATHER_PIECES;
      const size_t pieceBytes = blockBytes / GATHER_PIECES;
      bool ok = true;
      for (int i = blockIdx.x; i < remote && ok; i += gridDim.x) {
        const int bi = i / GATHER_PIECES, piece = i % GATHER_PIECES;
        const int owner = (f.rank + 1 + bi / blocksPerRank) % f.nranks;
        const int blk = bi % blocksPerRank;
        if (ct == 0) ok = wait_flag64(&f.arrive[owner], epoch, giveUp, g.waitNs);
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (*giveUp) break;
        const uint4* src = (const uint4*)((const char*)f.peerA[owner] + (size_t)blk * blockBytes + (size_t)piece * pieceBytes);
        uint4* dst = (uint4*)((char*)f.gathered + ((size_t)owner * blocksPerRank + blk) * blockBytes + (size_t)piece * pieceBytes);
        const size_t n16 = pieceBytes / 16;
        for (size_t p = ct; p < n16; p += 128 * 8) {
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) if (p + u * 128 < n16) v[u] = ld_peer16(src + p + u * 128);
#pragma unroll
          for (int u = 0; u < 8; ++u) if (p + u * 128 < n16) dst[p + u * 128] = v[u];
        }
        asm volatile("fence.proxy.async.global;" ::: "memory");
        __threadfence();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (ct == 0) atomicAdd(&f.blockReady[owner * blocksPerRank + blk], 1u);     // release: the fence above
      }
      // when every CTA is through, the peers may reuse their shards
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (ct == 0) {
        __threadfence();
        if (atomicAdd(f.doneCount, 1u) == gridDim.x - 1) {
          *f.doneCount = 0;
          if (f.epochCounter) *f.epochCounter = epoch;     // every CTA has read the old value long ago
          __threadfence_system();
          for (int j = 0; j < f.nranks; ++j) if (j != f.rank) st_rel_sys(f.peerDone[j], epoch);
        }
      }
      if (blockIdx.x == 0 && ct < f.nranks && ct != f.rank) wait_flag64(&f.done[ct], epoch, giveUp, g.waitNs);   // my shard stays put until read
    } else if (f.mode == 2 && f.nranks > 1) {
      // reduce the tiles I own as their n partial copies arrive: slot[j] written by rank j's epilogue
      const int tilesMine = (f.rowsPerRank / BM) * nTiles;
      for (int i = blockIdx.x; i < tilesMine; i += gridDim.x) {
        const int tm = i / nTiles, tn = i % nTiles;
        if (ct < f.nranks) wait_flag32(f.myTileFlags + (size_t)ct * tilesMine + i, (uint32_t)epoch, giveUp, true, g.waitNs);
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (*giveUp) break;
        // 128 rows x 256 columns = 4096 chunks of 16 bytes; consecutive threads take consecutive chunks of a
        // row (coalesced), four chunks in flight per thread and slot
        const size_t tileOff = (size_t)(tm * BM) * g.N + tn * BN;
        for (int p = ct; p < BM * (BN / 8); p += 128 * 4) {
          float acc[4][8];
          size_t off[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int q = p + u * 128;                       // chunk index: row = q / 32, 16-byte column = q % 32
            off[u] = tileOff + (size_t)(q >> 5) * g.N + (q & 31) * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
          }
          for (int j = 0; j < f.nranks; ++j) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = ld_peer16(f.mySlots + (size_t)j * f.rowsPerRank * g.N + off[u]);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
              for (int q = 0; q < 4; ++q) { acc[u][2 * q] += __uint_as_float(w[q] << 16); acc[u][2 * q + 1] += __uint_as_float(w[q] & 0xffff0000u); }
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 o;
            o.x = pack_bf16x2(acc[u][0], acc[u][1]); o.y = pack_bf16x2(acc[u][2], acc[u][3]);
            o.z = pack_bf16x2(acc[u][4], acc[u][5]); o.w = pack_bf16x2(acc[u][6], acc[u][7]);
            *(uint4*)(f.reduced + off[u]) = o;
          }
        }
      }
      // all my tiles reduced in every CTA: the peers may write the next call's partial tiles
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (ct == 0) {
        __threadfence();
        if (atomicAdd(f.doneCount, 1u) == gridDim.x - 1) {
          *f.doneCount = 0;
          if (f.epochCounter) *f.epochCounter = epoch;     // every CTA has read the old value long ago
          __threadfence_system();
          for (int j = 0; j < f.nranks; ++j) if (j != f.rank) st_rel_sys(f.peerDone[j], epoch);
        }
      }
    }
  }

  // ---------------------------------------------------------------- leave
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmemBase, TMEM_COLS);
  if (threadIdx.x == 0 && *giveUp && !dead) { atomicExch(g.err, 1u); *(volatile uint32_t*)g.errHost = 1u; __threadfence_system(); }
}

// ---- host side
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encodeFn() {
  static EncodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeTiled)p;
    (void)cudaGetLastError();
  });
  return fn;
}

// rows x cols bf16, row-major (cols contiguous), tiles of boxRows x 64 columns, 128-byte swizzle
ncclResult_t makeMapUncached(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t boxRows);

// Encoding a tensor map costs microseconds of host time per call; layers call with the same few
// (pointer, shape) pairs every step, so the encoded maps are kept.
ncclResult_t makeMap(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t boxRows) {
  struct Key { const void* p; uint64_t r, c; uint32_t b; bool operator<(const Key& o) const { return std::tie(p, r, c, b) < std::tie(o.p, o.r, o.c, o.b); } };
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  Key k{base, rows, cols, boxRows};
  {
    std::lock_guard<std::mutex> l(mu);
    auto it = cache.find(k);
    if (it != cache.end()) { *m = it->second; return ncclSuccess; }
  }
  DFCHECK(makeMapUncached(m, base, rows, cols, boxRows));
  std::lock_guard<std::mutex> l(mu);
  if (cache.size() > 4096) cache.clear();
  cache[k] = *m;
  return ncclSuccess;
}

ncclResult_t makeMapUncached(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t boxRows) {
  EncodeTiled fn = encodeFn();
  if (!fn) { DF_WARN("cuTensorMapEncodeTiled is not available"); return ncclSystemError; }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {BK, boxRows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { DF_WARN("cuTensorMapEncodeTiled failed (%d) for %llu x %llu at %p", (int)r, (unsigned long long)rows, (unsigned long long)cols, base); return ncclInvalidArgument; }
  return ncclSuccess;
}

std::atomic<int> g_reservedSms{0};

struct ErrWords { uint32_t* dev = nullptr; volatile uint32_t* host = nullptr; };
ErrWords errWords() {                       // one pair per device, created on first use
  static ErrWords w[64];
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> l(mu);
  if (!w[dev].dev) {
    cudaMalloc((void**)&w[dev].dev, 4);
    cudaMemset(w[dev].dev, 0, 4);
    uint32_t* h = nullptr;
    cudaHostAlloc((void**)&h, 4, cudaHostAllocMapped | cudaHostAllocPortable);
    *h = 0;
    w[dev].host = h;
  }
  return w[dev];
}

ncclResult_t launch(const void* A, const void* B, void* C, int M, int N, int K, const FusedArgs* f, cudaStream_t stream,
                    int aMn = 0, int bMn = 0) {
  if (M <= 0 || N <= 0 || K <= 0 || M % BM || N % BN || K % BK) {
    DF_WARN("tcgen05 GEMM needs M %% %d == 0, N %% %d == 0, K %% %d == 0 (got %d x %d x %d)", BM, BN, BK, M, N, K);
    return ncclInvalidArgument;
  }
  if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) return ncclInvalidArgument;
  const ErrWords ew = errWords();
  if (*ew.host) { DF_WARN("an earlier tensor-core kernel on this device gave up on a bounded wait; call dfcclGemmCheck to clear"); return dfcclTimeout; }
  // plain products whose sizes allow it run on CTA pairs (tiles of 256 x 256, half the shared-memory traffic per FLOP)
  if ((!f || f->mode == 0 || f->nranks <= 1) && gemmPairEligible(M, N, K) && paramI64("GEMM_PAIR", 1) != 0)
    return gemmPairLaunch(A, B, C, M, N, K, stream, aMn, bMn, ew.dev, (uint32_t*)ew.host);
  CUtensorMap ma, mb;
  // K-major operand [rows, K]: boxes of [tile rows] x 64 K-columns; MN-major operand [K, cols]: boxes of 64 K-rows x 64 columns
  if (!aMn) DFCHECK(makeMap(&ma, A, (uint64_t)M, (uint64_t)K, BM)); else DFCHECK(makeMap(&ma, A, (uint64_t)K, (uint64_t)M, BK));
  if (!bMn) DFCHECK(makeMap(&mb, B, (uint64_t)N, (uint64_t)K, BN)); else DFCHECK(makeMap(&mb, B, (uint64_t)K, (uint64_t)N, BK));
  static std::once_flag once;
  std::call_once(once, [] { cudaFuncSetAttribute(dfcclGemmKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); });
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.C = (__nv_bfloat16*)C; g.M = M; g.N = N; g.K = K; g.ldc = N; g.err = ew.dev; g.errHost = (uint32_t*)ew.host;
  g.aMn = aMn ? 1 : 0; g.bMn = bMn ? 1 : 0;
  { int64_t ms = paramI64("WAIT_TIMEOUT_MS", 30000); g.waitNs = (uint64_t)(ms > 0 ? ms : 30000) * 1000000ull; }
  if (f) g.f = *f; else { g.f.nranks = 1; g.f.mode = 0; }
  if (g.f.mode == 0 || g.f.nranks <= 1) { int64_t gm = paramI64("GEMM_RASTER_GROUP", 8); g.groupM = (int)(gm < 1 ? 1 : gm > 64 ? 64 : 2 * gm); }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = (M / BM) * (N / BN);
  // The CTAs of a fused launch serve one another (gathered pieces, partial tiles), so all of them must be resident
  // at once: SMs that a co-running persistent kernel (the daemon) may occupy are left out of the grid.
  const int usable = std::max(1, sms - g_reservedSms.load());
  // fused modes keep one CTA per usable SM even with few tiles: the communication warps of idle CTAs still work
  const int grid = (g.f.mode == 0) ? (tiles < sms ? tiles : sms) : usable;
  dfcclGemmKernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, g);
  CUDACHECK(cudaGetLastError());
  return ncclSuccess;
}

}  // namespace

ncclResult_t gemmMakeMap(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t boxRows) { return makeMap(m, base, rows, cols, boxRows); }
ncclResult_t gemmLaunch(const void* A, const void* B, void* C, int M, int N, int K, const FusedArgs* f, cudaStream_t stream, int aMn, int bMn) {
  return launch(A, B, C, M, N, K, f, stream, aMn, bMn);
}
bool gemmGaveUp() { return *errWords().host != 0; }
void gemmReserveSmsAtLeast(int n) {
  int cur = g_reservedSms.load();
  while (cur < n && !g_reservedSms.compare_exchange_weak(cur, n)) {}
}

}  // namespace dfccl

using namespace dfccl;
#define DF_API extern "C" __attribute__((visibility("default")))

// C[M,N] (bf16, row-major) = A[M,K] * B[N,K]^T, fp32 accumulation in tensor memory.
DF_API ncclResult_t dfcclGemmBf16(const void* A, const void* B, void* C, int M, int N, int K, cudaStream_t stream) {
  return launch(A, B, C, M, N, K, nullptr, stream);
}

// The same product with either operand stored transposed (the contraction index slow): A as [K, M] when `aTransposed`,
// B as [K, N] when `bTransposed`, both row-major.  The weight gradient of a linear layer (both) and its data gradient
// (B) then need no transposed copy: the tensor cores read MN-major operands as they are.
DF_API ncclResult_t dfcclGemmBf16Ex(const void* A, const void* B, void* C, int M, int N, int K, int aTransposed, int bTransposed, cudaStream_t stream) {
  return launch(A, B, C, M, N, K, nullptr, stream, aTransposed, bTransposed);
}

// CTA pairs of the cta_group::2 kernel that can be resident together on the current device.
DF_API ncclResult_t dfcclGemmPairResident(int* pairs) {
  if (!pairs) return ncclInvalidArgument;
  *pairs = gemmPairResident();
  return ncclSuccess;
}

// SMs the fused launches leave free for a persistent kernel that runs beside them (e.g. the daemon's blocks).
DF_API ncclResult_t dfcclGemmReserveSms(int n) {
  if (n < 0 || n > 128) return ncclInvalidArgument;
  g_reservedSms.store(n);
  return ncclSuccess;
}

// Non-zero after a kernel of this file gave up on a bounded wait (reads and clears the word).
DF_API ncclResult_t dfcclGemmCheck(int* failed) {
  uint32_t v = 0;
  const ErrWords ew = errWords();
  CUDACHECK(cudaMemcpy(&v, ew.dev, 4, cudaMemcpyDeviceToHost));
  if (v) { CUDACHECK(cudaMemset(ew.dev, 0, 4)); *ew.host = 0; }
  if (failed) *failed = (int)v;
  return ncclSuccess;
}

// The fused forms are driven from dfccl_b200/ops/fused_linear.py, which owns the symmetric buffers
// and the rendezvous words; it passes them here packed in this struct (same layout as FusedArgs).
DF_API ncclResult_t dfcclGemmFused(const void* A, const void* B, void* C, int M, int N, int K, const void* fusedArgs, size_t fusedBytes,
                                   cudaStream_t stream) {
  if (!fusedArgs || fusedBytes != sizeof(FusedArgs)) { DF_WARN("dfcclGemmFused: argument block of %zu bytes, expected %zu", fusedBytes, sizeof(FusedArgs)); return ncclInvalidArgument; }
  FusedArgs f;
  memcpy(&f, fusedArgs, sizeof(f));
  if (f.nranks < 1 || f.nranks > 8 || f.rank < 0 || f.rank >= f.nranks) return ncclInvalidArgument;
  if (f.nranks > 1 && (f.rowsPerRank % BM || f.rowsPerRank * f.nranks != M)) { DF_WARN("dfcclGemmFused: rows per rank must be a multiple of %d and sum to M", BM); return ncclInvalidArgument; }
  return launch(A, B, C, M, N, K, &f, stream);
}
DF_API size_t dfcclGemmFusedArgsSize(void) { return sizeof(FusedArgs); }
