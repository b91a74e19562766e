// bf16 GEMM on CTA pairs (tcgen05 cta_group::2), hand-written for sm_100a:
//     C[M,N] = A[M,K] * B[N,K]^T,  tiles of 256 x 256, one tile per pair of CTAs (a cluster of two SMs).
// Each CTA of a pair loads 128 rows of A and 128 rows of B per 64-wide K block (32 KB per stage instead of the 48 KB
// of the one-CTA form, so six stages fit), the leader's single MMA thread issues 256 x 256 x 16 instructions that read
// both CTAs' shared memory, and each CTA ends up with its 128 rows of the accumulator in its own tensor memory.
// The tensor cores of an SM thus see every B row once per pair instead of once per CTA: half the shared-memory
// operand traffic per FLOP, which is what bounds the one-CTA kernel.
//
// Roles per CTA: warp 0 = TMA producer (one elected thread; completion of both CTAs' loads is counted on the
// LEADER's barrier), warp 1 = tensor-memory owner, and in the leader the MMA issuer; warps 2-5 = epilogue over the
// CTA's own accumulator half.  Stages are released and accumulators handed over with tcgen05.commit to both CTAs;
// the epilogues of both CTAs arrive on the leader's accumulator-empty barrier.  No TMA load uses cluster multicast.
// Every wait is bounded and ends in the error word of the device.
//
// The reference has no tensor-core code (it is a collective library); this kernel serves the tensor-parallel
// workloads' plain GEMMs (weight and data gradients, unfused forwards).
#include "tc_common.h"
#include "gemm.h"
#include "../common/param.h"
#include "../common/log.h"
#include <algorithm>
#include <mutex>

namespace dfccl {
namespace {

using namespace tc;

constexpr int PM = 256, PN = 256, BK = 64, HALF = 128, STAGES = 6, UMMA_K = 16;
constexpr int A_BYTES = HALF * BK * 2, B_BYTES = HALF * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;   // per CTA
constexpr int MN_BLOCK_BYTES = 64 * BK * 2;
constexpr int TMEM_COLS = 512;                       // two accumulators of 256 fp32 columns (128 lanes each, per CTA)
constexpr int NUM_THREADS = 192;                     // 6 warps
constexpr int EPI_ROW_BYTES = 64 * 2 + 16;
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 4 * EPI_WARP_BYTES + 1024 + 256;
constexpr uint64_t WAIT_NS = 4000000000ull;          // nothing here waits on another GPU: seconds mean a lost partner

struct PairArgs {
  __nv_bfloat16* C;
  int M, N, K, ldc;
  int aMn, bMn;
  int groupM;                       // row tiles per rasterisation group
  uint32_t* err;
  uint32_t* errHost;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
dfcclGemmPairKernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const PairArgs g) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
  uint8_t* epiSmem = smem + STAGES * STAGE_BYTES;
  uint64_t* fullBar = (uint64_t*)(epiSmem + 4 * EPI_WARP_BYTES);     // used in the leader only
  uint64_t* emptyBar = fullBar + STAGES;                             // in both CTAs (commit to both)
  uint64_t* accFull = emptyBar + STAGES;                             // [2] in both CTAs
  uint64_t* accEmpty = accFull + 2;                                  // [2] used in the leader only: 8 epilogue warps arrive
  uint32_t* tmemBaseSlot = (uint32_t*)(accEmpty + 2);
  volatile uint32_t* giveUp = tmemBaseSlot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cr = cluster_ctarank();             // 0 = leader
  const int mTiles = g.M / PM, nTiles = g.N / PN, kBlocks = g.K / BK;
  const int numTiles = mTiles * nTiles;
  const int pair = blockIdx.x >> 1, numPairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&fullBar[s], 1); mbar_init(&emptyBar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&accFull[a], 1); mbar_init(&accEmpty[a], 8); }
    *giveUp = *(volatile uint32_t*)g.err;            // an earlier kernel gave up: do nothing (both CTAs read the same word)
    mbar_fence_init();
    tma_prefetch_desc(&mapA);
    tma_prefetch_desc(&mapB);
  }
  if (warp == 1) tmem_alloc_pair(tmemBaseSlot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                // the partner's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmemBase = *tmemBaseSlot;
  const bool dead = *giveUp != 0;

  if (dead) {
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs; bytes counted in the leader)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < numTiles && ok; t += numPairs) {
        int mt, nt;
        raster_tile(t, mTiles, nTiles, g.groupM, mt, nt);
        const int rowA = mt * PM + (int)cr * HALF, rowB = nt * PN + (int)cr * HALF;
        for (int kb = 0; kb < kBlocks; ++kb) {
          if (!mbar_wait(&emptyBar[stage], phase ^ 1, giveUp, WAIT_NS)) { ok = false; break; }
          if (cr == 0) mbar_expect_tx(&fullBar[stage], 2 * STAGE_BYTES);        // my bytes and the partner's
          const uint32_t bar = mapa_u32(smem_u32(&fullBar[stage]), 0);
          uint8_t* sa = smem + stage * STAGE_BYTES;
          if (!g.aMn) tma_load_2d_pair(sa, &mapA, kb * BK, rowA, bar);
          else for (int i = 0; i < HALF / 64; ++i) tma_load_2d_pair(sa + i * MN_BLOCK_BYTES, &mapA, rowA + 64 * i, kb * BK, bar);
          if (!g.bMn) tma_load_2d_pair(sa + A_BYTES, &mapB, kb * BK, rowB, bar);
          else for (int i = 0; i < HALF / 64; ++i) tma_load_2d_pair(sa + A_BYTES + i * MN_BLOCK_BYTES, &mapB, rowB + 64 * i, kb * BK, bar);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) for (int i = 0; i < 20000; ++i) __nanosleep(200);     // copies already issued land before the CTA goes away
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (cr == 0 && elect_one()) {
      const uint32_t idesc = umma_idesc_bf16(PM, PN, g.aMn, g.bMn);
      const uint32_t stepA = g.aMn ? 128u : 2u, stepB = g.bMn ? 128u : 2u;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = pair; t < numTiles && ok; t += numPairs, ++it) {
        const int ab = it & 1;
        if (!mbar_wait(&accEmpty[ab], ((it >> 1) & 1) ^ 1, giveUp, WAIT_NS)) break;
        tc_fence_after();
        const uint32_t d = tmemBase + ab * PN;
        for (int kb = 0; kb < kBlocks; ++kb) {
          if (!mbar_wait(&fullBar[stage], phase, giveUp, WAIT_NS)) { ok = false; break; }
          tc_fence_after();
          const uint8_t* pa = smem + stage * STAGE_BYTES;
          const uint64_t da = g.aMn ? umma_smem_desc_mn_sw128(pa, MN_BLOCK_BYTES) : umma_smem_desc_sw128(pa);
          const uint64_t db = g.bMn ? umma_smem_desc_mn_sw128(pa + A_BYTES, MN_BLOCK_BYTES) : umma_smem_desc_sw128(pa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_pair(d, da + stepA * k, db + stepB * k, idesc, (kb | k) != 0);
          umma_commit_pair(&emptyBar[stage]);         // both CTAs' stage is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&accFull[ab]);       // both halves of the accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue: my 128 rows, TMEM -> bf16 -> global
    const int quarter = warp & 3;
    const uint32_t accEmptyLeader0 = mapa_u32(smem_u32(&accEmpty[0]), 0), accEmptyLeader1 = mapa_u32(smem_u32(&accEmpty[1]), 0);
    int it = 0;
    for (int t = pair; t < numTiles; t += numPairs, ++it) {
      int mt, nt;
      raster_tile(t, mTiles, nTiles, g.groupM, mt, nt);
      const int ab = it & 1;
      if (!mbar_wait(&accFull[ab], (it >> 1) & 1, giveUp, WAIT_NS)) break;
      tc_fence_after();
      uint8_t* stg = epiSmem + (warp - 2) * EPI_WARP_BYTES;
      __nv_bfloat16* cbase = g.C + (size_t)(mt * PM + (int)cr * HALF + quarter * 32) * g.ldc + nt * PN;   // row 0 of this warp's 32 rows
#pragma unroll 1
      for (int c4 = 0; c4 < PN / 64; ++c4) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld32(tmemBase + ((uint32_t)(quarter * 32) << 16) + ab * PN + c4 * 64 + h * 32, r);
          tmem_ld_wait();
          uint4* srow = (uint4*)(stg + lane * EPI_ROW_BYTES + h * 64);
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
        for (int q = 0; q < 8; ++q) {                 // 32 rows x 8 chunks of 16 bytes; 8 lanes cover one 128-byte row segment
          const int chunk = q * 32 + lane, rr = chunk >> 3, cc = chunk & 7;
          const uint4 o = *(const uint4*)(stg + rr * EPI_ROW_BYTES + cc * 16);
          *(uint4*)(cbase + (size_t)rr * g.ldc + c4 * 64 + cc * 8) = o;
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(ab ? accEmptyLeader1 : accEmptyLeader0);   // 8 epilogue warps of the pair release the accumulator
    }
  }

  // ---------------------------------------------------------------- leave: nothing of the pair may still use my shared or tensor memory
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmemBase, TMEM_COLS);
  if (threadIdx.x == 0 && *giveUp && !dead) { atomicExch(g.err, 1u); *(volatile uint32_t*)g.errHost = 1u; __threadfence_system(); }
}

}  // namespace

bool gemmPairEligible(int M, int N, int K) { return M > 0 && N > 0 && K > 0 && M % PM == 0 && N % PN == 0 && K % BK == 0; }

namespace {
int maxResidentPairs(int dev, int sms) {
  // pairs that can be resident together (a GPC with an odd number of free SMs leaves one unpaired)
  static int maxPairs[64];
  static std::mutex mu;
  std::lock_guard<std::mutex> l(mu);
  if (!maxPairs[dev & 63]) {
    static std::once_flag once;
    std::call_once(once, [] { cudaFuncSetAttribute(dfcclGemmPairKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); });
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(sms & ~1); cfg.blockDim = dim3(NUM_THREADS); cfg.dynamicSmemBytes = SMEM_BYTES;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, dfcclGemmPairKernel, &cfg) != cudaSuccess || n <= 0) { (void)cudaGetLastError(); n = sms / 2; }
    maxPairs[dev & 63] = std::min(n, sms / 2);
  }
  return maxPairs[dev & 63];
}
}  // namespace

int gemmPairResident() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return maxResidentPairs(dev, sms);
}

ncclResult_t gemmPairLaunch(const void* A, const void* B, void* C, int M, int N, int K, cudaStream_t stream, int aMn, int bMn,
                            uint32_t* errDev, uint32_t* errHost) {
  CUtensorMap ma, mb;
  if (!aMn) DFCHECK(gemmMakeMap(&ma, A, (uint64_t)M, (uint64_t)K, HALF)); else DFCHECK(gemmMakeMap(&ma, A, (uint64_t)K, (uint64_t)M, BK));
  if (!bMn) DFCHECK(gemmMakeMap(&mb, B, (uint64_t)N, (uint64_t)K, HALF)); else DFCHECK(gemmMakeMap(&mb, B, (uint64_t)K, (uint64_t)N, BK));
  PairArgs g;
  memset(&g, 0, sizeof(g));
  g.C = (__nv_bfloat16*)C; g.M = M; g.N = N; g.K = K; g.ldc = N; g.aMn = aMn ? 1 : 0; g.bMn = bMn ? 1 : 0;
  g.err = errDev; g.errHost = errHost;
  { int64_t gm = paramI64("GEMM_RASTER_GROUP", 8); g.groupM = (int)(gm < 1 ? 1 : gm > 64 ? 64 : gm); }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = (M / PM) * (N / PN);
  const int pairs = std::min(tiles, maxResidentPairs(dev, sms));
  dfcclGemmPairKernel<<<2 * pairs, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, g);
  CUDACHECK(cudaGetLastError());
  return ncclSuccess;
}

}  // namespace dfccl
