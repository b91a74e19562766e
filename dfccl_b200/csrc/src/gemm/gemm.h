// Internal interface of the tensor-core GEMM translation unit: the argument block of its communication-fused forms
// and the launcher, for the rank context (registered tensor-parallel operators) and the C entry points.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "dfccl.h"

namespace dfccl {

constexpr int GEMM_BM = 128, GEMM_BN = 256, GEMM_BK = 64;     // tile the problem sizes must be multiples of

struct FusedArgs {
  // ---- all-gather -> GEMM
  int nranks, rank;                 // nranks <= 1: plain GEMM
  int rowsPerRank;                  // rows of A each rank contributes (multiple of BM)
  const __nv_bfloat16* peerA[8];    // each rank's shard [rowsPerRank, K] as mapped here (own entry unused)
  __nv_bfloat16* gathered;          // local [M, K] buffer the tensor map of A covers
  uint32_t* blockReady;             // [M / BM] local counters: a block is in place when it reaches epoch * GATHER_PIECES
  // ---- GEMM -> reduce-scatter
  __nv_bfloat16* slot[8];           // owner j's receive area for MY partial tiles: [rowsPerRank, N] bf16, as mapped here
  uint32_t* tileFlag[8];            // owner j's flags [nranks][tilesPerOwner] as mapped here (I write row `rank`)
  const __nv_bfloat16* mySlots;     // my receive areas: [nranks][rowsPerRank, N]
  const uint32_t* myTileFlags;      // my flags [nranks][tilesPerOwner]
  __nv_bfloat16* reduced;           // my output [rowsPerRank, N]
  // ---- rendezvous words (symmetric heap), written by peers
  volatile uint64_t* arrive;        // [nranks] local: peer j posted epoch -> its buffers are ready
  volatile uint64_t* done;          // [nranks] local: peer j posted epoch -> it no longer reads my buffers
  volatile uint64_t* peerArrive[8]; // where I post for peer j (its arrive[rank])
  volatile uint64_t* peerDone[8];
  uint32_t* doneCount;              // local counter of CTAs that finished their communication work
  uint64_t epoch;                   // this call's number (used when epochCounter is null)
  uint64_t* epochCounter;           // local device word: calls finished so far; this call is that + 1.  Kept on the device
                                    // so that a launch captured in a CUDA graph finds the right number at every replay.
  int mode;                         // 0 plain, 1 all-gather -> GEMM, 2 GEMM -> reduce-scatter
};

// C[M,N] = A[M,K] * B[N,K]^T on `stream`; `f` selects a fused form (null = plain GEMM).  aMn / bMn: the operand is
// stored with the contraction index slow (A as [K, M], B as [K, N], row-major) and read by the tensor cores as it is.
ncclResult_t gemmLaunch(const void* A, const void* B, void* C, int M, int N, int K, const FusedArgs* f, cudaStream_t stream,
                        int aMn = 0, int bMn = 0);
// The CTA-pair kernel (cta_group::2, tiles of 256 x 256) for plain GEMMs whose sizes allow it.
bool gemmPairEligible(int M, int N, int K);
int gemmPairResident();
ncclResult_t gemmPairLaunch(const void* A, const void* B, void* C, int M, int N, int K, cudaStream_t stream, int aMn, int bMn,
                            uint32_t* errDev, uint32_t* errHost);
// Cached tensor map of a row-major bf16 matrix [rows, cols] cut into boxes of boxRows x 64 columns, 128-byte swizzle.
ncclResult_t gemmMakeMap(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t boxRows);
// True when a kernel of the current device gave up on a bounded wait (pinned word, no device access).
bool gemmGaveUp();
// SMs the fused launches leave to a co-resident persistent kernel: raised to at least `n`.
void gemmReserveSmsAtLeast(int n);

}  // namespace dfccl
