/* Compute-side entry points of dfccl-b200: the tcgen05 GEMM with a collective inside, the fused
 * optimizer step, the fabric probes and the introspection calls of topology and tuner.
 * (The collective interfaces are in dfccl.h.)  None of this exists in the reference, which is a
 * collective library only; these serve the tensor-parallel and data-parallel workloads built on it. */
#ifndef DFCCL_OPS_H_
#define DFCCL_OPS_H_
#include "dfccl.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory, TMA operand loads)
 * C[M,N] (bf16, row-major) = A[M,K] * B[N,K]^T with fp32 accumulation.  M % 128 == 0, N % 256 == 0, K % 64 == 0,
 * pointers 16-byte aligned. */
ncclResult_t dfcclGemmBf16(const void* A, const void* B, void* C, int M, int N, int K, cudaStream_t stream);
/* The same with either operand stored transposed (contraction index slow): A as [K, M] when aTransposed, B as [K, N] when
 * bTransposed, row-major.  No copy is made: the kernel describes such an operand to the tensor cores as MN-major. */
ncclResult_t dfcclGemmBf16Ex(const void* A, const void* B, void* C, int M, int N, int K, int aTransposed, int bTransposed,
                             cudaStream_t stream);

/* The same kernel with a collective inside (driven by dfccl_b200/ops/fused_linear.py, which owns the symmetric
 * buffers and rendezvous words): `fusedArgs` is the argument block of csrc/src/gemm/tcgen05_gemm.cu (its size is
 * checked against dfcclGemmFusedArgsSize()).  mode 1: A is the local [M,K] buffer the peers' row blocks are
 * gathered into while the tensor cores work on blocks already present (all-gather -> GEMM); mode 2: partial output
 * tiles are stored into their owner's memory and summed there (GEMM -> reduce-scatter). */
ncclResult_t dfcclGemmFused(const void* A, const void* B, void* C, int M, int N, int K, const void* fusedArgs, size_t fusedBytes,
                            cudaStream_t stream);
size_t dfcclGemmFusedArgsSize(void);
/* Reads and clears the "a bounded wait ran out" word of this device's GEMM kernels. */
ncclResult_t dfcclGemmCheck(int* failed);
// CTA pairs of the cta_group::2 GEMM kernel that can be resident together on the current device.
ncclResult_t dfcclGemmPairResident(int* pairs);
/* SMs the fused launches leave free for a persistent kernel that runs beside them (the daemon's blocks). */
ncclResult_t dfcclGemmReserveSms(int n);

/* ---- fused SGD with momentum over a flat bucket: master (fp32) -= lr * (momentum = mu * momentum + grad + wd * master),
 * param = cast(master).  paramType: ncclBfloat16 or ncclFloat32.  All arrays 16-byte aligned. */
ncclResult_t dfcclFusedSgdStep(void* master, const void* grad, void* momentum, void* param, size_t n, int paramType,
                               float lr, float mu, float wd, int firstStep, cudaStream_t stream);
/* AdamW (decoupled weight decay) over the same flat arrays; `step` counts from 1, both moment arrays start at zero. */
ncclResult_t dfcclFusedAdamWStep(void* master, const void* grad, void* moment1, void* moment2, void* param, size_t n, int paramType,
                                 float lr, float beta1, float beta2, float eps, float wd, int step, cudaStream_t stream);
ncclResult_t dfcclOpsWarm(void);   /* load these kernels now (before any stream can block) */

/* ---- fabric probes (roofline inputs): mean device time in microseconds */
/* direction 0 = read the peer's heap, 1 = write it; loadKind selects the load instruction form; `unroll` independent
 * 16-byte accesses in flight per thread. */
ncclResult_t dfcclProbePeerCopy(ncclComm_t comm, int peer, size_t bytes, int direction, int loadKind, int unroll, int blocks,
                                int iters, double* usOut);
/* Round trip of one flag word between this rank and `peer` (both call it). */
ncclResult_t dfcclProbeFlagRoundTrip(ncclComm_t comm, int peer, int iters, double* usOut);
/* Round trip "the stream releases a word, a resident kernel answers, the stream goes on" on the current device: what one
 * stream-ordered submission costs before any collective runs.  mode bit 0: the write is a one-thread kernel instead of a
 * stream memory operation; bit 1: so is the wait; bit 2: the write also stores a mirror word in pinned host memory. */
/* Cost in nanoseconds of the single memory operations the daemon's control path is made of, timed by one thread on the
 * current device: [0] load of a pinned host word, [1] store to it, [2] that store + system fence, [3] device store +
 * system fence, [4] device store + device fence, [5] system fence alone, [6] device atomic, [7] device load (independent
 * loads), [8] / [9] device store + acq_rel fence of system / device scope, [10] device load (dependent chain),
 * [11] release store of system scope, [12] one read of the nanosecond timer. */
ncclResult_t dfcclProbeMemoryOps(int iters, uint64_t nsOut[13]);
ncclResult_t dfcclProbeStreamRoundTrip(int mode, int iters, int delayUs, double* usOut);   /* the kernel answers delayUs late */

/* ---- introspection */
int dfcclTopoXml(char* buf, int cap);          /* the detected (or injected) topology as XML; returns the length */
void dfcclTopoReset(void);
int dfcclTopoGpuCount(void);
/* Path policy: 1 when devices a and b may use one another's memory directly (peer access exists, P2P_DISABLE is not
 * set, the path is within P2P_LEVEL = LOC | NVL | PIX | PXB | PHB | SYS), 0 when not, -1 on error. */
int dfcclTopoP2pAllowed(int a, int b);
ncclResult_t dfcclTunerChoose(int kind, size_t bytes, int nranks, int maxBlocks, int nvls, int pinnedAlgo, int* algo,
                              int* nBlocks, double* predictedUs);
double dfcclTunerPredictUs(int kind, int algo, size_t bytes, int nranks, int nBlocks);
const char* dfcclLastError(void);
ncclResult_t dfcclHeapPeerBase(ncclComm_t comm, int peer, void** base);
/* Transport the members selected together: 0 peer memory, 1 heap in registered host shared memory (GPUs of one host
 * without peer access, or NCCL_P2P_DISABLE=1), 2 host-staged over the network transport. */
ncclResult_t dfcclCommTransport(ncclComm_t comm, int* kind);

#ifdef __cplusplus
}
#endif
#endif
