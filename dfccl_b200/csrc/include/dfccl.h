/* dfccl.h - public C interface of the B200-native deadlock-free collective library.
 *
 * Three groups of entry points:
 *   1. nccl*   : the stream-ordered communicator interface, source compatible with
 *                the subset of NCCL 2.12 that the reference exports
 *                (reference: src/nccl.h.in:54-108, 169-179, 248-453).
 *   2. ofccl*  : the register-then-submit interface of the reference
 *                (reference: src/nccl.h.in:202-235, 253-378): prepare a collective
 *                under an integer id, finalize the rank context, then submit
 *                (sendbuff, recvbuff, id, callback) in any order on any rank.
 *   3. dfccl*  : additions that have no counterpart in the reference: symmetric
 *                heap allocation, fused scale / cast registration, stream-ordered
 *                submission without a host callback, statistics, error status,
 *                the in-process CPU backend and loopback rank groups used by tests.
 *
 * Every p-prefixed profiling alias of the reference (pncclAllReduce, pofcclRun...)
 * is exported as well, so that a tool can interpose on the plain names
 * (reference: PROFAPI in src/include/core.h:17-31).
 */
#ifndef DFCCL_H_
#define DFCCL_H_

#include <stddef.h>
#include <stdint.h>

#ifndef DFCCL_NO_CUDA_TYPES
#include <cuda_runtime.h>
#else
typedef struct CUstream_st* cudaStream_t;
#endif

#define NCCL_MAJOR 2
#define NCCL_MINOR 12
#define NCCL_PATCH 12
#define NCCL_SUFFIX "dfccl-b200"
#define NCCL_VERSION(X, Y, Z) (((X) <= 2 && (Y) <= 8) ? (X)*1000 + (Y)*100 + (Z) : (X)*10000 + (Y)*100 + (Z))
#define NCCL_VERSION_CODE NCCL_VERSION(NCCL_MAJOR, NCCL_MINOR, NCCL_PATCH)

#define DFCCL_VERSION_CODE 100 /* 0.1.0 of this library */

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ncclComm* ncclComm_t;
typedef struct ofcclRankCtx* ofcclRankCtx_t;

/* Completion callback: runs on the context's poller thread, once per submit. */
typedef int (*CallbackFunc)(int collId, void* args);

#define NCCL_UNIQUE_ID_BYTES 128
typedef struct { char internal[NCCL_UNIQUE_ID_BYTES]; } ncclUniqueId;

typedef enum {
  ncclSuccess = 0,
  ncclUnhandledCudaError = 1,
  ncclSystemError = 2,
  ncclInternalError = 3,
  ncclInvalidArgument = 4,
  ncclInvalidUsage = 5,
  ncclNumResults = 6,
  /* extensions (never returned by an nccl* or ofccl* call of the reference) */
  dfcclTimeout = 6,        /* a bounded device wait ran out */
  dfcclAborted = 7,        /* the communicator or context was aborted */
  dfcclNumResults = 8
} ncclResult_t;

typedef enum { ncclNumOps_dummy = 5 } ncclRedOp_dummy_t;
typedef enum {
  ncclSum = 0, ncclProd = 1, ncclMax = 2, ncclMin = 3, ncclAvg = 4,
  ncclNumOps = 5, /* first value handed out by ncclRedOpCreatePreMulSum */
  ncclMaxRedOp = 0x7fffffff >> (32 - 8 * sizeof(ncclRedOp_dummy_t))
} ncclRedOp_t;

typedef enum {
  ncclInt8 = 0, ncclChar = 0, ncclUint8 = 1, ncclInt32 = 2, ncclInt = 2, ncclUint32 = 3,
  ncclInt64 = 4, ncclUint64 = 5, ncclFloat16 = 6, ncclHalf = 6, ncclFloat32 = 7, ncclFloat = 7,
  ncclFloat64 = 8, ncclDouble = 8, ncclBfloat16 = 9, ncclNumTypes = 10
} ncclDataType_t;

typedef enum { ncclScalarDevice = 0, ncclScalarHostImmediate = 1 } ncclScalarResidence_t;

/* ------------------------------------------------------------------ communicator */
ncclResult_t ncclGetVersion(int* version);
ncclResult_t ncclGetUniqueId(ncclUniqueId* uniqueId);
ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank);
ncclResult_t ncclCommInitAll(ncclComm_t* comm, int ndev, const int* devlist);
ncclResult_t ncclCommDestroy(ncclComm_t comm);
ncclResult_t ncclCommAbort(ncclComm_t comm);
const char* ncclGetErrorString(ncclResult_t result);
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* asyncError);
ncclResult_t ncclCommCount(const ncclComm_t comm, int* count);
ncclResult_t ncclCommCuDevice(const ncclComm_t comm, int* device);
ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank);
ncclResult_t ncclRedOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t datatype,
                                      ncclScalarResidence_t residence, ncclComm_t comm);
ncclResult_t ncclRedOpDestroy(ncclRedOp_t op, ncclComm_t comm);

/* ------------------------------------------------------------------ stream-ordered collectives */
ncclResult_t ncclReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype,
                        ncclRedOp_t op, int root, ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclBcast(void* buff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm,
                       cudaStream_t stream);
ncclResult_t ncclBroadcast(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype,
                           int root, ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype,
                           ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount,
                               ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, ncclDataType_t datatype,
                           ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclSend(const void* sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm,
                      cudaStream_t stream);
ncclResult_t ncclRecv(void* recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm,
                      cudaStream_t stream);
ncclResult_t ncclGroupStart(void);
ncclResult_t ncclGroupEnd(void);

/* ------------------------------------------------------------------ register-then-submit */
/* `rank` doubles as the CUDA device ordinal the daemon kernel runs on, as in the
 * reference (src/enqueue_ofccl.cc:853); use dfcclInitRankCtxOnDevice to choose. */
ncclResult_t ofcclInitRankCtx(ofcclRankCtx_t* rankCtx, int rank);
ncclResult_t ofcclFinalizeRankCtx7StartHostThrds(ofcclRankCtx_t rankCtx);
ncclResult_t ofcclPrepareDone(ofcclRankCtx_t rankCtx); /* finalize + eager daemon launch */
ncclResult_t ofcclDestroy(ofcclRankCtx_t rankCtx);

ncclResult_t ofcclPrepareReduce(size_t count, ncclDataType_t datatype, ncclRedOp_t op, int root,
                                ncclComm_t comm, int collId, ofcclRankCtx_t rankCtx);
ncclResult_t ofcclRunReduce(const void* sendbuff, void* recvbuff, int collId, CallbackFunc callback,
                            void* callbackArgs, ofcclRankCtx_t rankCtx);
ncclResult_t ofcclPrepareBcast(size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, int collId,
                               ofcclRankCtx_t rankCtx);
ncclResult_t ofcclRunBcast(void* buff, int collId, CallbackFunc callback, void* callbackArgs,
                           ofcclRankCtx_t rankCtx);
ncclResult_t ofcclPrepareBroadcast(size_t count, ncclDataType_t datatype, int root, ncclComm_t comm,
                                   int collId, ofcclRankCtx_t rankCtx);
ncclResult_t ofcclRunBroadcast(const void* sendbuff, void* recvbuff, int collId, CallbackFunc callback,
                               void* callbackArgs, ofcclRankCtx_t rankCtx);
ncclResult_t ofcclPrepareAllReduce(size_t count, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm,
                                   int collId, ofcclRankCtx_t rankCtx);
ncclResult_t ofcclRunAllReduce(const void* sendbuff, void* recvbuff, int collId, CallbackFunc callback,
                               void* callbackArgs, ofcclRankCtx_t rankCtx);
ncclResult_t ofcclPrepareReduceScatter(size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op,
                                       ncclComm_t comm, int collId, ofcclRankCtx_t rankCtx);
ncclResult_t ofcclRunReduceScatter(const void* sendbuff, void* recvbuff, int collId, CallbackFunc callback,
                                   void* callbackArgs, ofcclRankCtx_t rankCtx);
ncclResult_t ofcclPrepareAllGather(size_t sendcount, ncclDataType_t datatype, ncclComm_t comm, int collId,
                                   ofcclRankCtx_t rankCtx);
ncclResult_t ofcclRunAllGather(const void* sendbuff, void* recvbuff, int collId, CallbackFunc callback,
                               void* callbackArgs, ofcclRankCtx_t rankCtx);

/* ------------------------------------------------------------------ dfccl extensions */

/* Backends a communicator can live on. */
typedef enum {
  dfcclBackendCuda = 0, /* one GPU per rank, peer memory over NVLink / NVSwitch */
  dfcclBackendHost = 1  /* host memory + CPU threads standing in for thread blocks (tests, no GPU) */
} dfcclBackend_t;

/* Collective kinds (also the values of `kind` in dfcclCollInfo). */
typedef enum {
  dfcclCollAllReduce = 0, dfcclCollAllGather = 1, dfcclCollReduceScatter = 2,
  dfcclCollBroadcast = 3, dfcclCollReduce = 4, dfcclCollNumKinds = 5
} dfcclColl_t;

/* Data-path schedules of the engine. */
typedef enum {
  dfcclAlgoAuto = 0,
  dfcclAlgoOneShot = 1,  /* every rank reads all inputs, reduces locally */
  dfcclAlgoTwoShot = 2,  /* owner reduces its shard from all peers and writes it to all peers */
  dfcclAlgoNvls = 3,     /* switch-side reduce / broadcast through a multicast mapping */
  dfcclAlgoPush = 4      /* small all-reduce in one hop: every rank writes its input into slots at every peer, then reduces locally */
} dfcclAlgo_t;

/* Select the backend for communicators created afterwards by this thread's process
 * (default: DFCCL_BACKEND env, else cuda when a GPU is visible, else host). */
ncclResult_t dfcclSetBackend(dfcclBackend_t backend);
ncclResult_t dfcclGetBackend(dfcclBackend_t* backend);

/* Single-process group of `nranks` communicators that all live on ONE device
 * (cuda backend) or in host memory (host backend).  Their daemons run as one
 * kernel launch, so a single GPU can exercise every multi-rank code path. */
ncclResult_t dfcclCommInitLoopback(ncclComm_t* comms, int nranks, int device);

/* Split: ranks passing the same color form a new communicator ordered by key. */
ncclResult_t dfcclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm);

/* Symmetric heap: memory every peer of every communicator of this process can
 * load from and store to.  Buffers from here take the zero-copy path; any other
 * device pointer is staged through the heap by the engine. */
ncclResult_t dfcclMemAlloc(void** ptr, size_t bytes, ncclComm_t comm);
ncclResult_t dfcclMemFree(void* ptr, ncclComm_t comm);
ncclResult_t dfcclHeapInfo(ncclComm_t comm, void** base, size_t* bytes, size_t* used);

/* NVLS arena (opt-in): `bytes` of every member's device memory bound to one NVLink-switch multicast
 * object.  All-reduces (sum; f32, bf16, f16) of at least DFCCL_NVLS_MIN_BYTES then run as
 * multimem.ld_reduce + multimem.st; buffers from dfcclNvlsAlloc are used in place, others are copied
 * through the arena.  dfcclNvlsInit is collective over the communicator (DFCCL_NVLS=1 does the same at
 * communicator creation with DFCCL_NVLS_BYTES); *available is 0 when the devices, the driver or the
 * process layout cannot do it, and nothing changes then.  dfcclNvlsAlloc must be called with the same
 * sizes in the same order by every member (offsets are symmetric); the memory lives as long as the
 * communicator. */
ncclResult_t dfcclNvlsInit(ncclComm_t comm, size_t bytes, int* available);
ncclResult_t dfcclNvlsAlloc(void** ptr, size_t bytes, ncclComm_t comm);
ncclResult_t dfcclNvlsInfo(ncclComm_t comm, void** unicastBase, void** multicastBase, size_t* bytes, size_t* used);

ncclResult_t dfcclInitRankCtxOnDevice(ofcclRankCtx_t* rankCtx, int rank, int device);
/* Daemon grid of this context: thread blocks per rank and threads per block (multiple of 32, <= 512);
 * 0 keeps the default (DFCCL_DAEMON_BLOCKS / DFCCL_DAEMON_THREADS).  Call before finalizing.  All ranks
 * of a collective must use the same number of blocks. */
ncclResult_t dfcclSetDaemonGeometry(ofcclRankCtx_t rankCtx, int blocks, int threads);

/* Registration with the fused epilogue: out = cast<outType>(scale * reduce(in)).
 * `scale` multiplies the reduced value (ncclAvg sets it to 1/nranks by itself).
 * `algo` pins a schedule (dfcclAlgoAuto lets the tuner pick by size). */
typedef struct {
  int kind;                 /* dfcclColl_t */
  size_t count;             /* NCCL conventions: AllGather sendcount, ReduceScatter recvcount */
  ncclDataType_t inType;
  ncclDataType_t outType;
  ncclRedOp_t op;
  int root;
  float scale;
  int algo;                 /* dfcclAlgo_t */
  int nBlocks;              /* 0 = tuner's choice */
  int flags;                /* DFCCL_COLL_* */
} dfcclCollInfo;
/* The buffers of every submission of this collective lie in the communicator's multicast arena (dfcclNvlsAlloc):
 * the multimem schedule then works on them in place and reserves no staging slots for the collective.  A submission
 * that breaks the promise is refused. */
#define DFCCL_COLL_ARENA_BUFFERS 1
ncclResult_t dfcclPrepare(const dfcclCollInfo* info, ncclComm_t comm, int collId, ofcclRankCtx_t rankCtx);

/* Generic submit (what every ofcclRun* wrapper calls). */
ncclResult_t dfcclRun(const void* sendbuff, void* recvbuff, int collId, CallbackFunc callback,
                      void* callbackArgs, ofcclRankCtx_t rankCtx);

/* Stream-ordered submit: the collective starts once `stream` has executed everything
 * enqueued before this call, and work enqueued on `stream` after dfcclStreamWait
 * runs after the collective completed.  No host thread is involved in either edge
 * (stream memory operations on a device flag); `callback` may be NULL. */
ncclResult_t dfcclRunOnStream(const void* sendbuff, void* recvbuff, int collId, cudaStream_t stream,
                              CallbackFunc callback, void* callbackArgs, ofcclRankCtx_t rankCtx);
ncclResult_t dfcclStreamWait(int collId, cudaStream_t stream, ofcclRankCtx_t rankCtx);
/* The same in two steps, for steps that are captured in a CUDA graph.  dfcclRunDeferred publishes the submission
 * (buffers, callback) without touching any stream; dfcclTriggerOnStream enqueues its release on `stream` as a
 * one-thread kernel that counts the releases of `collId` on the device.  That kernel can be captured: every replay
 * of the graph releases the next published submission of the id, at the point of the captured step where the
 * collective's input is complete - a gradient bucket is reduced while the rest of the backward pass still runs.
 * Each submission must be released exactly once; which of the two calls comes first does not matter. */
ncclResult_t dfcclRunDeferred(const void* sendbuff, void* recvbuff, int collId, CallbackFunc callback,
                              void* callbackArgs, ofcclRankCtx_t rankCtx);
ncclResult_t dfcclTriggerOnStream(int collId, cudaStream_t stream, ofcclRankCtx_t rankCtx);
/* ---- tensor-parallel operators whose collective runs inside the GEMM kernel, registered with the rank context like
 * any other collective: their rendezvous words, epoch counter and receive areas are allocated and exchanged when the
 * context is finalized, they are counted in dfcclGetStats, a bounded wait that ran out inside one of them surfaces in
 * dfcclGetAsyncError, and the SMs of this context's daemon are kept out of their grids (all CTAs of a fused launch
 * must be resident at once).  The operators themselves are stream-ordered kernels: members of a communicator issue
 * them in the same order, in any order relative to the collectives they submit to the daemon. */
typedef enum {
  dfcclFusedAllGatherGemm = 1,     /* out[M, n] = all_gather(x_shard)[M, k] * w[n, k]^T,        M = rowsPerRank * nranks */
  dfcclFusedGemmReduceScatter = 2  /* out[rowsPerRank, n] = my rows of sum over ranks of x[M, k] * w[n, k]^T */
} dfcclFusedKind_t;
typedef struct {
  int kind;          /* dfcclFusedKind_t */
  int rowsPerRank;   /* rows of the sharded operand / result each rank owns (a multiple of 128) */
  int k;             /* contraction length on this rank (a multiple of 64) */
  int n;             /* output columns on this rank (a multiple of 256) */
} dfcclFusedInfo;
ncclResult_t dfcclPrepareFusedGemm(const dfcclFusedInfo* info, ncclComm_t comm, int collId, ofcclRankCtx_t rankCtx);
/* After finalize, all-gather -> GEMM only: *shard = where this rank's [rowsPerRank, k] rows go (writing the input there
 * saves the copy), *gathered = the [M, k] operand, complete after a call (the weight gradient needs it). */
ncclResult_t dfcclFusedGemmOperand(int collId, ofcclRankCtx_t rankCtx, void** shard, void** gathered);
/* bf16 operands; x: [rowsPerRank, k] (all-gather -> GEMM) or [M, k] (GEMM -> reduce-scatter); w: [n, k]. */
ncclResult_t dfcclRunFusedGemm(int collId, const void* x, const void* w, void* out, cudaStream_t stream, ofcclRankCtx_t rankCtx);
/* The same with the weight handed over transposed, wT: [k, n] (a backward pass runs the operators on W^T and passes W as
 * it is stored; no copy is made). */
ncclResult_t dfcclRunFusedGemmT(int collId, const void* x, const void* wT, void* out, cudaStream_t stream, ofcclRankCtx_t rankCtx);

/* By default dfcclStreamWait (outside a stream capture) launches an instance of the daemon before the wait and
 * keeps it resident until nothing is outstanding, so that a stream parked on a completion never depends on a
 * relaunch from a host thread - the safe choice for eager steps of thousands of launches, at the price of the
 * daemon's SMs from the moment the host enqueues the wait.  A step that is enqueued with a handful of calls
 * (a replayed CUDA graph) can switch it off and leave the wake-up to the poller. */
ncclResult_t dfcclSetHoldOnWait(ofcclRankCtx_t rankCtx, int on);

/* Host-side wait for the last submission of collId (status of that execution is returned). */
ncclResult_t dfcclWait(int collId, int timeoutMs, ofcclRankCtx_t rankCtx);
ncclResult_t dfcclWaitAll(int timeoutMs, ofcclRankCtx_t rankCtx);

/* Abort: every block of the daemon leaves at its next poll; pending callbacks are
 * dropped; the context can only be destroyed afterwards. */
ncclResult_t dfcclAbort(ofcclRankCtx_t rankCtx);
ncclResult_t dfcclGetAsyncError(ofcclRankCtx_t rankCtx, ncclResult_t* asyncError);

/* Counters (device counters are summed over blocks when the daemon parks or exits,
 * so they lag a running daemon by at most one idle period). */
typedef struct {
  uint64_t sqesSubmitted, cqesDelivered, callbacksRun;
  uint64_t daemonLaunches, daemonVoluntaryQuits;
  uint64_t ctxSwitches, ctxSaves, ctxLoads;       /* preemptions / parked cursors written / read */
  uint64_t waitPolls, waitTimeouts;
  uint64_t bytesReduced, bytesCopied;
  uint64_t sqFullRetries;
  uint64_t maxSwitchNs, totalSwitchNs;            /* measured cost of one preemption on the device */
  uint64_t deviceEvents;                          /* entries drained from the device trace ring */
  uint64_t dataYields;                            /* data phases left at a slice boundary for other queued work */
  uint64_t schedulerPasses;                       /* passes of the per-block scheduler loop, summed over blocks */
  uint64_t nsTriggers, nsWalk, nsQueues;          /* time of those passes by part: trigger list, task-queue walk, queue upkeep */
  uint64_t fusedLaunches;                         /* registered fused GEMM + collective operators launched */
} dfcclStats;
ncclResult_t dfcclGetStats(ofcclRankCtx_t rankCtx, dfcclStats* stats);
/* Host-memory counters only (submissions, completions, launches, quits; deviceEvents = daemon believed alive):
 * never touches the device, so it answers while the GPU is busy or stuck. */
ncclResult_t dfcclGetHostStats(ofcclRankCtx_t rankCtx, dfcclStats* stats);

/* Device trace ring: (globaltimer ns, block, collId, event) tuples written by the
 * daemon when DFCCL_TRACE=1; drained by the poller into a Chrome-trace JSON file. */
ncclResult_t dfcclTraceDump(ofcclRankCtx_t rankCtx, const char* path);

/* Fault injection on the HOST side only (tests): nothing here faults a GPU. */
typedef enum {
  dfcclFaultNone = 0,
  dfcclFaultDropSqe = 1,     /* the next `arg` submissions are accepted but never reach the device */
  dfcclFaultDelaySqeUs = 2,  /* delay every submission by `arg` microseconds */
  dfcclFaultFreezePoller = 3 /* poller thread sleeps `arg` milliseconds before each callback */
} dfcclFault_t;
ncclResult_t dfcclInjectFault(ofcclRankCtx_t rankCtx, dfcclFault_t fault, int64_t arg);

#ifdef __cplusplus
}
#endif
#endif /* DFCCL_H_ */
