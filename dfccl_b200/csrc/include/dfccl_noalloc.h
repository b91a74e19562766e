/* dfccl_noalloc.h - a collective entry point that never allocates.
 *
 * This call has no counterpart in the reference library; it is an addition of this
 * library.
 *
 * Who it is for.  Every other entry point of the library may allocate: communicators
 * take a symmetric heap, buffers that are not part of that heap are staged through
 * scratch memory that grows on demand, launch tables come from cudaMalloc.  Some
 * callers cannot afford that:
 *   - code that runs inside a process whose device memory is already spoken for - a
 *     framework's caching allocator that has reserved the whole GPU, a job under a
 *     hard memory quota - where one more cudaMalloc simply fails;
 *   - latency-critical loops (serving, control) in which the device-wide
 *     synchronisation that cudaMalloc / cudaFree imply is not acceptable;
 *   - callbacks of other libraries in which allocating is forbidden by contract.
 * For them this header offers the single-GPU all-reduce with a pre-multiplied sum -
 * out[i] = scale * in[i], the collective a one-rank data-parallel job runs on its
 * gradients - executed by the same step engine as ncclAllReduce, with every byte of
 * scratch (control words, per-block state, both staging areas) placed in one
 * file-scope device array that is part of the library image.
 *
 * Cost and limit.  The array is DFCCL_NOALLOC_SCRATCH_BYTES (16 MiB + 64 KiB) and every
 * GPU that loads the library holds it until the process exits.  One call moves at most
 * DFCCL_NOALLOC_MAX_BYTES (8 MiB) of payload; a larger request is rejected with
 * ncclInvalidArgument and nothing is launched.
 *
 * Rules.
 *   - The first call on a device looks up the array's device address, clears its
 *     control words, writes the kernel's control block (synchronous copies, no
 *     allocation) and waits for the device once, so that the block is in place whatever
 *     stream the kernel runs on.  Make that first call before any stream capture is begun.
 *   - All calls on a device share the array, and it keeps whatever the previous call
 *     left: each call overwrites the staging bytes it uses before reading them, and
 *     the set-up clears the words that must start at zero.  Two calls that overlap on
 *     the GPU (different streams, no ordering between them) race on the staging areas;
 *     order them.
 *   - sendbuff and recvbuff are ordinary device pointers supplied by the caller, 
 *     `count` elements of `datatype` each; they may be the same pointer.
 */
#ifndef DFCCL_NOALLOC_H_
#define DFCCL_NOALLOC_H_

#include "dfccl.h"

#define DFCCL_NOALLOC_MAX_BYTES (8u << 20)
#define DFCCL_NOALLOC_SCRATCH_BYTES ((16u << 20) + (64u << 10))

#ifdef __cplusplus
extern "C" {
#endif

/* recvbuff[i] = scale * sendbuff[i] for i < count, on the current device, enqueued on `stream`.
 * Integer datatypes truncate the scaled value toward zero.  Returns ncclInvalidArgument for a
 * null buffer, an unknown datatype or more than DFCCL_NOALLOC_MAX_BYTES of payload. */
ncclResult_t dfcclAllReduceNoAlloc(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype,
                                   float scale, cudaStream_t stream);

/* 0, or the failure code of the first kernel of dfcclAllReduceNoAlloc that gave up on the current device (1 = a wait
 * ran out, 2 = aborted, 3 = no kernel for the datatype).  The kernels leave it in the static array; this call copies
 * four bytes back (synchronously, allocating nothing) and covers the kernels that have finished by then. */
ncclResult_t dfcclNoAllocStatus(uint32_t* status);

#ifdef __cplusplus
}
#endif
#endif /* DFCCL_NOALLOC_H_ */
