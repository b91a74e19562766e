#pragma once
#include "../comm/comm.h"
namespace dfccl {
// Queue one send or receive of the calling thread's open group (or of an implicit group of one).
ncclResult_t p2pEnqueue(ncclComm* comm, bool isSend, void* buf, size_t count, ncclDataType_t type, int peer, cudaStream_t stream);
// Launch everything queued by this thread, one kernel per (communicator, stream).
ncclResult_t p2pFlush();
}  // namespace dfccl
