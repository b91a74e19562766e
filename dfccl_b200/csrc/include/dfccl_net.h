/* Network transport interface of dfccl-b200 (version 1).
 *
 * Communicators whose members cannot map each other's memory (different hosts, or DFCCL_FORCE_NET=1)
 * move their data through an implementation of this table: point-to-point, connection oriented,
 * asynchronous sends and receives that are matched in posting order per connection.  A built-in TCP
 * implementation is always present; an external one is loaded from the shared object named by
 * DFCCL_NET_PLUGIN (default "libdfccl-net.so") when it exports a `dfcclNetPlugin_v1` table whose
 * init() succeeds and whose devices() reports at least one device.
 *
 * Role of the reference's external network plugin interface (reference: src/include/nccl_net.h,
 * ext-net/dummy/plugin.c); the shape is kept (listen / connect / accept handles of fixed size,
 * isend / irecv / test), memory registration and device offload are left out: buffers are host memory. */
#ifndef DFCCL_NET_H_
#define DFCCL_NET_H_
#include <stddef.h>

/* Return values are ncclResult_t codes (0 = success) carried as int, so that a plugin needs no other header. */
typedef int dfcclNetResult_t;

#ifdef __cplusplus
extern "C" {
#endif

#define DFCCL_NET_HANDLE_BYTES 128

typedef struct {
  const char* name;   /* interface or device name */
  int speedMbps;
  int maxComms;
} dfcclNetProperties_v1_t;

typedef struct {
  const char* name;
  dfcclNetResult_t (*init)(void);
  dfcclNetResult_t (*devices)(int* ndev);
  dfcclNetResult_t (*getProperties)(int dev, dfcclNetProperties_v1_t* props);
  /* Create a receiving endpoint; `handle` (DFCCL_NET_HANDLE_BYTES) is shipped to the sender out of band. */
  dfcclNetResult_t (*listen)(int dev, void* handle, void** listenComm);
  dfcclNetResult_t (*connect)(int dev, const void* handle, void** sendComm);
  dfcclNetResult_t (*accept)(void* listenComm, void** recvComm);
  /* Asynchronous; the buffer stays untouched by the caller until test() reports done. */
  dfcclNetResult_t (*isend)(void* sendComm, const void* data, size_t bytes, void** request);
  dfcclNetResult_t (*irecv)(void* recvComm, void* data, size_t bytes, void** request);
  dfcclNetResult_t (*test)(void* request, int* done, size_t* bytes);   /* frees the request once done */
  dfcclNetResult_t (*closeSend)(void* sendComm);
  dfcclNetResult_t (*closeRecv)(void* recvComm);
  dfcclNetResult_t (*closeListen)(void* listenComm);
} dfcclNet_v1_t;

#ifdef __cplusplus
}
#endif
#endif
