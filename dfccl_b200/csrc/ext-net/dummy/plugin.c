/* Smallest possible external network plugin: it loads, initialises and reports no device, so the
 * library falls back to its built-in TCP transport.  Build:
 *     gcc -shared -fPIC -I../../include plugin.c -o libdfccl-net.so
 * Same purpose as the reference's ext-net/dummy/plugin.c. */
#include "dfccl_net.h"

static dfcclNetResult_t p_init(void) { return 0; }
static dfcclNetResult_t p_devices(int* n) { *n = 0; return 0; }
static dfcclNetResult_t p_props(int dev, dfcclNetProperties_v1_t* p) { (void)dev; (void)p; return 3; }
static dfcclNetResult_t p_listen(int dev, void* h, void** c) { (void)dev; (void)h; (void)c; return 3; }
static dfcclNetResult_t p_connect(int dev, const void* h, void** c) { (void)dev; (void)h; (void)c; return 3; }
static dfcclNetResult_t p_accept(void* l, void** c) { (void)l; (void)c; return 3; }
static dfcclNetResult_t p_isend(void* c, const void* d, size_t n, void** r) { (void)c; (void)d; (void)n; (void)r; return 3; }
static dfcclNetResult_t p_irecv(void* c, void* d, size_t n, void** r) { (void)c; (void)d; (void)n; (void)r; return 3; }
static dfcclNetResult_t p_test(void* r, int* done, size_t* n) { (void)r; (void)done; (void)n; return 3; }
static dfcclNetResult_t p_close(void* c) { (void)c; return 3; }

dfcclNet_v1_t dfcclNetPlugin_v1 = {
  "dummy", p_init, p_devices, p_props, p_listen, p_connect, p_accept, p_isend, p_irecv, p_test, p_close, p_close, p_close
};
