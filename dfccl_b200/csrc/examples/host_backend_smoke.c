/* Register-then-submit in plain C on the host backend (no GPU needed): three "ranks" played by threads of this
 * process register the same all-reduces and submit them each in its own order.  Used by the packaging test to check
 * that the static archive links from a C program and runs:
 *
 *   nvcc -x c host_backend_smoke.c -I ../include -L ../build-make/lib -ldfccl_static -lpthread -ldl -lrt -o smoke && ./smoke
 *
 * Same call sequence as a user of the reference writes (reference: src/nccl.h.in:318-333). */
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include "dfccl.h"

#define RANKS 3
#define COLLS 4
#define COUNT 5003

#define CHECK(x) do { ncclResult_t r_ = (x); if (r_ != ncclSuccess) { fprintf(stderr, "%s failed: %s\n", #x, ncclGetErrorString(r_)); exit(1); } } while (0)

static ncclComm_t comms[RANKS];
static int callbacks[RANKS];
static int bad[RANKS];

static int onDone(int collId, void* args) { (void)collId; ++*(int*)args; return 0; }

static void* rankMain(void* arg) {
  const int r = (int)(long)arg;
  ofcclRankCtx_t ctx;
  float *in[COLLS], *out[COLLS];
  CHECK(ofcclInitRankCtx(&ctx, r));
  for (int c = 0; c < COLLS; ++c) CHECK(ofcclPrepareAllReduce(COUNT, ncclFloat, ncclSum, comms[r], c, ctx));
  CHECK(ofcclFinalizeRankCtx7StartHostThrds(ctx));
  for (int c = 0; c < COLLS; ++c) {
    CHECK(dfcclMemAlloc((void**)&in[c], COUNT * sizeof(float), comms[r]));
    CHECK(dfcclMemAlloc((void**)&out[c], COUNT * sizeof(float), comms[r]));
    for (int i = 0; i < COUNT; ++i) in[c][i] = (float)(r + 1 + c);
  }
  for (int k = 0; k < COLLS; ++k) {
    const int c = (k + r) % COLLS;                          /* a different order on every rank */
    CHECK(ofcclRunAllReduce(in[c], out[c], c, onDone, &callbacks[r], ctx));
  }
  CHECK(dfcclWaitAll(60000, ctx));
  for (int c = 0; c < COLLS; ++c)
    for (int i = 0; i < COUNT; ++i)
      if (out[c][i] != (float)(RANKS * (RANKS + 1) / 2 + RANKS * c)) { bad[r] = 1; break; }
  CHECK(ofcclDestroy(ctx));
  return NULL;
}

int main(void) {
  pthread_t th[RANKS];
  CHECK(dfcclSetBackend(dfcclBackendHost));
  CHECK(dfcclCommInitLoopback(comms, RANKS, -1));
  for (long r = 0; r < RANKS; ++r) pthread_create(&th[r], NULL, rankMain, (void*)r);
  for (int r = 0; r < RANKS; ++r) pthread_join(th[r], NULL);
  int total = 0, wrong = 0;
  for (int r = 0; r < RANKS; ++r) { total += callbacks[r]; wrong += bad[r]; ncclCommDestroy(comms[r]); }
  printf("%d callbacks, %d ranks with wrong results\n", total, wrong);
  return total == RANKS * COLLS && wrong == 0 ? 0 : 1;
}
