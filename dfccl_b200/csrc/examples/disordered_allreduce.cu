// Register-then-submit in C: every GPU of this process registers the same four all-reduces and then
// submits them in ITS OWN order; an in-order library would deadlock, here every callback fires.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -I ../include disordered_allreduce.cu \
//        -L ../build-make/lib -ldfccl -o disordered_allreduce && ./disordered_allreduce
//
// Same call sequence as a user of the reference writes (reference: src/nccl.h.in:318-333).
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>
#include "dfccl.h"

#define CHECK(x) do { ncclResult_t r_ = (x); if (r_ != ncclSuccess) { fprintf(stderr, "%s failed: %s\n", #x, ncclGetErrorString(r_)); exit(1); } } while (0)

static std::atomic<int> g_done{0};
static int onDone(int collId, void* args) { (void)collId; (void)args; g_done++; return 0; }

int main() {
  int ndev = 0;
  cudaGetDeviceCount(&ndev);
  if (ndev < 2) { printf("needs two GPUs\n"); return 0; }
  ndev = ndev > 4 ? 4 : ndev;
  const int kColls = 4;
  const size_t count = 1 << 20;
  std::vector<ncclComm_t> comms(ndev);
  CHECK(ncclCommInitAll(comms.data(), ndev, nullptr));
  std::vector<std::thread> ranks;
  for (int r = 0; r < ndev; ++r) ranks.emplace_back([&, r] {
    cudaSetDevice(r);
    ofcclRankCtx_t ctx;
    CHECK(ofcclInitRankCtx(&ctx, r));
    for (int c = 0; c < kColls; ++c) CHECK(ofcclPrepareAllReduce(count, ncclFloat, ncclSum, comms[r], c, ctx));
    CHECK(ofcclFinalizeRankCtx7StartHostThrds(ctx));
    std::vector<float*> in(kColls), out(kColls);
    for (int c = 0; c < kColls; ++c) {
      CHECK(dfcclMemAlloc((void**)&in[c], count * sizeof(float), comms[r]));     // symmetric heap: zero-copy path
      CHECK(dfcclMemAlloc((void**)&out[c], count * sizeof(float), comms[r]));
      std::vector<float> h(count, (float)(r + 1));
      cudaMemcpy(in[c], h.data(), count * sizeof(float), cudaMemcpyHostToDevice);
    }
    for (int k = 0; k < kColls; ++k) {
      const int c = (k + r) % kColls;                      // a different order on every rank
      CHECK(ofcclRunAllReduce(in[c], out[c], c, onDone, nullptr, ctx));
    }
    CHECK(dfcclWaitAll(60000, ctx));
    float first = 0.f;
    cudaMemcpy(&first, out[0], sizeof(float), cudaMemcpyDeviceToHost);
    printf("rank %d: out[0][0] = %.0f (expected %d)\n", r, first, ndev * (ndev + 1) / 2);
    CHECK(ofcclDestroy(ctx));
  });
  for (auto& t : ranks) t.join();
  for (auto c : comms) ncclCommDestroy(c);
  printf("%d callbacks\n", g_done.load());
  return g_done.load() == ndev * kColls ? 0 : 1;
}
