// Host twin of the device runtime: every "thread block" is one OS thread that runs
// the very same scheduler / engine / data-path code compiled for the host.  Used by
// the host backend (tests without a GPU) - the protocol, the queues, preemption and
// the quit / relaunch handshake are exercised exactly as on the device.
#include "../device/daemon_impl.h"
#include "../device/launch.h"
#include <memory>
#include <thread>
#include <vector>

namespace dfccl {

void runDaemonHost(RankDev** rankTable, int nRanks, int blocksPerRank) {
  std::vector<std::thread> ts;
  for (int r = 0; r < nRanks; ++r)
    for (int b = 0; b < blocksPerRank; ++b)
      ts.emplace_back([=] {
        std::unique_ptr<BlockShared> sh(new BlockShared());
        daemonBlockMain(rankTable[r], b, sh.get());
      });
  for (auto& t : ts) t.join();
}

void runStandaloneHost(RankDev* rd, const CollStatic& cs, uint64_t send, uint64_t recv, uint32_t epoch, uint32_t sqeFlags) {
  std::vector<std::thread> ts;
  for (int b = 0; b < cs.nBlocks; ++b)
    ts.emplace_back([=, &cs] {
      std::unique_ptr<BlockShared> sh(new BlockShared());
      standaloneBlockMain(rd, b, sh.get(), &cs, send, recv, epoch, sqeFlags);
    });
  for (auto& t : ts) t.join();
}

}  // namespace dfccl
