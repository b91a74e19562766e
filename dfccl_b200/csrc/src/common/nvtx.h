// NVTX ranges around the host-side entry points (visible in Nsight Systems timelines).  Header-only
// NVTX v3: with no tool attached a range costs a couple of predictable branches.  DFCCL_NVTX=0 turns
// them off entirely.  Role of the reference's NVTX=1 build switch (reference: makefiles/common.mk:14,
// src/include/nvtx.h).
#pragma once
#include <nvtx3/nvToolsExt.h>
#include "param.h"

namespace dfccl {

inline bool nvtxOn() {
  // NVTX binds to an attached tool lazily at the first call and does so without synchronisation; making that
  // first call here, under the guard of the static initialiser, keeps it to one thread
  static const bool on = [] {
    const bool v = paramI64("NVTX", 1) != 0;
    if (v) { nvtxRangePushA("dfccl:init"); nvtxRangePop(); }
    return v;
  }();
  return on;
}

struct NvtxRange {
  bool live;
  explicit NvtxRange(const char* name) : live(nvtxOn()) { if (live) nvtxRangePushA(name); }
  ~NvtxRange() { if (live) nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

}  // namespace dfccl
