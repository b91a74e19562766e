// Point-to-point transfers (ncclSend / ncclRecv): the sender pushes straight into
// the receiver's buffer once the receiver has published where that buffer is.
// All operations of one group run in ONE kernel so that a rank's sends and
// receives progress side by side (reference behaviour: grouped send/recv fused
// into one launch, src/collectives/device/sendrecv.h:13-75, src/group.cc:236-311).
// Block layout: one block per (operation list, channel); a list holds the sends
// to one peer or the receives from one peer, in program order.
#pragma once
#include "datapath.h"
#include "platform.h"
#include "types.h"

#define DF_P2P_CHANNELS 8
#define DF_P2P_MAX_OPS 24

namespace dfccl {

struct P2pOp {
  uint64_t buf;          // local address of the user buffer
  uint64_t bytes;
  uint64_t stagingOff;   // receiver: heap offset peers write to when the user buffer is outside the heap (else the buffer's own offset)
  uint32_t seq;
  uint32_t staged;
};
struct P2pList {
  int32_t isSend, peer, nOps, channels;
  FlagSlot* mine;        // [DF_P2P_CHANNELS] slots the peer writes (in my heap)
  FlagSlot* theirs;      // [DF_P2P_CHANNELS] slots I write (in the peer's heap)
  char* peerHeap;
  char* myHeap;
  P2pOp ops[DF_P2P_MAX_OPS];
};
struct P2pShared { DataArgs args; int32_t ok; uint64_t off; };

DF_HD bool p2pWait(P2pShared* sh, RankDev* rd, const volatile uint64_t* word, uint64_t want) {
  if (df_tid() == 0) {
    uint64_t t0 = df_now_ns();
    uint32_t spins = 0;
    int ok = 1;
    while (ld_acquire_sys_u64(word) < want) {
      if ((++spins & 255) == 0) {
        if (ctl_load(&rd->ctl->abortFlag)) { ok = 0; rd->ctl->pad = ST_ABORTED; break; }
        if (rd->waitTimeoutNs && df_now_ns() - t0 > rd->waitTimeoutNs) { ok = 0; rd->ctl->pad = ST_TIMEOUT; break; }
      }
    }
    sh->ok = ok;
  }
  df_sync();
  return sh->ok != 0;
}

DF_HD void p2pBlockMain(RankDev* rd, const P2pList* l, int chan, P2pShared* sh) {
  if (chan >= l->channels) return;
  for (int i = 0; i < l->nOps; ++i) {
    const P2pOp* op = &l->ops[i];
    uint64_t per = (op->bytes + l->channels - 1) / l->channels;
    per = (per + 15) & ~15ull;
    uint64_t beg = per * chan < op->bytes ? per * chan : op->bytes;
    uint64_t end = beg + per < op->bytes ? beg + per : op->bytes;
    if (l->isSend) {
      if (!p2pWait(sh, rd, &l->mine[chan].arrive, op->seq)) return;
      if (df_tid() == 0) {
        sh->args.nsrc = 1; sh->args.ndst = 1; sh->args.n = end - beg;
        sh->args.src[0] = (const char*)op->buf + beg;
        sh->args.dst[0] = l->peerHeap + ld_relaxed_sys_u64(&l->mine[chan].recvOff) + beg;
      }
      df_sync();
      if (end > beg) copy_multi(&sh->args);
      df_sync();
      if (df_tid() == 0) { fence_sys(); st_release_sys_u64(&l->theirs[chan].done, op->seq); }
    } else {
      if (df_tid() == 0) {
        st_relaxed_sys_u64(&l->theirs[chan].recvOff, op->stagingOff);
        st_release_sys_u64(&l->theirs[chan].arrive, op->seq);
      }
      if (!p2pWait(sh, rd, &l->mine[chan].done, op->seq)) return;
      if (op->staged) {
        if (df_tid() == 0) {
          sh->args.nsrc = 1; sh->args.ndst = 1; sh->args.n = end - beg;
          sh->args.src[0] = l->myHeap + op->stagingOff + beg;
          sh->args.dst[0] = (char*)op->buf + beg;
        }
        df_sync();
        if (end > beg) copy_multi(&sh->args);
        df_sync();
      }
    }
  }
}

}  // namespace dfccl
