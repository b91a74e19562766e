// Step engine: one registered collective, executed by one block, as a resumable
// sequence of phases (types.h: Phase).  Two kinds of phases exist:
//   * bounded waits (PH_TRIGGER, PH_WAIT_ARRIVE, PH_WAIT_DONE) poll words in LOCAL
//     memory that a peer, the host or a stream memory operation writes.  A wait
//     that runs out of budget returns to the scheduler without side effects: it
//     consumed nothing and wrote nothing, so parking the collective is saving
//     (phase, cursor) - there is no connection state to unwind.
//   * actions (posting flags, moving data) never wait for anybody.
// This replaces the reference's preemptible ring primitives, where a context
// switch had to unwind a half-executed slice and re-synchronise every thread role
// (src/collectives_ofccl/device/ofccl_prims_simple.h:118-140,217-491 and the
// resumable ring loops in ofccl_all_reduce.h:44-217): on an NVSwitch fabric every
// peer is one hop away, so each collective is "everybody arrived -> direct loads
// and stores of peer buffers -> everybody done" and the only blocking points are
// the two rendezvous.
//
// Schedules (kind x algo), all expressed as N-source / M-destination reduce-copy
// (plus the push schedule of small all-reduces: inputs are written into slots at the peers together with the arrival
// flag, every rank reduces locally and is done - one NVLink hop, no staging, no done handshake):
//   AllReduce two-shot  : block b, rank r owns shard r of slice b: reads it from all
//                         ranks, reduces, scales, casts, writes it to all ranks.
//   AllReduce one-shot  : every rank reads slice b from all ranks, writes only itself.
//   AllGather           : rank r pushes its slice b into every rank's output.
//   ReduceScatter       : rank r reads slice b of chunk r from all ranks.
//   Broadcast           : non-roots pull slice b from the root.
//   Reduce              : like two-shot AllReduce, but shards are written to the root only.
#pragma once
#include "datapath.h"
#include "nvls.h"
#include "platform.h"
#include "types.h"
namespace dfccl {

enum RunResult : int { RC_DONE = 0, RC_STALLED = 1, RC_YIELD = 2 };

struct BlockShared {
  CollStatic cs;                 // static context of the loaded collective
  CollDyn dyn;                   // its dynamic context (authoritative copy while loaded)
  DataArgs args;
  int32_t loadedColl;            // -1 = nothing loaded
  int32_t standalone;            // 1 = stream-ordered kernel: no queues, completion is the kernel's end
  int32_t dynDirty;
  int32_t waitOk;
  uint32_t waitSpins;
  int32_t ctl0, ctl1;
  uint64_t ctl64;
  DevStats stats;
  uint64_t frontier;
  uint32_t nActive;
  uint32_t quit;                 // 1 = voluntary, 2 = final, 3 = abort
  uint32_t abortSeen;            // the host's abort flag as last read by thread 0 (the flag lives in host memory: one
                                 // read costs a PCIe round trip, so it is sampled once per scheduler pass, not per wait)
  // peers' buffer offsets of the running submission, fetched by one lane per peer (one memory round trip for all)
  uint64_t peerSend[DF_MAX_RANKS], peerRecv[DF_MAX_RANKS];
  // stream-ordered submissions not yet released by their stream: polled all at once, one thread per entry,
  // without loading any context; a released one joins the task queue
  uint32_t nTrig;
  uint32_t trigFired;
  uint16_t active[DF_MAX_ACTIVE];
  // per task-queue entry: 0 = needs a visit, 1 = parked in the wait for the peers' arrival, 2 = parked in the wait for
  // their done flags.  Parked entries are not visited (a visit loads the context and polls for a while); their flag
  // words are looked at by one thread each in a scan over the whole queue, which marks the ready ones for a visit.
  uint8_t actWait[DF_MAX_ACTIVE];
  uint32_t nReady;
  uint32_t ctl1Full;               // this pass visits parked entries too (set by thread 0 at the end of the previous pass)
  uint16_t trigColl[DF_MAX_ACTIVE];
  uint32_t trigVal[DF_MAX_ACTIVE];  // low 32 bits of the value the trigger word must reach
};

DF_HD void trace(RankDev* rd, int b, uint16_t ev, int coll) {
  if (rd->trace == nullptr) return;
  unsigned long long i = atomic_add_u64((unsigned long long*)&rd->traceHead, 1ull);
  TraceEvent* e = &rd->trace[i & (rd->traceCap - 1)];
  e->ns = df_now_ns(); e->block = (uint16_t)b; e->event = ev; e->collId = coll;
}

DF_HD uint64_t umin64(uint64_t a, uint64_t b) { return a < b ? a : b; }

DF_HD bool abortRequested(const RankDev* rd) {
  return ctl_load(rd->abortWord ? rd->abortWord : &rd->ctl->abortFlag) != 0;
}

// [beg,end) of part idx when [0,total) is cut into nparts pieces on `align` boundaries
DF_HD void partRange(uint64_t total, int nparts, int idx, uint64_t align, uint64_t* beg, uint64_t* end) {
  uint64_t per = (total + nparts - 1) / nparts;
  per = (per + align - 1) / align * align;
  *beg = umin64(total, per * (uint64_t)idx);
  *end = umin64(total, *beg + per);
}

// bytes of the user's send / recv buffer (staging copies)
DF_HD uint64_t sendBytes(const CollStatic* c) {
  uint64_t e = dtypeSize(c->inType);
  switch (c->kind) {
    case dfcclCollReduceScatter: return c->count * c->nranks * e;
    default: return c->count * e;
  }
}
DF_HD uint64_t recvBytes(const CollStatic* c) {
  uint64_t e = dtypeSize(c->outType);
  switch (c->kind) {
    case dfcclCollAllGather: return c->count * c->nranks * e;
    default: return c->count * e;
  }
}

// Relative index of daemon block b in collective c (>= c->nBlocks: b takes no part).  Flags, data partitions and
// staging partitions are indexed by it; per-block state (saved contexts, statistics, trace) by the block itself.
DF_HD int relBlock(const RankDev* rd, const CollStatic* c, int b) {
  const int r = b - c->blockBase;
  return r < 0 ? r + (int)rd->nBlocks : r;
}

// ---- context switch: load / save the (static, dynamic) context of a collective
DF_HD void loadColl(BlockShared* sh, RankDev* rd, int b, int coll) {
  if (sh->loadedColl == coll) return;
  const int tid = df_tid(), nt = df_nthreads();
  uint64_t t0 = 0;
  if (tid == 0) t0 = df_now_ns();
  if (sh->loadedColl >= 0 && sh->dynDirty) {           // park the previous one
    CollDyn* g = &rd->dyn[(uint64_t)b * rd->maxColls + sh->loadedColl];
    const uint4* s = (const uint4*)&sh->dyn;
    for (int i = tid; i < (int)(sizeof(CollDyn) / 16); i += nt) ((uint4*)g)[i] = s[i];
    if (tid == 0) sh->stats.ctxSaves++;
  }
  df_sync();
  {
    const uint4* s = (const uint4*)&rd->colls[coll];
    uint4* d = (uint4*)&sh->cs;
    for (int i = tid; i < (int)(sizeof(CollStatic) / 16); i += nt) d[i] = s[i];
    const uint4* sd = (const uint4*)&rd->dyn[(uint64_t)b * rd->maxColls + coll];
    uint4* dd = (uint4*)&sh->dyn;
    for (int i = tid; i < (int)(sizeof(CollDyn) / 16); i += nt) dd[i] = sd[i];
  }
  if (tid == 0) {
    if (sh->loadedColl >= 0) {
      sh->stats.ctxSwitches++;
      uint64_t dt = df_now_ns() - t0;
      sh->stats.totalSwitchNs += dt;
      if (dt > sh->stats.maxSwitchNs) sh->stats.maxSwitchNs = dt;
    }
    sh->stats.ctxLoads++;
    sh->loadedColl = coll;
    sh->dynDirty = 0;
  }
  df_sync();
}

DF_HD void saveLoaded(BlockShared* sh, RankDev* rd, int b) {
  if (sh->loadedColl >= 0 && sh->dynDirty && df_tid() == 0) {
    rd->dyn[(uint64_t)b * rd->maxColls + sh->loadedColl] = sh->dyn;
    sh->stats.ctxSaves++;
    sh->dynDirty = 0;
  }
}

DF_HD void setPhase(BlockShared* sh, int phase) {
  df_sync();                                   // everybody is done reading the old phase
  if (df_tid() == 0) { sh->dyn.phase = phase; sh->dyn.cursor = 0; sh->dyn.stallSinceNs = 0; sh->dynDirty = 1; }
  df_sync();
}

// ---- bounded waits (first warp polls, everybody learns the outcome)
// which: 0 = arrive flags, 1 = done flags, 2 = local trigger word
DF_HD bool boundedWait(BlockShared* sh, RankDev* rd, int b, int which, uint32_t budget) {
  if (df_tid() < df_warpsize()) {
    const int lane = df_lane(), ws = df_warpsize();
    const int n = sh->cs.nranks, me = sh->cs.rank;
    const uint64_t epoch = sh->dyn.epoch;
    FlagSlot* mine = sh->cs.myFlags + (uint64_t)b * n;
    uint32_t spins = 0;
    bool ok;
    for (;;) {
      bool laneOk = true;
      if (which == 2) {
        if (lane == 0) laneOk = ld_relaxed_sys_u64(&rd->trigger[sh->loadedColl]) >= sh->dyn.trigger;
      } else {
        for (int j = lane; j < n; j += ws) {
          if (j == me) continue;
          uint64_t v = ld_relaxed_sys_u64(which == 0 ? &mine[j].arrive : &mine[j].done);
          laneOk = laneOk && v >= epoch;
        }
      }
      bool laneStop = false;
      if ((spins & 255) == 255 && lane == 0) laneStop = abortRequested(rd);
      ok = df_warp_all(laneOk);
      const bool stop = !df_warp_all(!laneStop);      // uniform: every lane leaves the loop together
      ++spins;
      if (ok || stop || spins >= budget) break;
    }
    // polls are relaxed loads (an acquire at system scope per poll costs a fence each time); the one
    // fence that orders the payload accesses after the flags is paid when the wait succeeds
    if (ok && lane == 0) fence_sys();
    if (lane == 0) { sh->waitOk = ok ? 1 : 0; sh->waitSpins = spins; sh->stats.waitPolls += spins; }
  }
  df_sync();
  return sh->waitOk != 0;
}

// Called by all threads when a wait ran out.  Returns true if the collective must fail now.
DF_HD bool noteStall(BlockShared* sh, RankDev* rd) {
  if (df_tid() == 0) {
    uint64_t now = df_now_ns();
    sh->ctl0 = 0;
    if (sh->standalone ? abortRequested(rd) : (sh->abortSeen != 0)) { sh->dyn.status = ST_ABORTED; sh->ctl0 = 1; }
    else if (sh->dyn.stallSinceNs == 0) { sh->dyn.stallSinceNs = now; sh->dynDirty = 1; }
    else if (rd->waitTimeoutNs && now - sh->dyn.stallSinceNs > rd->waitTimeoutNs) {
      sh->dyn.status = ST_TIMEOUT; sh->ctl0 = 1; sh->stats.waitTimeouts++;
    }
  }
  df_sync();
  return sh->ctl0 != 0;
}

DF_HD uint64_t mySendOff(const BlockShared* sh) {
  return (sh->dyn.sqeFlags & SQE_SEND_STAGED) ? sh->cs.stagingSendOff : sh->dyn.send;
}
DF_HD uint64_t myRecvOff(const BlockShared* sh) {
  return (sh->dyn.sqeFlags & SQE_RECV_STAGED) ? sh->cs.stagingRecvOff : sh->dyn.recv;
}
// Offsets the peers posted with their arrival, one lane per peer; everybody calls it, ends with a barrier.
DF_HD void fetchPeerOffsets(BlockShared* sh, int b) {
  const CollStatic* c = &sh->cs;
  const int n = c->nranks, j = df_tid();
  if (j < n) {
    const FlagSlot* f = &c->myFlags[(uint64_t)b * n + j];
    sh->peerSend[j] = j == c->rank ? mySendOff(sh) : ld_relaxed_sys_u64(&f->sendOff);
    sh->peerRecv[j] = j == c->rank ? myRecvOff(sh) : ld_relaxed_sys_u64(&f->recvOff);
  }
#if !DF_DEVICE_CODE
  for (int k = 1; k < n; ++k) {                  // one host thread plays the whole block
    const FlagSlot* f = &c->myFlags[(uint64_t)b * n + k];
    sh->peerSend[k] = k == c->rank ? mySendOff(sh) : ld_relaxed_sys_u64(&f->sendOff);
    sh->peerRecv[k] = k == c->rank ? myRecvOff(sh) : ld_relaxed_sys_u64(&f->recvOff);
  }
#endif
  df_sync();
}
DF_HD const char* sendPtrOf(const BlockShared* sh, int j) { return sh->cs.peerHeap[j] + sh->peerSend[j]; }
DF_HD char* recvPtrOf(const BlockShared* sh, int j) { return sh->cs.peerHeap[j] + sh->peerRecv[j]; }

// Schedules in which a user buffer is touched by this rank only use it where it is (no staging copy even when it
// lies outside the symmetric heap): both buffers of the push schedule, the input of a multimem all-gather or
// broadcast, the output of a multimem reduce-scatter.
DF_HD bool rawSend(const CollStatic* c) {
  return c->algo == dfcclAlgoPush || (c->algo == dfcclAlgoNvls && (c->kind == dfcclCollAllGather || c->kind == dfcclCollBroadcast));
}
DF_HD bool rawRecv(const CollStatic* c) { return c->algo == dfcclAlgoPush || (c->algo == dfcclAlgoNvls && c->kind == dfcclCollReduceScatter); }

// Push schedule: the user's buffers are only touched by this rank, so they are used where they are.
DF_HD const char* pushSendPtr(const BlockShared* sh) {
  return (sh->dyn.sqeFlags & SQE_SEND_STAGED) ? (const char*)(uintptr_t)sh->dyn.send : sh->cs.peerHeap[sh->cs.rank] + sh->dyn.send;
}
DF_HD char* pushRecvPtr(const BlockShared* sh) {
  return (sh->dyn.sqeFlags & SQE_RECV_STAGED) ? (char*)(uintptr_t)sh->dyn.recv : sh->cs.peerHeap[sh->cs.rank] + sh->dyn.recv;
}
// slot that `writer` fills at member `owner` for this epoch's parity
DF_HD char* pushSlot(const BlockShared* sh, int owner, int writer) {
  const CollStatic* c = &sh->cs;
  return c->peerPush[owner] + ((uint64_t)(sh->dyn.epoch & 1u) * c->nranks + writer) * c->pushSlotBytes;
}
// Push schedule, outgoing half: what the peers need of my input goes into my slot at each of them (block b moves its
// part of the range).  All-reduce: the whole input to everybody.  All-gather: my piece to everybody.
// Reduce-scatter: chunk j of my input to member j.
DF_HD void pushOut(BlockShared* sh, int b) {
  const CollStatic* c = &sh->cs;
  const int n = c->nranks, me = c->rank;
  const uint64_t es = dtypeSize(c->inType);
  if (c->kind == dfcclCollReduceScatter) {
    for (int k = 1; k < n; ++k) {                  // a different chunk for every member: one copy each
      const int j = (me + k) % n;
      if (df_tid() == 0) {
        DataArgs* a = &sh->args;
        uint64_t bb, be;
        partRange(c->count, c->nBlocks, b, 16, &bb, &be);
        a->nsrc = 1; a->ndst = 1; a->n = (be - bb) * es;
        // the chunk sits in the slot at the misalignment it has in the input (chunks of odd length start off the
        // 16-byte grid), so that the receiver's sources - its own chunk and the slots - all line up alike
        a->src[0] = pushSendPtr(sh) + ((uint64_t)j * c->count + bb) * es;
        a->dst[0] = pushSlot(sh, j, me) + (((uint64_t)j * c->count * es) & 15) + bb * es;
        sh->stats.bytesCopied += a->n;
      }
      df_sync();
      if (sh->args.n) copy_multi(&sh->args);
      df_sync();
    }
    return;
  }
  if (df_tid() == 0) {
    DataArgs* a = &sh->args;
    uint64_t bb, be;
    if (c->kind == dfcclCollAllGather) partRange(c->count * es, c->nBlocks, b, 16, &bb, &be);        // bytes, as its data phase
    else { partRange(c->count, c->nBlocks, b, 16, &bb, &be); bb *= es; be *= es; }
    a->nsrc = 1; a->ndst = 0; a->n = be - bb;
    a->src[0] = pushSendPtr(sh) + bb;
    for (int k = 1; k < n; ++k) { const int j = (me + k) % n; a->dst[a->ndst++] = pushSlot(sh, j, me) + bb; }
    sh->stats.bytesCopied += a->n * a->ndst;
  }
  df_sync();
  if (sh->args.n && sh->args.ndst) copy_multi(&sh->args);
  df_sync();
}

// Push schedule, all-gather: every member's piece is in its slot here; block b copies its part of each into the
// output (my own piece comes from my input, unless the call is in place).  Pieces are small: no slicing.
DF_HD void pushGatherLocal(BlockShared* sh, int b) {
  const CollStatic* c = &sh->cs;
  const int n = c->nranks, me = c->rank;
  const uint64_t bytes = c->count * dtypeSize(c->inType);
  for (int j = 0; j < n; ++j) {
    if (df_tid() == 0) {
      DataArgs* a = &sh->args;
      uint64_t bb, be;
      partRange(bytes, c->nBlocks, b, 16, &bb, &be);
      a->nsrc = 1; a->ndst = 1; a->n = be - bb;
      a->src[0] = (j == me ? pushSendPtr(sh) : (const char*)pushSlot(sh, me, j)) + bb;
      a->dst[0] = pushRecvPtr(sh) + (uint64_t)j * bytes + bb;
      if (a->dst[0] == a->src[0]) a->n = 0;                 // in place: my piece already sits where it belongs
      sh->stats.bytesCopied += a->n;
    }
    df_sync();
    if (sh->args.n) copy_multi(&sh->args);
    df_sync();
  }
}

// ---- PH_DATA: thread 0 builds the pointer lists, everybody moves the data.
// The block's share is moved in slices of `rd->sliceBytes` (0 = all at once): after a slice the cursor is saved and
// the function returns true when more is left, so that the caller can hand the block to another collective and
// come back later - the resumable data phase (reference: slice / offset saved inside one primitive and
// currentStep / gridOffset in the ring loop, src/collectives_ofccl/device/ofccl_prims_simple.h:239-244,326-346,
// ofccl_all_reduce.h:86-93,192-205).  A slice never waits for anybody, so leaving between two slices has no side
// effect beyond the cursor.  `sh->ctl0` tells the caller whether anything else wants the block.
DF_HD bool dataPhase(BlockShared* sh, RankDev* rd, int b) {
  const CollStatic* c = &sh->cs;
  const int n = c->nranks, me = c->rank;
  const uint64_t es = dtypeSize(c->inType), eo = dtypeSize(c->outType);
  // schedules that read or write peers' buffers need the offsets the peers posted
  if (c->kind == dfcclCollAllGather && c->algo == dfcclAlgoPush && n > 1) { pushGatherLocal(sh, b); return false; }
  const bool needOffsets = n > 1 && c->algo != dfcclAlgoPush && c->algo != dfcclAlgoNvls;
  if (needOffsets) fetchPeerOffsets(sh, b);
  else if (df_tid() == 0) { sh->peerSend[me] = mySendOff(sh); sh->peerRecv[me] = myRecvOff(sh); }   // thread 0 is the only reader
  if (df_tid() == 0) {
    DataArgs* a = &sh->args;
    bool reduce = true, nvls = false;
    int nvlsKind = 0;          // 3 = reduce-scatter, 4 = all-gather on the multimem schedule
    a->scale = c->scale; a->postDiv = c->postDiv; a->nsrc = 0; a->ndst = 0; a->n = 0;
    uint64_t bb, be;
    switch (c->kind) {
      case dfcclCollAllReduce: {
        partRange(c->count, c->nBlocks, b, 16, &bb, &be);
        if (c->algo == dfcclAlgoPush && n > 1) {
          // everything is here: my own input plus the slots the peers filled
          a->src[a->nsrc++] = pushSendPtr(sh) + bb * es;
          for (int k = 1; k < n; ++k) a->src[a->nsrc++] = pushSlot(sh, me, (me + k) % n) + bb * es;
          a->dst[a->ndst++] = pushRecvPtr(sh) + bb * eo;
          a->n = be - bb;
        } else if (c->algo == dfcclAlgoNvls && n > 1) {
          // my slice of this block's range, as byte offsets into the arena (symmetric on all members)
          uint64_t sb, se;
          partRange(be - bb, n, me, 16, &sb, &se);
          sb += bb; se += bb;
          const uint64_t in = (sh->dyn.sqeFlags & SQE_SEND_STAGED) ? c->nvlsIn : sh->dyn.send;
          const uint64_t out = (sh->dyn.sqeFlags & SQE_RECV_STAGED) ? c->nvlsOut : sh->dyn.recv;
          a->src[0] = (const char*)(uintptr_t)(in + sb * es); a->nsrc = 1;
          a->dst[0] = (char*)(uintptr_t)(out + sb * eo); a->ndst = 1;
          a->n = se - sb;
          nvls = true;
        } else if (c->algo == dfcclAlgoOneShot || n == 1) {
          for (int j = 0; j < n; ++j) a->src[a->nsrc++] = sendPtrOf(sh, j) + bb * es;
          a->dst[a->ndst++] = recvPtrOf(sh, me) + bb * eo;
          a->n = be - bb;
        } else {
          uint64_t sb, se;
          partRange(be - bb, n, me, 16, &sb, &se);
          sb += bb; se += bb;
          for (int k = 0; k < n; ++k) { int j = (me + k) % n; a->src[a->nsrc++] = sendPtrOf(sh, j) + sb * es; }
          for (int k = 0; k < n; ++k) { int j = (me + k) % n; a->dst[a->ndst++] = recvPtrOf(sh, j) + sb * eo; }
          a->n = se - sb;
        }
        break;
      }
      case dfcclCollReduce: {
        partRange(c->count, c->nBlocks, b, 16, &bb, &be);
        uint64_t sb, se;
        partRange(be - bb, n, me, 16, &sb, &se);
        sb += bb; se += bb;
        for (int k = 0; k < n; ++k) { int j = (me + k) % n; a->src[a->nsrc++] = sendPtrOf(sh, j) + sb * es; }
        a->dst[a->ndst++] = recvPtrOf(sh, c->root) + sb * eo;
        a->n = se - sb;
        break;
      }
      case dfcclCollReduceScatter: {
        partRange(c->count, c->nBlocks, b, 16, &bb, &be);
        if (c->algo == dfcclAlgoNvls && n > 1) {
          // the switch reduces my block of every member's input (arena); the result stays here
          const uint64_t in = (sh->dyn.sqeFlags & SQE_SEND_STAGED) ? c->nvlsIn : sh->dyn.send;
          a->src[0] = (const char*)(uintptr_t)(in + ((uint64_t)me * c->count + bb) * es); a->nsrc = 1;
          a->dst[0] = pushRecvPtr(sh) + bb * eo; a->ndst = 1;
          a->n = be - bb;
          nvlsKind = 3;
          break;
        }
        if (c->algo == dfcclAlgoPush && n > 1) {
          // my chunk of my own input plus my chunk of every peer's input, which they put into their slots here
          a->src[a->nsrc++] = pushSendPtr(sh) + ((uint64_t)me * c->count + bb) * es;
          for (int k = 1; k < n; ++k) a->src[a->nsrc++] = pushSlot(sh, me, (me + k) % n) + (((uint64_t)me * c->count * es) & 15) + bb * es;
          a->dst[a->ndst++] = pushRecvPtr(sh) + bb * eo;
          a->n = be - bb;
          break;
        }
        for (int k = 0; k < n; ++k) { int j = (me + k) % n; a->src[a->nsrc++] = sendPtrOf(sh, j) + ((uint64_t)me * c->count + bb) * es; }
        a->dst[a->ndst++] = recvPtrOf(sh, me) + bb * eo;
        a->n = be - bb;
        break;
      }
      case dfcclCollAllGather: {
        reduce = false;
        uint64_t bytes = c->count * es;
        partRange(bytes, c->nBlocks, b, 16, &bb, &be);
        if (c->algo == dfcclAlgoNvls && n > 1) {
          // one multicast store puts my piece into every member's output (arena)
          const uint64_t out = (sh->dyn.sqeFlags & SQE_RECV_STAGED) ? c->nvlsOut : sh->dyn.recv;
          a->src[0] = pushSendPtr(sh) + bb; a->nsrc = 1;
          a->dst[0] = (char*)(uintptr_t)(out + (uint64_t)me * bytes + bb); a->ndst = 1;
          a->n = be - bb;
          nvlsKind = 4;
          break;
        }
        a->src[0] = sendPtrOf(sh, me) + bb; a->nsrc = 1;
        for (int k = 0; k < n; ++k) {
          int j = (me + k) % n;
          char* d = recvPtrOf(sh, j) + (uint64_t)me * bytes + bb;
          if (d != a->src[0]) a->dst[a->ndst++] = d;          // in-place: my own slot already holds it
        }
        a->n = be - bb;
        break;
      }
      case dfcclCollBroadcast: {
        reduce = false;
        uint64_t bytes = c->count * es;
        partRange(bytes, c->nBlocks, b, 16, &bb, &be);
        if (c->algo == dfcclAlgoNvls && n > 1) {
          // the root's multicast stores put its buffer into every member's output (arena); the others move nothing and
          // learn from the root's done flag that their output is complete
          if (me == c->root) {
            const uint64_t out = (sh->dyn.sqeFlags & SQE_RECV_STAGED) ? c->nvlsOut : sh->dyn.recv;
            a->src[0] = pushSendPtr(sh) + bb; a->nsrc = 1;
            a->dst[0] = (char*)(uintptr_t)(out + bb); a->ndst = 1;
            a->n = be - bb;
            nvlsKind = 4;
          }
          break;
        }
        a->src[0] = sendPtrOf(sh, c->root) + bb; a->nsrc = 1;
        char* d = recvPtrOf(sh, me) + bb;
        if (d != a->src[0]) a->dst[a->ndst++] = d;
        a->n = be - bb;
        break;
      }
      default: break;
    }
    // ---- the slice of this visit: [cursor, cursor + slice) of the block's share, in the unit of a->n (elements
    // for reducing kinds, bytes for copying kinds); slices are multiples of 16 units, so every pointer keeps its
    // 16-byte alignment
    const uint64_t total = a->n;
    const uint64_t unitIn = reduce ? es : 1, unitOut = reduce ? eo : 1;
    uint64_t cur = sh->dyn.cursor < total ? sh->dyn.cursor : total;
    uint64_t win = total - cur;
    if (rd->sliceBytes && !sh->standalone) {
      uint64_t sliceUnits = rd->sliceBytes / unitIn & ~(uint64_t)15;
      if (sliceUnits < 16) sliceUnits = 16;
      if (win > sliceUnits) win = sliceUnits;
    }
    if (cur) {
      for (int j = 0; j < a->nsrc; ++j) a->src[j] += cur * unitIn;
      for (int j = 0; j < a->ndst; ++j) a->dst[j] += cur * unitOut;
    }
    a->n = win;
    sh->ctl64 = cur + win < total ? cur + win : 0;             // the next cursor; 0 = this was the last slice
    sh->ctl1 = nvlsKind ? nvlsKind : nvls ? 2 : reduce ? 1 : 0;
    if (reduce) sh->stats.bytesReduced += a->n * es * a->nsrc; else sh->stats.bytesCopied += a->n * (a->ndst ? a->ndst : 0);
  }
  df_sync();
  if (sh->args.n != 0 && sh->args.ndst != 0) {
    if (sh->ctl1 == 2) {
      if (!nvlsDispatch(c->inType, c->outType, c->mcHeap, c->nvlsPeers, n, (uint64_t)(uintptr_t)sh->args.src[0],
                        (uint64_t)(uintptr_t)sh->args.dst[0], sh->args.n, (float)c->scale) && df_tid() == 0) sh->dyn.status = ST_BAD_ARG;
    } else if (sh->ctl1 == 3) {
      if (!nvlsDispatchToLocal(c->inType, c->outType, c->mcHeap, c->nvlsPeers, n, (uint64_t)(uintptr_t)sh->args.src[0], sh->args.dst[0],
                               sh->args.n, (float)c->scale) && df_tid() == 0) sh->dyn.status = ST_BAD_ARG;
    } else if (sh->ctl1 == 4) {
      nvlsBroadcastBytes(c->mcHeap, c->nvlsPeers, n, sh->args.src[0], (uint64_t)(uintptr_t)sh->args.dst[0], sh->args.n);
    } else if (sh->ctl1) {
      if (!reduce_dispatch(c->inType, c->outType, c->op, &sh->args) && df_tid() == 0) sh->dyn.status = ST_BAD_ARG;
    } else {
      copy_multi(&sh->args);
    }
  }
  df_sync();
  if (df_tid() == 0) {
    sh->ctl0 = 0;
    if (sh->ctl64) {
      sh->dyn.cursor = sh->ctl64; sh->dynDirty = 1;
      // anything else for this block?  queued collectives, submissions waiting for their stream, or entries of the
      // device ring this block has not consumed yet
      sh->ctl0 = (sh->nActive > 1 || sh->nTrig > 0 || ld_relaxed_sys_u64(&rd->devSqTail) != sh->frontier) ? 1 : 0;
    }
  }
  df_sync();
  return sh->ctl64 != 0;
}

// ---- staging copies for buffers outside the symmetric heap
// Block b copies exactly the bytes that block b of the peers (or of this rank) touches in
// PH_DATA, because the flags of block b are the only ordering between the two: the same
// partition as dataPhase, element-based for reducing kinds, byte-based for copying kinds.
DF_HD void stageCopy(BlockShared* sh, int b, bool in) {
  const CollStatic* c = &sh->cs;
  const bool reducing = c->kind == dfcclCollAllReduce || c->kind == dfcclCollReduce || c->kind == dfcclCollReduceScatter;
  const uint64_t e = in ? dtypeSize(c->inType) : dtypeSize(c->outType);
  const int segs = (in && c->kind == dfcclCollReduceScatter) || (!in && c->kind == dfcclCollAllGather) ? c->nranks : 1;
  const uint64_t segBytes = c->count * e;
  uint64_t bb, be;
  if (reducing) { partRange(c->count, c->nBlocks, b, 16, &bb, &be); bb *= e; be *= e; }
  else partRange(segBytes, c->nBlocks, b, 16, &bb, &be);
  for (int s = 0; s < segs; ++s) {
    if (df_tid() == 0) {
      DataArgs* a = &sh->args;
      a->nsrc = 1; a->ndst = 1; a->n = be - bb;
      const uint64_t off = (uint64_t)s * segBytes + bb;
      if (in) { a->src[0] = (const char*)sh->dyn.send + off; a->dst[0] = c->peerHeap[c->rank] + c->stagingSendOff + off; }
      else { a->src[0] = c->peerHeap[c->rank] + c->stagingRecvOff + off; a->dst[0] = (char*)sh->dyn.recv + off; }
      sh->stats.bytesCopied += a->n;
    }
    df_sync();
    if (sh->args.n) copy_multi(&sh->args);
    df_sync();
  }
}

// ---- completion: count blocks; the last one publishes the device flag and the CQE
DF_HD void publishCompletion(RankDev* rd, int coll, uint32_t st, uint32_t epoch) {
  // The device flag releases a stream of THIS GPU (its wait is a stream memory operation, the consumers are kernels
  // launched behind it): everything the blocks wrote here is ordered before it by a fence of GPU scope, a quarter
  // of the cost of a system-scope one.  (What the blocks wrote into peers' memory was ordered by the fence before
  // their done flags, and this rank's result was complete when every peer's done flag had arrived.)
  fence_gpu();
  st_relaxed_sys_u64(&rd->doneEpoch[coll], ((uint64_t)st << 56) | epoch);
  // the host's entry: a host thread may read the result right after the callback, so the data is ordered system-wide
  unsigned long long idx = atomic_add_u64((unsigned long long*)&rd->devCqTail, 1ull);
  uint32_t gen = (uint32_t)(idx / rd->cqCap) + 1u;
  fence_sys();
  st_relaxed_sys_u64(&rd->hostCq[idx & (rd->cqCap - 1)], cqeEncode(gen, st, (uint32_t)coll));
}

DF_HD void completeColl(BlockShared* sh, RankDev* rd, int b) {
  if (sh->standalone) {                           // stream-ordered kernel: report errors only
    if (df_tid() == 0 && sh->dyn.status != ST_OK) rd->ctl->pad = sh->dyn.status;
    df_sync();
    return;
  }
  if (df_tid() == 0) {
    const int coll = sh->loadedColl;
    uint32_t status = sh->dyn.status;
    // the cached copy stays authoritative while the collective is loaded; it reaches global memory when another
    // collective is loaded, when the block parks, or when the next submission of this id is consumed
    sh->dyn.phase = PH_COMPLETE;
    sh->dynDirty = 1;
    sh->stats.collsDone++;
    if (sh->cs.nBlocks == 1) {
      publishCompletion(rd, coll, status > 255 ? (uint32_t)ST_TIMEOUT : status, sh->dyn.epoch);
    } else {
      if (status != ST_OK) atomic_add_u32(&rd->failCount[coll], status << 16 | 1u);
      fence_gpu();
      uint32_t prev = atomic_add_u32(&rd->doneCount[coll], 1u);
      if (prev + 1 == (uint32_t)sh->cs.nBlocks) {
        uint32_t fails = atomic_exch_u32(&rd->failCount[coll], 0u);
        atomic_exch_u32(&rd->doneCount[coll], 0u);
        uint32_t st = fails ? (fails >> 16) / (fails & 0xffff) : ST_OK;   // all failing blocks report the same cause
        if (st > 255) st = ST_TIMEOUT;
        publishCompletion(rd, coll, st, sh->dyn.epoch);
      }
    }
    trace(rd, b, TR_DONE, coll);
  }
  df_sync();
}

// The first phase from `phase` on that has something to do for the loaded submission (a phase change costs two
// block-wide barriers, a small collective would otherwise spend more time changing phases than moving data).
DF_HD int nextPhase(const BlockShared* sh, int phase) {
  const CollStatic* c = &sh->cs;
  const int n = c->nranks, me = c->rank;
  for (;; ++phase) {
    switch (phase) {
      case PH_COPY_IN:
        if ((sh->dyn.sqeFlags & SQE_SEND_STAGED) && !rawSend(c) && !(c->kind == dfcclCollBroadcast && me != c->root)) return phase;
        break;
      case PH_POST_ARRIVE: case PH_WAIT_ARRIVE:
        if (n > 1) return phase;
        break;
      case PH_POST_DONE: case PH_WAIT_DONE:
        if (n > 1 && c->algo != dfcclAlgoPush) return phase;
        break;
      case PH_COPY_OUT:
        if ((sh->dyn.sqeFlags & SQE_RECV_STAGED) && !rawRecv(c) && !(c->kind == dfcclCollReduce && me != c->root)) return phase;
        break;
      default: return phase;          // PH_DATA, PH_COMPLETE (PH_TRIGGER is never skipped to)
    }
  }
}

// A wait of the loaded collective with its adaptive budget.  The budget is what the scheduler grants or, if larger,
// the patience this submission has earned: after a wait succeeded within s polls the next waits of the same
// submission may spend factor x s polls (capped), because a collective whose peers are demonstrably in it is worth
// staying with (reference: RECV_SUCCESS_FACTOR, src/collectives_ofccl/device/ofccl_prims_simple.h:79-88,143-151).
DF_HD bool patientWait(BlockShared* sh, RankDev* rd, int b, int which, uint32_t budget) {
  const uint32_t eff = budget > sh->dyn.patience ? budget : sh->dyn.patience;
  const bool ok = boundedWait(sh, rd, b, which, eff);
  if (ok && df_tid() == 0 && !sh->standalone && rd->recvSuccessFactor) {
    uint64_t p = (uint64_t)sh->waitSpins * rd->recvSuccessFactor;
    const uint64_t cap = (uint64_t)rd->spinBudget * 64u;
    if (p > cap) p = cap;
    if (p > sh->dyn.patience) { sh->dyn.patience = (uint32_t)p; sh->dynDirty = 1; }
  }
  return ok;
}

// Run the loaded-or-to-be-loaded collective until it completes, a wait runs out (RC_STALLED) or its data phase
// reaches a slice boundary while other work is queued (RC_YIELD).
// `budget` is the number of polls one wait may spend.
// `*moved` is set when at least one phase (or slice) was left behind during this visit.
DF_HD int runColl(BlockShared* sh, RankDev* rd, int b, int coll, uint32_t budget, bool* moved) {
  if (!sh->standalone) loadColl(sh, rd, b, coll);
  const int rb = sh->standalone ? b : relBlock(rd, &sh->cs, b);      // my index among this collective's blocks
  const int n = sh->cs.nranks, me = sh->cs.rank;
  const int tid = df_tid(), nt = df_nthreads();
  const int entryPhase = sh->dyn.phase;
  for (;;) {
    const int phase = sh->dyn.phase;
    if (phase != entryPhase) *moved = true;
    switch (phase) {
      case PH_TRIGGER:
        // (the daemon releases stream-ordered submissions from its trigger list and enters at PH_COPY_IN; this
        // phase serves entries that were parked here by an earlier instance)
        if (sh->dyn.sqeFlags & SQE_TRIGGERED) {
          if (!boundedWait(sh, rd, rb, 2, sh->standalone ? budget : 1u)) { if (noteStall(sh, rd)) { setPhase(sh, PH_COMPLETE); break; } return RC_STALLED; }
        }
        if (tid == 0) trace(rd, b, TR_START, coll);
        setPhase(sh, nextPhase(sh, PH_COPY_IN));
        break;
      case PH_COPY_IN:
        if ((sh->dyn.sqeFlags & SQE_SEND_STAGED) && !rawSend(&sh->cs)) {
          bool needed = !(sh->cs.kind == dfcclCollBroadcast && me != sh->cs.root);
          if (needed) stageCopy(sh, rb, true);
          if (tid == 0) fence_sys();
        }
        setPhase(sh, nextPhase(sh, PH_POST_ARRIVE));
        break;
      case PH_POST_ARRIVE: {
        if (sh->cs.algo == dfcclAlgoPush && n > 1) {
          // the payload travels with the arrival flag: stores to a peer, one fence, then the flag
          pushOut(sh, rb);
          if (tid == 0) fence_sys();
          df_sync();
        }
        const uint64_t so = mySendOff(sh), ro = myRecvOff(sh), epoch = sh->dyn.epoch;
        const bool pushed = sh->cs.algo == dfcclAlgoPush && n > 1;
        for (int j = tid; j < n; j += nt) {
          if (j == me) continue;
          FlagSlot* s = sh->cs.peerFlags[j] + (uint64_t)rb * n + me;
          // push: the fence of thread 0 above, between two block-wide barriers, already orders every thread's payload
          // stores before these flag stores (a second fence per flag would only add its latency); the offsets are
          // not used by that schedule
          if (pushed) { st_relaxed_sys_u64(&s->arrive, epoch); continue; }
          st_relaxed_sys_u64(&s->sendOff, so);
          st_relaxed_sys_u64(&s->recvOff, ro);
          st_release_sys_u64(&s->arrive, epoch);
        }
        setPhase(sh, PH_WAIT_ARRIVE);
        break;
      }
      case PH_WAIT_ARRIVE:
        if (n > 1 && !patientWait(sh, rd, rb, 0, budget)) {
          if (noteStall(sh, rd)) { setPhase(sh, PH_COMPLETE); break; }
          if (tid == 0) trace(rd, b, TR_STALL, coll);
          return RC_STALLED;
        }
        if (tid == 0) trace(rd, b, TR_ARRIVED, coll);
        setPhase(sh, PH_DATA);
        break;
      case PH_DATA: {
        if (tid == 0) trace(rd, b, TR_DATA_BEGIN, coll);
        const bool more = dataPhase(sh, rd, rb);
        if (tid == 0) trace(rd, b, TR_DATA_END, coll);
        if (more) {                                   // the cursor is saved; the phase stays PH_DATA
          *moved = true;
          if (sh->ctl0) {
            if (tid == 0) { sh->stats.yields++; trace(rd, b, TR_YIELD, coll); }
            return RC_YIELD;
          }
          break;
        }
        // (push schedule: no done handshake - nobody reads my buffers and my slots are not reused before the
        // peers' next-but-one call)
        setPhase(sh, nextPhase(sh, PH_POST_DONE));
        break;
      }
      case PH_POST_DONE: {
        if (n > 1) {
          // all payload stores of this block were issued before the barrier inside setPhase; one fence
          // by the posting thread makes them visible system-wide before any done flag is
          const uint64_t epoch = sh->dyn.epoch;
          if (tid == 0) {
            fence_sys();
            for (int j = 0; j < n; ++j)
              if (j != me) st_relaxed_sys_u64(&(sh->cs.peerFlags[j] + (uint64_t)rb * n + me)->done, epoch);
          }
        }
        setPhase(sh, PH_WAIT_DONE);
        break;
      }
      case PH_WAIT_DONE:
        if (n > 1 && !patientWait(sh, rd, rb, 1, budget)) {
          if (noteStall(sh, rd)) { setPhase(sh, PH_COMPLETE); break; }
          if (tid == 0) trace(rd, b, TR_STALL, coll);
          return RC_STALLED;
        }
        if (tid == 0) trace(rd, b, TR_PEERS_DONE, coll);
        setPhase(sh, nextPhase(sh, PH_COPY_OUT));
        break;
      case PH_COPY_OUT:
        if ((sh->dyn.sqeFlags & SQE_RECV_STAGED) && !rawRecv(&sh->cs)) {
          bool needed = !(sh->cs.kind == dfcclCollReduce && me != sh->cs.root);
          if (needed) stageCopy(sh, rb, false);
        }
        setPhase(sh, PH_COMPLETE);
        break;
      default:  // PH_COMPLETE
        completeColl(sh, rd, b);
        return RC_DONE;
    }
  }
}

}  // namespace dfccl
