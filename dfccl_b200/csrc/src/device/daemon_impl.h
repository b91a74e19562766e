// Per-block scheduler of the persistent daemon.
//
// Every block of a rank runs daemonBlockMain independently; nothing in here makes
// one block of a GPU wait for another block of the same GPU.  Each block
//   1. mirrors newly published submission entries from the host-pinned ring into
//      the device-resident ring (whichever block wins the fetch lock does it, so a
//      single block polls host memory at any time),
//   2. consumes every entry of the device ring in order (its own frontier), and
//      appends the collectives it takes part in (block index < nBlocks of the
//      collective) to its task queue,
//   3. walks the task queue: runs each collective until it finishes or a bounded
//      wait gives up, in which case the collective stays queued and the next one
//      is loaded - the preemption that makes any per-rank issue order deadlock-free,
//   4. leaves voluntarily when it has been idle (or only stalled) for long enough,
//      parking its frontier and task queue in global memory for the next launch.
// Same responsibilities as the reference's daemonKernel loop
// (src/collectives_ofccl/device/enqueue_ofccl_dev.cu:1026-1483: sqRead :85-173,
// checkSQ7TidyTaskQ :491-627, traverseTaskQ :922-1023, voluntary quit :1107-1117,
// state save :1374-1480), with a device-resident queue mirror, time-based instead
// of count-based quit thresholds and a two-integer cursor per parked collective.
#pragma once
#include "engine.h"

namespace dfccl {

// Try to mirror host entries into the device ring.  Thread 0 only.
DF_HD void fetchSubmissions(RankDev* rd) {
  if (atomic_cas_u32(&rd->fetchLock, 0u, 1u) != 0u) return;
  uint64_t devTail = ld_relaxed_sys_u64(&rd->devSqTail);
  uint64_t hostTail = ld_acquire_sys_u64(rd->hostSqTail);
  if (hostTail != devTail) {
    // do not overwrite entries some block has not consumed yet
    uint64_t minFront = ~0ull;
    for (uint32_t i = 0; i < rd->nBlocks; ++i) minFront = umin64(minFront, ld_relaxed_sys_u64(&rd->frontier[i]));
    uint64_t limit = umin64(hostTail, minFront + rd->sqCap);
    const uint32_t mask = rd->sqCap - 1;
    for (uint64_t s = devTail; s < limit; ++s) {
      const uint4* src = (const uint4*)&rd->hostSq[s & mask];
      uint4* dst = (uint4*)&rd->devSq[s & mask];
      uint4 a = ld16(src), bq = ld16(src + 1);
      st16(dst, a); st16(dst + 1, bq);
    }
    if (limit != devTail) {
      fence_gpu();
      st_release_sys_u64(&rd->devSqTail, limit);
      st_release_sys_u64(rd->hostSqHead, limit);
    }
  }
  fence_gpu();
  atomic_exch_u32(&rd->fetchLock, 0u);
}

// Consume new entries of the device ring.  Thread 0 only.  Returns the number consumed.
DF_HD int consumeSubmissions(BlockShared* sh, RankDev* rd, int b) {
  uint64_t tail = ld_acquire_sys_u64(&rd->devSqTail);
  int got = 0;
  const uint32_t mask = rd->sqCap - 1;
  while (sh->frontier < tail) {
    const Sqe* e = &rd->devSq[sh->frontier & mask];
    uint4 w0 = ld16(e), w1 = ld16((const char*)e + 16);
    Sqe q;
    __builtin_memcpy(&q, &w0, 16);
    __builtin_memcpy((char*)&q + 16, &w1, 16);
    if (q.flags & SQE_QUIT) { sh->quit = 2; break; }       // the frontier stays on the quit entry
    const int coll = q.collId;
    const bool mine = coll >= 0 && (uint32_t)coll < rd->maxColls && rd->colls[coll].valid && b < rd->colls[coll].nBlocks;
    CollDyn* d = mine ? &rd->dyn[(uint64_t)b * rd->maxColls + coll] : nullptr;
    if (mine) {
      // A stream-ordered caller may publish the next submission of a collective while this block
      // still runs the previous one.  The entry is never dropped: consumption stops here and
      // resumes once the running submission has completed.
      const CollDyn* cur = sh->loadedColl == coll ? &sh->dyn : d;
      if (cur->epoch != 0 && cur->phase != PH_COMPLETE) break;
      if (sh->loadedColl == coll) {                         // re-armed below in global memory: drop the cached copy
        saveLoaded(sh, rd, b);
        sh->loadedColl = -1;
      }
    }
    ++sh->frontier;
    ++got;
    sh->stats.sqesSeen++;
    if (!mine) continue;
    d->send = q.send; d->recv = q.recv; d->trigger = q.trigger; d->cursor = 0;
    d->epoch = d->epoch + 1; d->phase = PH_TRIGGER; d->sqeFlags = q.flags; d->status = ST_OK; d->stallSinceNs = 0;
    if (sh->nActive < DF_MAX_ACTIVE) sh->active[sh->nActive++] = (uint16_t)coll;
    trace(rd, b, TR_SQE, coll);
  }
  st_release_sys_u64(&rd->frontier[b], sh->frontier);
  return got;
}

DF_HD void blockRestore(BlockShared* sh, RankDev* rd, int b) {
  const int tid = df_tid(), nt = df_nthreads();
  BlockSaved* sv = &rd->saved[b];
  if (tid == 0) {
    sh->loadedColl = -1; sh->standalone = 0; sh->dynDirty = 0; sh->quit = 0; sh->abortSeen = 0;
    sh->frontier = sv->frontier; sh->nActive = sv->nActive;
    DevStats z = {};
    sh->stats = z;
    sv->exited = 0;
  }
  df_sync();
  for (uint32_t i = tid; i < sh->nActive; i += nt) sh->active[i] = sv->active[i];
  df_sync();
}

DF_HD void blockPark(BlockShared* sh, RankDev* rd, int b) {
  const int tid = df_tid(), nt = df_nthreads();
  saveLoaded(sh, rd, b);
  BlockSaved* sv = &rd->saved[b];
  for (uint32_t i = tid; i < sh->nActive; i += nt) sv->active[i] = sh->active[i];
  df_sync();
  if (tid == 0) {
    sv->frontier = sh->frontier; sv->nActive = sh->nActive;
    // fold this launch's counters into the totals the host reads
    DevStats* g = &rd->stats[b];
    g->ctxSwitches += sh->stats.ctxSwitches; g->ctxSaves += sh->stats.ctxSaves; g->ctxLoads += sh->stats.ctxLoads;
    g->waitPolls += sh->stats.waitPolls; g->waitTimeouts += sh->stats.waitTimeouts;
    g->bytesReduced += sh->stats.bytesReduced; g->bytesCopied += sh->stats.bytesCopied;
    g->totalSwitchNs += sh->stats.totalSwitchNs; g->sqesSeen += sh->stats.sqesSeen; g->collsDone += sh->stats.collsDone;
    g->visits += sh->stats.visits;
    if (sh->stats.maxSwitchNs > g->maxSwitchNs) g->maxSwitchNs = sh->stats.maxSwitchNs;
    trace(rd, b, TR_QUIT, (int)sh->quit);
    fence_sys();
    sv->exited = 1;
    uint32_t prev = atomic_add_u32(&rd->exitedBlocks, 1u);
    if (prev + 1 == rd->nBlocks) {                     // last block of this rank out: tell the host
      atomic_exch_u32(&rd->exitedBlocks, 0u);
      st_release_sys_u32(&rd->quitting, 0u);
      if (sh->quit == 2) ctl_store(&rd->ctl->finalQuit, 1);
      if (sh->quit == 1) rd->ctl->voluntaryQuits = rd->ctl->voluntaryQuits + 1;
      fence_sys();
      st_release_sys_u32(&rd->ctl->alive, 0u);
    }
  }
}

DF_HD void daemonBlockMain(RankDev* rd, int b, BlockShared* sh) {
  const int tid = df_tid();
  blockRestore(sh, rd, b);
  if (tid == 0) trace(rd, b, TR_LAUNCH, 0);
  uint64_t lastUseful = df_now_ns();     // only thread 0's copy is ever consulted
  const uint64_t bornNs = lastUseful;
  uint64_t lastAbortCheck = 0;
  uint32_t idleBackoff = 32;

  for (;;) {
    // ---- 1. task queue traversal (every value steering control flow here is block-uniform)
    bool progressed = false;
    uint32_t trigWaits = 0;          // collectives whose stream has not released them yet
    const uint32_t nAct = sh->nActive;
    for (uint32_t i = 0; i < nAct; ++i) {
      const int coll = sh->active[i];
      if (coll == 0xffff) continue;
      // the head of the queue is the oldest submission: give it more patience
      // with nothing else queued there is nothing to switch to: polling longer is free
      const uint32_t budget = rd->spinBudget * ((i == 0 || nAct == 1) ? rd->headTries : 1u);
      bool moved = false;
      int rc = runColl(sh, rd, b, coll, budget, &moved);
      if (rc == RC_DONE || moved) progressed = true;
      if (rc == RC_STALLED && sh->dyn.phase == PH_TRIGGER) ++trigWaits;
      if (tid == 0) {
        sh->stats.visits++;
        if (rc == RC_DONE) sh->active[i] = 0xffff;
      }
    }
    df_sync();
    // ---- 2. compaction, new submissions, idle decision: thread 0 decides, everybody obeys
    if (tid == 0) {
      uint32_t w = 0;
      for (uint32_t i = 0; i < sh->nActive; ++i) if (sh->active[i] != 0xffff) sh->active[w++] = sh->active[i];
      sh->nActive = w;
      // once one block of this rank has left voluntarily the others take no new work and follow as
      // soon as they cannot progress: a collective needs all its blocks, so the relaunch comes sooner
      const bool winding = ld_acquire_sys_u32(&rd->quitting) != 0;
      if (!winding) {
        if (ld_relaxed_sys_u64(&rd->devSqTail) == sh->frontier) fetchSubmissions(rd);
        if (consumeSubmissions(sh, rd, b) > 0) progressed = true;
      }
      const uint64_t now = df_now_ns();
      // the abort word lives in host memory: one read over PCIe costs more than a whole pass over a short
      // task queue, so it is sampled every 20 us instead of every pass
      if (now - lastAbortCheck > 20000) { sh->abortSeen = ctl_load(&rd->ctl->abortFlag); lastAbortCheck = now; }
      if (sh->abortSeen) sh->quit = 3;
      else if (rd->maxLifetimeNs && now - bornNs > rd->maxLifetimeNs && !sh->quit) {
        // safety net: no instance of the daemon outlives this, whatever its state; the host relaunches it
        sh->quit = 1;
        st_release_sys_u32(&rd->quitting, 1u);
      }
      else if (progressed) lastUseful = now;
      // only waiting for streams to release submissions: nothing a resident daemon can speed up, and
      // the host relaunches it when a trigger fires, so leave as quickly as when idle
      else if (!sh->quit && (winding || now - lastUseful > ((sh->nActive && trigWaits < nAct) ? rd->stallQuitNs : rd->idleQuitNs))) {
        // a stream parked on one of this context's completion words must not depend on a host thread's
        // relaunch: while the host holds the instance it only leaves by age (or with the others)
        if (!winding && ctl_load(&rd->ctl->hold)) lastUseful = now;
        else {
          sh->quit = 1;
          st_release_sys_u32(&rd->quitting, 1u);
        }
      }
      sh->ctl0 = progressed ? 1 : 0;
    }
    df_sync();
    if (sh->quit) break;
    if (sh->ctl0) idleBackoff = 32;
    else if (sh->nActive == 0) {            // nothing to do: poll gently
      df_backoff(idleBackoff);
      if (idleBackoff < 1024) idleBackoff *= 2;
    }
  }
  blockPark(sh, rd, b);
}

// Stream-ordered execution of ONE collective by a plain (non-persistent) kernel: the
// same phases, but a wait that runs out is simply retried until the time limit.
DF_HD void standaloneBlockMain(RankDev* rd, int b, BlockShared* sh, const CollStatic* cs, uint64_t send, uint64_t recv,
                               uint32_t epoch, uint32_t sqeFlags) {
  const int tid = df_tid(), nt = df_nthreads();
  {
    const uint4* s = (const uint4*)cs;
    uint4* d = (uint4*)&sh->cs;
    for (int i = tid; i < (int)(sizeof(CollStatic) / 16); i += nt) d[i] = s[i];
  }
  if (tid == 0) {
    sh->loadedColl = 0; sh->standalone = 1; sh->dynDirty = 0; sh->quit = 0; sh->abortSeen = 0;
    DevStats z = {};
    sh->stats = z;
    CollDyn d = {};
    // epoch 0 = take it from the device: one more than the collectives this communicator has finished
    d.send = send; d.recv = recv; d.epoch = epoch ? epoch : rd->saEpoch + 1u; d.phase = PH_COPY_IN; d.sqeFlags = sqeFlags; d.status = ST_OK;
    sh->dyn = d;
  }
  df_sync();
  for (;;) {
    bool moved = false;
    if (runColl(sh, rd, b, 0, 4096u, &moved) == RC_DONE) break;
  }
  if (epoch == 0) {                       // the last block out publishes the new count (every block has read the old one by now)
    df_sync();
    if (tid == 0) {
      const uint32_t mine = sh->dyn.epoch;
      if (atomic_add_u32(&rd->exitedBlocks, 1u) + 1u == (uint32_t)sh->cs.nBlocks) {
        atomic_exch_u32(&rd->exitedBlocks, 0u);
        rd->saEpoch = mine;
        fence_sys();
      }
    }
  }
}

}  // namespace dfccl
