// Per-block scheduler of the persistent daemon.
//
// Every block of a rank runs daemonBlockMain independently; nothing in here makes
// one block of a GPU wait for another block of the same GPU.  Each block
//   1. finds new submissions in the device-resident ring (the host writes entries
//      and tail there with stream memory operations: no block reads host memory),
//   2. consumes every entry of that ring in order (its own frontier), and
//      appends the collectives it takes part in (relative block index < nBlocks of the
//      collective) to its task queue,
//   3. walks the task queue: runs each collective until it finishes or a bounded
//      wait gives up, in which case the collective stays queued and the next one
//      is loaded - the preemption that makes any per-rank issue order deadlock-free,
//   4. leaves voluntarily when it has been idle (or only stalled) for long enough,
//      parking its frontier and task queue in global memory for the next launch.
// Same responsibilities as the reference's daemonKernel loop
// (src/collectives_ofccl/device/enqueue_ofccl_dev.cu:1026-1483: sqRead :85-173,
// checkSQ7TidyTaskQ :491-627, traverseTaskQ :922-1023, voluntary quit :1107-1117,
// state save :1374-1480), with a device-resident queue mirror, a trigger list for
// submissions that wait for their stream (polled without loading any context),
// time-based instead of count-based quit thresholds and a two-integer cursor per
// parked collective.
#pragma once
#include "engine.h"

namespace dfccl {

// Consume new entries of the device ring.  Thread 0 only.  Returns the number consumed.
// A submission that waits for its stream goes to the trigger list, everything else to the task queue.
DF_HD int consumeSubmissions(BlockShared* sh, RankDev* rd, int b) {
  uint64_t tail = ld_relaxed_sys_u64(&rd->devSqTail);
  if (tail == sh->frontier) return 0;
  // The entries were written (by the host, through stream memory operations, each preceded by a fence) before the
  // tail that announced them.  On this side the entry loads are issued after the branch on the tail's value, which
  // the hardware does not speculate past; the fence keeps the compiler and the memory pipeline from hoisting them.
  fence_gpu();
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
    const bool mine = coll >= 0 && (uint32_t)coll < rd->maxColls && rd->colls[coll].valid && relBlock(rd, &rd->colls[coll], b) < rd->colls[coll].nBlocks;
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
      if ((q.flags & SQE_TRIGGERED) ? sh->nTrig >= DF_MAX_ACTIVE : sh->nActive >= DF_MAX_ACTIVE) break;   // (cannot happen: one outstanding submission per id)
    }
    ++sh->frontier;
    ++got;
    sh->stats.sqesSeen++;
    if (!mine) continue;
    d->send = q.send; d->recv = q.recv; d->trigger = q.trigger; d->cursor = 0;
    d->epoch = d->epoch + 1; d->sqeFlags = q.flags; d->status = ST_OK; d->stallSinceNs = 0; d->patience = 0;
    trace(rd, b, TR_SQE, coll);
    if (q.flags & SQE_TRIGGERED) {
      d->phase = PH_TRIGGER;
      sh->trigColl[sh->nTrig] = (uint16_t)coll; sh->trigVal[sh->nTrig] = (uint32_t)q.trigger; ++sh->nTrig;
    } else {
      d->phase = PH_COPY_IN;          // runColl skips ahead to the first phase that has work
      sh->actWait[sh->nActive] = 0;
      sh->active[sh->nActive++] = (uint16_t)coll;
      trace(rd, b, TR_START, coll);
    }
  }
  if (got) st_relaxed_sys_u64(&rd->hostFrontier[b], sh->frontier);   // posted store: the host reads it when its ring looks full
  return got;
}

// Look at the trigger words of every submission that waits for its stream: one thread per entry, no context is
// loaded.  Released ones join the task queue in list order.  Everybody calls it; returns the number released.
DF_HD uint32_t pollTriggers(BlockShared* sh, RankDev* rd, int b) {
  const int tid = df_tid(), nt = df_nthreads();
  const uint32_t nTrig = sh->nTrig;
  if (tid == 0) sh->trigFired = 0;
  df_sync();
  for (uint32_t i = tid; i < nTrig; i += nt) {
    const uint32_t have = (uint32_t)ld_relaxed_sys_u64(&rd->trigger[sh->trigColl[i]]);
    if ((int32_t)(have - sh->trigVal[i]) >= 0) { sh->trigColl[i] |= 0x8000u; atomic_add_u32(&sh->trigFired, 1u); }
  }
  df_sync();
  const uint32_t fired = sh->trigFired;
  if (fired && tid == 0) {
    fence_sys();                     // what the stream's producers wrote, before anything this block does with it
    uint32_t w = 0;
    for (uint32_t i = 0; i < nTrig; ++i) {
      const uint16_t e = sh->trigColl[i];
      if (e & 0x8000u) {
        const int coll = e & 0x7fff;
        rd->dyn[(uint64_t)b * rd->maxColls + coll].phase = PH_COPY_IN;
        if (sh->nActive < DF_MAX_ACTIVE) { sh->actWait[sh->nActive] = 0; sh->active[sh->nActive++] = (uint16_t)coll; }
        trace(rd, b, TR_START, coll);
      } else { sh->trigColl[w] = e; sh->trigVal[w] = sh->trigVal[i]; ++w; }
    }
    sh->nTrig = w;
  }
  if (fired) df_sync();
  return fired;
}

// Readiness scan: one thread per parked entry of the task queue reads that collective's flag words of this block
// (n loads of local memory) and marks the entry for a visit when every peer has posted the epoch the entry waits
// for.  No context is loaded and nobody spins: a queue of stalled collectives costs one scan per pass instead of a
// context switch and a polling budget each.  Everybody calls it; returns the number of entries that became ready.
DF_HD uint32_t scanParked(BlockShared* sh, RankDev* rd, int b) {
  const int tid = df_tid(), nt = df_nthreads();
  const uint32_t nAct = sh->nActive;
  if (tid == 0) sh->nReady = 0;
  df_sync();
  for (uint32_t i = tid; i < nAct; i += nt) {
    const uint32_t w = sh->actWait[i];
    if (w == 0) continue;
    const int coll = sh->active[i];
    if (coll == 0xffff) continue;
    const CollStatic* c = &rd->colls[coll];
    const int n = c->nranks, me = c->rank;
    const FlagSlot* f = c->myFlags + (uint64_t)relBlock(rd, c, b) * n;
    const uint64_t epoch = rd->dyn[(uint64_t)b * rd->maxColls + coll].epoch;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      if (j == me) continue;
      ok = ok && ld_relaxed_sys_u64(w == 1 ? &f[j].arrive : &f[j].done) >= epoch;
    }
    if (ok) { sh->actWait[i] = 0; atomic_add_u32(&sh->nReady, 1u); }
  }
  df_sync();
  return sh->nReady;
}

DF_HD void blockRestore(BlockShared* sh, RankDev* rd, int b) {
  const int tid = df_tid(), nt = df_nthreads();
  BlockSaved* sv = &rd->saved[b];
  if (tid == 0) {
    sh->loadedColl = -1; sh->standalone = 0; sh->dynDirty = 0; sh->quit = 0; sh->abortSeen = 0; sh->ctl1Full = 0;
    sh->frontier = sv->frontier; sh->nActive = sv->nActive; sh->nTrig = sv->nTrig;
    DevStats z = {};
    sh->stats = z;
    sv->exited = 0;
  }
  df_sync();
  for (uint32_t i = tid; i < sh->nActive; i += nt) { sh->active[i] = sv->active[i]; sh->actWait[i] = 0; }    // everything gets a visit first
  for (uint32_t i = tid; i < sh->nTrig; i += nt) { sh->trigColl[i] = sv->trigColl[i]; sh->trigVal[i] = sv->trigVal[i]; }
  df_sync();
}

DF_HD void blockPark(BlockShared* sh, RankDev* rd, int b) {
  const int tid = df_tid(), nt = df_nthreads();
  saveLoaded(sh, rd, b);
  BlockSaved* sv = &rd->saved[b];
  for (uint32_t i = tid; i < sh->nActive; i += nt) sv->active[i] = sh->active[i];
  for (uint32_t i = tid; i < sh->nTrig; i += nt) { sv->trigColl[i] = sh->trigColl[i]; sv->trigVal[i] = sh->trigVal[i]; }
  df_sync();
  if (tid == 0) {
    sv->frontier = sh->frontier; sv->nActive = sh->nActive; sv->nTrig = sh->nTrig;
    // fold this launch's counters into the totals the host reads
    DevStats* g = &rd->stats[b];
    g->ctxSwitches += sh->stats.ctxSwitches; g->ctxSaves += sh->stats.ctxSaves; g->ctxLoads += sh->stats.ctxLoads;
    g->waitPolls += sh->stats.waitPolls; g->waitTimeouts += sh->stats.waitTimeouts;
    g->bytesReduced += sh->stats.bytesReduced; g->bytesCopied += sh->stats.bytesCopied;
    g->totalSwitchNs += sh->stats.totalSwitchNs; g->sqesSeen += sh->stats.sqesSeen; g->collsDone += sh->stats.collsDone;
    g->visits += sh->stats.visits; g->yields += sh->stats.yields; g->passes += sh->stats.passes;
    g->nsTriggers += sh->stats.nsTriggers; g->nsWalk += sh->stats.nsWalk; g->nsQueues += sh->stats.nsQueues;
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
  uint64_t lastUseful = df_now_ns();     // only thread 0's copies of these are ever consulted
  const uint64_t bornNs = lastUseful;
  uint64_t lastSlowCheck = 0, lastFullPass = 0;
  uint32_t winding = 0;
  uint32_t idleBackoff = 32;

  for (;;) {
    // ---- 0. submissions waiting for their stream (every value steering control flow here is block-uniform)
    bool progressed = false;
    const uint64_t tPass = tid == 0 ? df_now_ns() : 0;
    if (sh->nTrig && pollTriggers(sh, rd, b)) progressed = true;
    const uint64_t tWalk = tid == 0 ? df_now_ns() : 0;
    // ---- 1. task queue traversal: parked entries are skipped unless the scan found their flags ready; now and then
    // every entry is visited all the same, so that a wait that will never succeed reaches its time limit
    const uint32_t nAct = sh->nActive;
    if (nAct) {
      if (scanParked(sh, rd, b)) progressed = true;
      const bool fullPass = sh->ctl1Full != 0;
      for (uint32_t i = 0; i < nAct; ++i) {
        const int coll = sh->active[i];
        if (coll == 0xffff) continue;
        if (sh->actWait[i] && !fullPass) continue;
        // With other collectives queued a wait gives up after a few polls: the scan brings the block back when
        // the flags are there.  The oldest submission (head of the queue) gets more patience, and with nothing
        // else queued there is nothing to switch to: polling longer is free.
        const uint32_t base = nAct == 1 ? rd->spinBudget : (rd->spinBudget + 7u) / 8u;
        const uint32_t budget = base * ((i == 0 || nAct == 1) ? rd->headTries : 1u);
        bool moved = false;
        int rc = runColl(sh, rd, b, coll, budget, &moved);
        if (rc == RC_DONE || rc == RC_YIELD || moved) progressed = true;
        if (tid == 0) {
          sh->stats.visits++;
          if (rc == RC_DONE) sh->active[i] = 0xffff;
          sh->actWait[i] = rc == RC_STALLED ? (sh->dyn.phase == PH_WAIT_ARRIVE ? 1 : sh->dyn.phase == PH_WAIT_DONE ? 2 : 0) : 0;
        }
        // a collective released by its stream should not wait for a walk over a long queue
        if (sh->nTrig && i + 1 < nAct && pollTriggers(sh, rd, b)) progressed = true;
      }
    }
    df_sync();
    // ---- 2. compaction, new submissions, idle decision: thread 0 decides, everybody obeys
    if (tid == 0) {
      sh->stats.passes++;
      uint32_t w = 0;
      for (uint32_t i = 0; i < sh->nActive; ++i) if (sh->active[i] != 0xffff) { sh->active[w] = sh->active[i]; sh->actWait[w] = sh->actWait[i]; ++w; }
      sh->nActive = w;
      const uint64_t now = df_now_ns();
      sh->ctl1Full = 0;
      if (now - lastFullPass > 2000000) { sh->ctl1Full = 1; lastFullPass = now; }     // every 2 ms: visit parked entries too
      sh->stats.nsTriggers += tWalk - tPass; sh->stats.nsWalk += now - tWalk;
      // Words that change rarely are sampled rarely: the abort request and the "somebody left" word.  Every
      // 20 us, or right away when this pass achieved nothing.
      const bool slow = now - lastSlowCheck > 20000;
      if (slow) {
        sh->abortSeen = abortRequested(rd) ? 1u : 0u;
        lastSlowCheck = now;
      }
      if (slow || !progressed || winding) winding = ld_relaxed_sys_u32(&rd->quitting);
      // once one block of this rank has left voluntarily the others take no new work and follow as
      // soon as they cannot progress: a collective needs all its blocks, so the relaunch comes sooner
      if (!winding && consumeSubmissions(sh, rd, b) > 0) progressed = true;
      if (sh->abortSeen) sh->quit = 3;
      else if (rd->maxLifetimeNs && now - bornNs > rd->maxLifetimeNs && !sh->quit) {
        // safety net: no instance of the daemon outlives this, whatever its state; the host relaunches it
        sh->quit = 1;
        st_release_sys_u32(&rd->quitting, 1u);
      }
      else if (progressed) lastUseful = now;
      // only waiting for streams to release submissions: the host relaunches the daemon when a trigger fires, so by
      // default it leaves as quickly as when idle; a caller whose releases come in quick succession (the buckets
      // of a captured backward pass) can ask it to stay for longer and save the relaunches
      else if (!sh->quit && (winding || now - lastUseful > (sh->nActive ? rd->stallQuitNs : sh->nTrig ? rd->trigQuitNs : rd->idleQuitNs))) {
        // a stream parked on one of this context's completion words must not depend on a host thread's
        // relaunch: while the host holds the instance it only leaves by age (or with the others)
        if (!winding && ctl_load(&rd->ctl->hold)) lastUseful = now;
        else {
          sh->quit = 1;
          st_release_sys_u32(&rd->quitting, 1u);
        }
      }
      sh->ctl0 = progressed ? 1 : 0;
      sh->stats.nsQueues += df_now_ns() - now;
    }
    df_sync();
    if (sh->quit) break;
    if (sh->ctl0) idleBackoff = 32;
    else if (sh->nActive == 0 && sh->nTrig == 0) {            // nothing to do: poll gently
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
