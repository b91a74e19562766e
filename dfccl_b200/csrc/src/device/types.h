// Structures shared by the host runtime and the daemon kernel.
//
// Everything here is plain data laid out identically on both sides.  Roles map to
// the reference as follows (reference paths are relative to its src/):
//   Sqe / host SQ ring      - include/collectives_ofccl.h:129-145 (SQE, SQ)
//   CQ entry encoding       - include/collectives_ofccl.h:11-19,152-157
//   CollStatic              - StaticCollCtx   include/collectives_ofccl.h:320-343
//   CollDyn                 - DynamicCollCtx  include/collectives_ofccl.h:344-355
//   BlockSaved / BlockShared- BlkStatus       include/collectives_ofccl.h:171-318
// The differences are deliberate: queues have a device-resident mirror so that
// only one block at a time polls host memory; a collective owns flag words in
// every member's symmetric heap instead of a private communicator with FIFOs;
// the saved cursor of a parked collective is (phase, cursor) because the data
// movement between two waits never blocks.
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>

#define DF_MAX_RANKS 64        // ranks of one communicator the direct-access engine serves (one NVLink domain: 8 per node, up to 72 in a rack)
#define DF_MAX_BLOCKS 64       // daemon thread blocks per rank
#define DF_MAX_COLLS 2048      // collective ids per rank context (reference MAX_LENGTH = 2000)
#define DF_WARP 32

namespace dfccl {

// ---- submission queue entry (32 bytes, copied as two 16-byte words)
enum SqeFlags : uint32_t {
  SQE_QUIT = 1u,          // final quit: every block saves nothing and leaves for good
  SQE_TRIGGERED = 2u,     // do not start before trigger[collId] >= trigger value (stream-ordered submit)
  SQE_SEND_STAGED = 4u,   // sendbuff is outside the symmetric heap: copy it into the staging area first
  SQE_RECV_STAGED = 8u,   // recvbuff is outside the heap: peers write staging, copy out at the end
};
struct alignas(16) Sqe {
  int32_t collId;
  uint32_t flags;
  uint64_t send;          // heap offset, or raw local address when SQE_SEND_STAGED
  uint64_t recv;          // heap offset, or raw local address when SQE_RECV_STAGED
  uint64_t trigger;       // value trigger[collId] must reach (SQE_TRIGGERED)
};

// ---- completion entry: one 64-bit word, gen makes a slot self-validating
//   [63:32] generation of the ring slot (index / capacity + 1)   [31:24] status   [23:0] collId
static __host__ __device__ inline uint64_t cqeEncode(uint32_t gen, uint32_t status, uint32_t collId) {
  return ((uint64_t)gen << 32) | ((uint64_t)(status & 0xff) << 24) | (collId & 0xffffff);
}
static __host__ __device__ inline uint32_t cqeGen(uint64_t e) { return (uint32_t)(e >> 32); }
static __host__ __device__ inline uint32_t cqeStatus(uint64_t e) { return (uint32_t)(e >> 24) & 0xff; }
static __host__ __device__ inline uint32_t cqeColl(uint64_t e) { return (uint32_t)e & 0xffffff; }

// ---- per (collective, block, source rank) flag words, written by the source rank
struct alignas(32) FlagSlot {
  uint64_t arrive;        // epoch of the submission whose offsets are valid
  uint64_t sendOff;       // source rank's send buffer, offset in its heap
  uint64_t recvOff;       // source rank's recv buffer, offset in its heap
  uint64_t done;          // epoch whose data movement the source rank finished
};

// ---- phases of a collective on one block (the saved cursor)
enum Phase : int32_t {
  PH_TRIGGER = 0,         // bounded wait: local trigger word
  PH_COPY_IN = 1,         // local copy user send buffer -> staging (unregistered buffers)
  PH_POST_ARRIVE = 2,     // write my offsets + epoch into every peer's flag slot
  PH_WAIT_ARRIVE = 3,     // bounded wait: all peers arrived
  PH_DATA = 4,            // move data; never blocks
  PH_POST_DONE = 5,       // fence, then write done = epoch into every peer's flag slot
  PH_WAIT_DONE = 6,       // bounded wait: all peers done
  PH_COPY_OUT = 7,        // local copy staging -> user recv buffer
  PH_COMPLETE = 8,
};

enum CollStatus : uint32_t { ST_OK = 0, ST_TIMEOUT = 1, ST_ABORTED = 2, ST_BAD_ARG = 3 };

// ---- immutable description of a registered collective (one per collId per rank)
struct alignas(16) CollStatic {
  int32_t kind;           // dfcclColl_t
  int32_t inType, outType;
  int32_t op;             // ncclSum..ncclMin (Avg is folded into scale / postDiv at prepare time)
  int32_t nranks, rank, root;
  int32_t nBlocks;        // blocks that take part; the block at relative index b handles slice b of the data
  int32_t algo;           // dfcclAlgo_t actually used
  int32_t postDiv;        // integer average: divide the sum by this (0 = off)
  int32_t valid;
  int32_t blockBase;      // daemon block that plays relative block 0 of this collective: the nBlocks participants are
                          // blockBase, blockBase + 1, ... (mod the daemon's block count), so that collectives too small
                          // for every block do not all land on the first blocks.  A per-rank choice: ranks meet by
                          // relative index only.
  double scale;           // multiplies the reduced value (1.0 = off)
  uint64_t count;         // elements, NCCL convention of the kind
  uint64_t stagingSendOff, stagingRecvOff;      // my heap offsets of staging areas (0 = none)
  FlagSlot* myFlags;                            // [nBlocks][nranks] in my heap
  FlagSlot* peerFlags[DF_MAX_RANKS];            // the same block of member j, as mapped here
  char* peerHeap[DF_MAX_RANKS];                 // heap base of member j, as mapped here
  // NVLS schedule: the arena's multicast mapping (null where the view is emulated), the members' arena
  // blocks for the emulation (host backend; null on GPUs), and this collective's staging slots in the arena
  char* mcHeap;
  char** nvlsPeers;
  uint64_t nvlsIn, nvlsOut;
  // push schedule: slot area of member j as mapped here, laid out [2 parities][nranks writers][pushSlotBytes]
  char* peerPush[DF_MAX_RANKS];
  uint64_t pushSlotBytes;
};

// ---- mutable per (block, collective) state; what a context switch saves and loads
struct alignas(16) CollDyn {
  uint64_t send, recv;    // this submission's buffers (offset or raw address, see Sqe)
  uint64_t trigger;
  uint64_t cursor;        // progress inside PH_DATA / copies when sliced
  uint32_t epoch;         // submissions of this collective seen so far
  int32_t phase;
  uint32_t sqeFlags;
  uint32_t status;
  uint64_t stallSinceNs;  // first unsuccessful poll of the current wait (0 = not stalled)
  uint32_t patience;      // polls a wait of this submission may spend at least: raised after every wait that succeeded
                          // (reference: RECV_SUCCESS_FACTOR, src/collectives_ofccl/device/ofccl_prims_simple.h:79-88)
  uint32_t pad;
};

// ---- host-pinned control words
struct DaemonCtl {
  volatile uint32_t abortFlag;     // host sets; every block leaves at its next poll
  volatile uint32_t alive;         // host sets at launch; last exiting block clears
  volatile uint32_t finalQuit;     // device sets when it consumed the quit entry
  volatile uint32_t pad;           // stream-ordered kernels store a non-zero CollStatus here on failure
  volatile uint64_t launches;
  volatile uint64_t voluntaryQuits;
  // host sets while a stream is (or will be) parked on a completion word of this context: the running
  // instance then stays resident instead of leaving when it is idle or stalled, so that no relaunch
  // from a host thread is needed at the moment the GPU waits; cleared when nothing is outstanding
  volatile uint32_t hold;
  volatile uint32_t pad1;
};

struct DevStats {                  // per block, device memory
  unsigned long long ctxSwitches, ctxSaves, ctxLoads, waitPolls, waitTimeouts, bytesReduced, bytesCopied,
      maxSwitchNs, totalSwitchNs, sqesSeen, collsDone, visits,
      yields,        // data phases left at a slice boundary because other work was queued
      passes,        // scheduler passes (trigger poll + task-queue walk + queue maintenance)
      nsTriggers, nsWalk, nsQueues;   // where thread 0 saw the passes' time go: trigger list, task-queue walk, queue upkeep
};

struct TraceEvent { uint64_t ns; uint16_t block; uint16_t event; int32_t collId; };
enum TraceKind : uint16_t { TR_SQE = 1,          // submission consumed by this block
                            TR_START = 2,        // released by its stream (or submitted from the host)
                            TR_STALL = 3,        // a wait ran out of budget: the collective stays queued, the block moves on
                            TR_ARRIVED = 4,      // every peer has arrived
                            TR_DATA_BEGIN = 5, TR_DATA_END = 6,
                            TR_DONE = 7,         // this block's part is complete (the last block publishes the completion)
                            TR_QUIT = 8, TR_LAUNCH = 9,
                            TR_PEERS_DONE = 10,  // every peer has finished its data movement
                            TR_YIELD = 11 };     // data phase left at a slice boundary

#define DF_MAX_ACTIVE 2048   // task-queue capacity per block (>= DF_MAX_COLLS: one outstanding submit per id)

struct BlockSaved {                // survives a voluntary quit (reference: DynamicBlkStatus + activeCollIds)
  uint64_t frontier;               // SQ entries consumed by this block
  uint32_t nActive;
  uint32_t exited;
  uint32_t nTrig;                  // stream-ordered submissions whose stream has not released them yet
  uint32_t pad;
  uint16_t active[DF_MAX_ACTIVE];
  uint16_t trigColl[DF_MAX_ACTIVE];
  uint32_t trigVal[DF_MAX_ACTIVE];
};

// ---- everything the daemon needs for one rank; lives in device memory (host memory for the host backend)
struct RankDev {
  // submission path: the ring and its tail live in device memory and are written by the HOST (stream memory
  // operations on a stream of its own: entry words first, then the tail), so that no block ever reads host
  // memory to find work - a load of pinned host memory costs a PCIe round trip and such loads from many blocks
  // queue behind one another
  Sqe* devSq;
  uint64_t devSqTail;
  uint32_t sqCap;                  // power of two
  uint32_t pad0;
  volatile uint64_t* hostFrontier; // pinned, [nBlocks]: entries consumed by each block (posted stores; flow control for the host)
  volatile uint32_t* abortWord;    // where this rank's abort request is polled: device memory for the daemon (the host
                                   // writes it with a stream memory operation), the pinned control block otherwise
  // completion path
  volatile uint64_t* hostCq;       // pinned ring read by the poller
  uint64_t devCqTail;
  uint32_t cqCap;                  // power of two
  uint32_t nBlocks;
  // tables
  CollStatic* colls;               // [maxColls]
  CollDyn* dyn;                    // [nBlocks][maxColls]
  uint32_t* doneCount;             // [maxColls] blocks that finished the current submission
  uint32_t* failCount;             // [maxColls] of those, how many ended with an error
  volatile uint64_t* doneEpoch;    // [maxColls] device flag: epoch of the last finished submission
  volatile uint64_t* trigger;      // [maxColls] device flag written by stream memory operations
  BlockSaved* saved;               // [nBlocks]
  DevStats* stats;                 // [nBlocks]
  TraceEvent* trace;               // ring, or null
  uint64_t traceHead;
  uint32_t traceCap;
  uint32_t maxColls;
  DaemonCtl* ctl;                  // pinned
  // tunables (reference: src/enqueue_ofccl.cc:1287-1297)
  uint32_t spinBudget;             // BASE_CTX_SWITCH_THRESHOLD
  uint32_t headTries;              // NUM_TRY_TASKQ_HEAD
  uint32_t recvSuccessFactor;      // RECV_SUCCESS_FACTOR
  uint32_t exitedBlocks;
  volatile uint32_t quitting;      // a block left voluntarily during this launch
  uint32_t saEpoch;                // stream-ordered kernels: number of collectives this communicator has finished (their epoch
                                   // lives on the device so that a captured launch finds the right one at every replay)
  uint64_t idleQuitNs;             // leave after this long with an empty task queue and no new entry
  uint64_t stallQuitNs;            // leave after this long with only stalled collectives
  uint64_t trigQuitNs;             // leave after this long with nothing but submissions that wait for their stream
  uint64_t waitTimeoutNs;          // a single wait older than this fails with ST_TIMEOUT (0 = never)
  uint64_t maxLifetimeNs;          // one launch of the daemon leaves after this long regardless of its state (0 = never)
  uint64_t sliceBytes;             // PH_DATA yields after this many bytes when others are queued (0 = never)
};

}  // namespace dfccl
