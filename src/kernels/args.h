// Kernel argument blocks shared by host and device code.
// One block (< 4 KiB, passed by value) describes a whole collective for one rank. Pointer tables
// are indexed by rank: table[p] is where rank p's buffer is mapped in the address space of the
// GPU that runs the kernel (symmetric windows), so the same block layout serves real multi-GPU
// launches and the single-GPU emulation used by unit tests, where one cooperative grid plays
// every rank (rank = blockIdx.y) over buffers that all live on one device.
// Reference parity: ncclSymkDevWorkArgs / ncclDevKernelArgs (src/include/sym_kernels.h:75-114,
// src/include/device.h:419-496) play this role in the reference.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace b200 {

constexpr int kMaxRanks = 8;            // ranks of one load/store domain served by the kernels
constexpr int kBarrierSlots = 256;      // one slot per CTA index
constexpr int kMaxCtas = 148;           // never more CTAs than SMs: CTAs of one grid wait on peers' CTAs
constexpr int kCtaThreads = 512;

// Layout of the per-rank synchronisation page (first bytes of the resource window).
constexpr size_t kInboxBytes = kBarrierSlots * kMaxRanks * sizeof(uint32_t);   // 8 KiB
constexpr int kP2pSlots = 16;                      // mailbox chunks in flight per ordered pair: 8 MiB, enough for 16 CTAs per operation to keep the links busy
constexpr size_t kP2pChunkBytes = 512 << 10;
constexpr size_t kOffP2pReady = kInboxBytes;                                        // [src][slot] u32, written by sender
constexpr size_t kOffP2pAck = kOffP2pReady + kMaxRanks * kP2pSlots * 4;             // [dst][slot] u32, written by receiver
constexpr size_t kOffSignals = kOffP2pAck + kMaxRanks * kP2pSlots * 4;              // [src][kSignalsPerPeer] u64
constexpr int kSignalsPerPeer = 64;
constexpr size_t kOffSyncEnd = kOffSignals + kMaxRanks * kSignalsPerPeer * 8;
constexpr size_t kOffP2pRdv = 14 << 10;                                             // [src][kP2pRdvLines] 16-byte rendezvous lines written by receivers
constexpr int kP2pRdvLines = 4;                                                     // large operations of one ordered pair that one launch can run in rendezvous mode
constexpr size_t kP2pDirectMin = 256 << 10;                                         // messages from this size on wait for the receiver's descriptor first
constexpr int kMaxWinSlots = 256;                                                   // windows of a communicator that the device-side table knows
constexpr size_t kOffBcastDesc = 15 << 10;                                          // one 16-byte line: where the root's send buffer is (split broadcast)
constexpr size_t kOffMcBarrier = 13 << 10;                                          // [slot] u32: arrival counters of the multicast barrier
constexpr size_t kOffRingFlags = 16 << 10;                                          // [slot][src] u32: ring step counters
constexpr size_t kOffTreeFlags = 24 << 10;                                          // [slot][tree 2][src] u32: tree phase counters
constexpr size_t kSyncPageBytes = 64 << 10;
static_assert(kOffSyncEnd <= kOffMcBarrier && kOffMcBarrier + kBarrierSlots * 4 <= kOffRingFlags, "sync page overflow");
static_assert(kOffTreeFlags + kBarrierSlots * 2 * kMaxRanks * 4 <= kSyncPageBytes, "sync page overflow");
static_assert(kOffP2pRdv + kMaxRanks * kP2pRdvLines * 16 <= kOffRingFlags, "sync page overflow");
// private per-rank words: barrier epochs | flagged-line epoch (4) | p2p sequence numbers | ring / tree step bases
constexpr size_t kPrivLLEpoch = kBarrierSlots;
constexpr size_t kPrivP2pSeq = kPrivLLEpoch + 4;
constexpr size_t kPrivRingBase = kPrivP2pSeq + 2 * kMaxRanks + 4;
constexpr size_t kPrivTreeBase = kPrivRingBase + kBarrierSlots;
constexpr size_t kPrivMcEpoch = kPrivTreeBase + kBarrierSlots;       // epochs of the multicast barrier, per slot
constexpr size_t kPrivP2pDone = kPrivMcEpoch + kBarrierSlots;        // finished CTAs per operation of a send/recv launch
constexpr size_t kPrivWords = kPrivP2pDone + 32;

constexpr size_t kLLDataBytes = 1 << 20;                     // largest payload of the flagged-line protocol
constexpr size_t kLLLines = kLLDataBytes / 8;                // 8 payload bytes per 16-byte line
constexpr size_t kLLRegionBytes = 2 * kMaxRanks * kLLLines * 16;   // [parity][src][line]
constexpr size_t kMailboxBytes = (size_t)kMaxRanks * kP2pSlots * kP2pChunkBytes;  // [src][slot][chunk]
// Small sends travel as flagged 16-byte lines (8 payload bytes + the chunk's sequence number twice): no fence and no
// separate ready flag. The lines have an area of their own, so a line never holds anything but older lines.
constexpr size_t kP2pLLMax = 16384;                                              // largest message sent as flagged lines
constexpr size_t kP2pLLSlotBytes = kP2pLLMax * 2;
constexpr size_t kP2pLLBytes = (size_t)kMaxRanks * kP2pSlots * kP2pLLSlotBytes;   // [src][slot][line]

enum DevStatus : uint32_t { DEV_OK = 0, DEV_TIMEOUT = 1, DEV_ABORTED = 2 };
enum DevWaitKind : uint32_t { WAIT_BARRIER = 1, WAIT_LL = 2, WAIT_P2P_READY = 3, WAIT_P2P_ACK = 4, WAIT_SIGNAL = 5, WAIT_TILE = 6 };

struct SyncArgs {
  uint32_t* inbox[kMaxRanks];     // inbox[p]: rank p's barrier inbox [slot][src]
  uint32_t* epoch[kMaxRanks];     // epoch[r]: rank r's private epoch counters [slot]
  uint32_t* status[kMaxRanks];    // status[r]: {code, kind, peer, expected} written on a failed wait
  uint32_t* mcArrive;             // multicast alias of the barrier arrival counters [slot] (null: unicast barrier)
  const uint32_t* abortFlag;      // set by the host to make every wait give up
  unsigned long long timeoutNs;   // budget of one wait
  unsigned long long* stamps;     // time stamps of this launch for profiler plugins: [kStampCtas][2] = {start, stop} of CTA i in
                                  // nanoseconds of the GPU's global timer (null: not recorded)
};
constexpr int kStampCtas = 32;    // CTAs of a launch that record their start and stop (the first ones of the grid)

enum RedOp : int { RED_SUM = 0, RED_PROD = 1, RED_MAX = 2, RED_MIN = 3 };
enum ScaleMode : int { SCALE_NONE = 0, SCALE_MUL = 1, SCALE_INTDIV = 2 };

enum CollMode : int {
  MODE_PUSH = 0,     // writer stores into peers' buffers
  MODE_PULL = 1,     // reader loads from peers' buffers
  MODE_MC = 2,       // one multimem.st stream reaches every peer
  MODE_SPLIT = 3,    // broadcast only: the other ranks each pull a share of the root's buffer and store it to all of them
  MODE_BULK = 4,     // flag added to a mode when it is forced or tabled: moved by bulk-copy engines (few CTAs) instead of threads
};

struct CollArgs {
  int rank, nRanks;
  int emu;                              // 1: blockIdx.y selects the rank
  int func;                             // Func
  int root;
  int mode;                             // CollMode (copy collectives)
  int vec16;                            // every pointer and slice is 16-byte aligned
  int dstAll;                           // reductions: store the result to every rank (all-reduce) or locally
  const void* send[kMaxRanks];          // peer-visible inputs
  void* recv[kMaxRanks];                // peer-visible outputs
  const void* lsend[kMaxRanks];         // rank-private input pointers (lsend[r] is only touched by rank r)
  void* lrecv[kMaxRanks];               // rank-private output pointers
  const void* sendMc;                   // multicast alias of send (NVLS) or null
  void* recvMc;                         // multicast alias of recv
  size_t count;                         // elements: all-reduce/broadcast/reduce total; per-rank block otherwise
  size_t sendStride, recvStride;        // copy collectives: bytes between consecutive blocks of the input / output
  size_t sliceBegin[kMaxRanks];         // reductions: first element reduced by rank r
  size_t sliceCount[kMaxRanks];         // reductions: number of elements reduced by rank r
  size_t dstOff[kMaxRanks];             // reductions: element offset of rank r's result inside the output
  int scaleMode;
  float scaleF;
  double scaleD;
  long long intDiv;
  SyncArgs sync;
  // flagged-line (LL) resources
  void* ll[kMaxRanks];                  // ll[p]: rank p's LL region
  uint32_t* llEpoch[kMaxRanks];         // llEpoch[r]: {epoch, finished CTAs} private to rank r
  char* llMc;                           // multicast alias of the flagged-line region (null: unicast stores only)
  // split broadcast: where the root's send buffer is. The root fills bcastSlot (window slot + 1, 0 = not in a window) and
  // bcastOff and publishes them from the kernel; the emulation passes send[root] instead and leaves winTable null.
  void* const* winTable;                // device table [window slot][rank] of peer mappings
  int bcastSlot;
  unsigned long long bcastOff;
};

// Several small all-reduces of one group carried by one launch of the flagged-line kernel: item i
// owns lines [lineOff, lineOff + ceil(count * elemSize / 8)) of every region; buffers are given as
// byte offsets from lsend[rank] / lrecv[rank] (null bases outside the emulation, so the offsets are
// plain addresses there).
struct LLItem {
  long long sendOff, recvOff;
  uint32_t count;        // elements
  uint32_t lineOff;
};
constexpr int kMaxLLItems = 64;
struct LLBatchArgs {
  CollArgs c;            // c.count unused; func = all-reduce
  int nItems;
  uint32_t totalLines;
  LLItem items[kMaxLLItems];
};

struct P2pOp {
  int peer;
  int isSend;
  void* buf;             // rank-private user buffer
  size_t bytes;
  int ctaBegin, ctaCount;   // CTAs [ctaBegin, ctaBegin+ctaCount) of the grid serve this op
  uint32_t seqOffset;       // mailbox chunks of earlier ops of this launch with the same peer and direction
  // rendezvous mode (bytes >= kP2pDirectMin and rdvLine >= 0): the receiver tells the sender where the data goes
  int rdvLine;              // which of the pair's rendezvous lines this op uses (its ordinal among the pair's large ops of the launch), -1: none
  int winSlot;              // receive side: slot of the window that holds `buf` in the device-side table, -1: not in a peer-mapped window
  size_t winOff;            // receive side: offset of `buf` inside that window
};
constexpr int kMaxP2pOps = 32;
static_assert(kMaxP2pOps <= 32, "per-operation counters");

// Chunk size of a message in the mailbox protocol: both sides derive it from the byte count. About sixteen
// chunks per message (so that as many CTAs share it), between 64 KiB and the slot size.
#if defined(__CUDACC__)
__host__ __device__
#endif
inline size_t p2pChunkOf(size_t bytes) {
  size_t c = ((bytes + 15) / 16 + 65535) / 65536 * 65536;
  if (c < 65536) c = 65536;
  return c > kP2pChunkBytes ? kP2pChunkBytes : c;
}

struct P2pArgs {
  int rank, nRanks;
  int emu;
  int nOps[kMaxRanks];                   // ops of rank r (only [rank] outside emulation)
  P2pOp ops[kMaxP2pOps];                 // emulation packs every rank's ops back to back: opBase[r]
  int opBase[kMaxRanks];
  char* mailbox[kMaxRanks];              // mailbox[p]: rank p's mailbox region [src][slot][chunk]
  char* llbox[kMaxRanks];                // llbox[p]: rank p's flagged-line area for small messages [src][slot][line]
  uint32_t* ready[kMaxRanks];            // ready[p]: rank p's [src][slot] flags
  uint32_t* ack[kMaxRanks];              // ack[p]: rank p's [dst][slot] flags
  uint32_t* seq[kMaxRanks];              // seq[r]: private counters {send[kMaxRanks], recv[kMaxRanks]}
  void* rdv[kMaxRanks];                  // rdv[p]: rank p's rendezvous lines [src][kP2pRdvLines], written by the receivers of p's sends
  uint32_t* opDone[kMaxRanks];           // opDone[r]: private [kMaxP2pOps] counters of finished CTAs per operation
  void* const* winTable;                 // device table [kMaxWinSlots][kMaxRanks]: where window slot w of rank p is mapped here (null: no rendezvous mode)
  SyncArgs sync;
};

// Mesh-to-mesh resharding by peer loads: every destination rank pulls the runs of its tile straight out of the source
// ranks' tiles, which lie in a registered window.
struct ReshardRun {
  unsigned long long srcOff;   // bytes from the start of the source rank's tile
  unsigned long long dstOff;   // bytes from the start of this rank's destination tile
  unsigned long long bytes;
  int srcRank;
  int pad;
};
struct ReshardArgs {
  int rank, nRanks, emu;
  int nRuns;                              // runs this rank pulls
  const ReshardRun* runs;                 // device memory
  const char* winPeer[kMaxRanks];         // winPeer[p]: rank p's part of the window as mapped here
  const unsigned long long* tileOff;      // device memory [nRanks]: byte offset of rank p's source tile inside the window (all-gathered just before)
  char* dst;                              // this rank's destination tile
  SyncArgs sync;
};

struct SignalArgs {
  int rank, nRanks;
  uint64_t* signals[kMaxRanks];          // signals[p]: rank p's [src][kSignalsPerPeer] counters
  uint64_t* seen;                        // private [src][kSignalsPerPeer]: how many were consumed
  SyncArgs sync;
};

}  // namespace b200
