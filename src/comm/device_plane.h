// GPU data plane of a communicator: the resource window (flags, flagged-line buffers, mailboxes,
// staging area), algorithm selection and kernel launches.
// Reference parity: the roles of src/enqueue.cc (plan + launch), src/sym_kernels.cc (kernel choice)
// and src/scheduler/symmetric_sched.cc in the reference, reduced to one launch per collective.
#pragma once
#include <functional>

#include "../kernels/launch.h"
#include "../mem/symmetric.h"
#include "comm.h"

namespace b200 {

struct TuneEntry { size_t upto; int algo; int mode; int ctas; };
struct TunePick { bool valid; int algo, mode, ctas; };

struct TuningTable {
  // Crossover sizes in bytes (per-rank message size of the call); measured defaults, overridable
  // with NCCL_TUNING_FILE or the NCCL_B200_* parameters.
  size_t arLLMax[kMaxRanks + 1];       // all-reduce: flagged-line one-shot up to this size
  size_t arNvlsMin[kMaxRanks + 1];     // all-reduce: multimem from this size (below: P2P two-shot)
  size_t agMcMin[kMaxRanks + 1];       // all-gather / broadcast: multimem.st from this size
  size_t rsNvlsMin[kMaxRanks + 1];     // reduce-scatter: multimem.ld_reduce from this size
  size_t rsLLMax[kMaxRanks + 1];       // reduce-scatter / reduce: flagged lines up to this many bytes per receiver
  size_t llCopyMax[kMaxRanks + 1];     // copy collectives: flagged lines up to this block size
  size_t ceMin;                        // copy-engine all-gather / all-to-all from this size (0 = never)
  int llMcMin = 0;                     // flagged lines published by multimem.st from this many ranks on (0 = never)
  int barrierMcMin = 0;                // barriers arrive by multimem.red from this many ranks on (0 = never)
  int nvlsCtas, p2pCtas, copyCtas, sendrecvCtas;
  size_t bytesPerCta;                  // grow the grid by one CTA per this many bytes
  std::vector<TuneEntry> entries[5][kMaxRanks + 1];   // measured rows per collective and rank count (sched/tuning.cc)
};

struct DevicePlane {
  void* resBase = nullptr;
  size_t resSize = 0;
  SymWindow* resWin = nullptr;
  size_t offLL = 0, offP2pLL = 0, offMailbox = 0, offStage = 0, stageBytes = 0;
  uint32_t* priv = nullptr;           // private device words: epochs, ll epoch, p2p sequence numbers
  uint32_t* epochs = nullptr;
  uint32_t* llEpoch = nullptr;
  uint32_t* p2pSeq = nullptr;
  uint64_t* sigSeen = nullptr;
  cudaEvent_t lastEvent = nullptr;
  cudaStream_t sideStream = nullptr;  // copies of pipelined staging run here, beside the kernels on the caller's stream
  cudaEvent_t pipeEv[6] = {};         // fork | piece in place [2 halves] | kernel done [2 halves] | join
  cudaStream_t lastStream = nullptr;
  bool hasLast = false;
  int smCount = 0;
  uint64_t timeoutNs = 0;
  TuningTable tune;
  void* hostStage = nullptr;          // pinned staging for the host-socket fallback
  size_t hostStageBytes = 0;
  uint64_t ceEpoch = 0;
  uint64_t launches = 0;              // kernels launched by this communicator
  void* reshardRuns = nullptr;        // device copy of the run list of the last mesh-to-mesh reshard
  size_t reshardBytes = 0;
  unsigned long long* curStamp = nullptr;   // device-visible time-stamp slot of the task being launched (set by the profiler glue)
  int barrierMcMin = 0;               // barriers arrive by multimem.red from this many ranks on (0 = never)
  int llMcMin = 0;                    // flagged lines are published by multimem.st from this many ranks on (0 = never)
};

ncclResult_t devPlaneCreate(ncclComm* comm);
void devPlaneDestroy(ncclComm* comm);
ncclResult_t devPlaneRun(ncclComm* comm, const Task& t, ncclSimInfo_t* sim = nullptr);
ncclResult_t devPlaneRunP2pGroup(ncclComm* comm, const std::vector<Task>& tasks);
// Aggregation of a group's small all-reduces into one launch (flagged lines): whether a task qualifies, and the
// launch for a run of qualifying tasks of one type, operator and stream (`taken` = how many it carried).
bool devPlaneBatchable(ncclComm* comm, const Task& t);
ncclResult_t devPlaneRunLLBatch(ncclComm* comm, const Task* tasks, int count, int* taken);
// Kernels of one communicator share its barrier slots and epochs, so they run one after the other even
// when issued on different streams: makes `stream` wait for the communicator's previous launch.
ncclResult_t devPlaneOrderStreams(ncclComm* comm, cudaStream_t stream);
// Mesh-to-mesh reshard by peer loads (contrib/m2n.cc): `runs` is what this rank pulls, in host memory; the source tiles lie in
// `win` at the byte offsets that `tileOff` (device memory, one word per rank) holds when the kernel runs.
struct ReshardRun;
ncclResult_t devPlaneRunReshard(ncclComm* comm, SymWindow* win, const ReshardRun* runs, int nRuns, const unsigned long long* tileOff, void* dst,
                                size_t totalBytes, cudaStream_t stream);
ncclResult_t devPlaneCheckStatus(ncclComm* comm);   // turns a kernel-side time-out into an async error
void tuningDefaults(TuningTable* t);
ncclResult_t tuningLoadFile(TuningTable* t, const char* path);
// Predicted duration (microseconds) of a task, used by ncclGroupSimulateEnd.
float devPlaneEstimateUs(ncclComm* comm, const Task& t);
// Forces the algorithm / copy mode of the calling thread's next launches (tuning sweeps, tests); ALGO_AUTO, -1 = automatic.
void devPlaneForce(int algo, int mode);

// measured selection table (sched/tuning.cc)
bool tuneParse(TuningTable* t, const std::string& json);
void tuneLoadDefaults(TuningTable* t);
TunePick tunePick(const TuningTable& t, int func, int n, size_t bytes);

// copy-engine collectives (sched/ce_coll.cc): releases their stream waits when the communicator is aborted or revoked
void ceCollRelease(ncclComm* comm);

// memory manager (mem/memmgr.cc): classes of tracked allocations and the tracking calls their owners make
enum MemClass : int { MEM_PERSIST = 0, MEM_SCRATCH = 1, MEM_OFFLOAD = 2 };
void memTrack(ncclComm* comm, void* ptr, size_t bytes, int cls, const char* what, SymWindow** win = nullptr, int winFlags = 0,
              size_t zeroBytes = 0, std::function<void()> afterResume = nullptr);
void memUntrack(ncclComm* comm, void* ptr);
ncclResult_t memSuspend(ncclComm* comm);
ncclResult_t memResume(ncclComm* comm);
ncclResult_t memStats(ncclComm* comm, int stat, uint64_t* value);
void memMgrDestroy(ncclComm* comm);

}  // namespace b200
