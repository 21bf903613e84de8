// The communicator object and the task/plan types of the scheduler.
// Reference parity: struct ncclComm and planner types in src/include/comm.h:120-797
// (re-designed: one symmetric-memory data plane instead of per-channel transports).
#pragma once
#include <atomic>
#include <condition_variable>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "../core/bootstrap.h"
#include "../core/core.h"
#include "mnnvl.h"

struct ncclWindow_vidmem;

namespace b200 {

constexpr int kMaxLocalRanks = 16;       // ranks that can share one load/store (NVLink) domain here
constexpr uint64_t kCommMagic = 0x42323030434f4d4dull;  // "B200COMM"

enum Func : int {
  FUNC_BROADCAST = 0, FUNC_REDUCE = 1, FUNC_ALLGATHER = 2, FUNC_REDUCESCATTER = 3, FUNC_ALLREDUCE = 4,
  FUNC_SENDRECV = 5, FUNC_SEND = 6, FUNC_RECV = 7, FUNC_ALLTOALL = 8, FUNC_SCATTER = 9, FUNC_GATHER = 10,
  FUNC_ALLGATHERV = 11, FUNC_PUTSIGNAL = 12, FUNC_SIGNAL = 13, FUNC_WAITSIGNAL = 14, FUNC_COUNT = 15
};
const char* funcName(int f);

// Algorithms of the data plane; chosen per call from the measured selection table (sched/tuning.cc) in comm/device_plane.cc.
enum Algo : int {
  ALGO_AUTO = -1,
  ALGO_ONERANK = 0,
  ALGO_LL_ONESHOT = 1,    // flagged 16-byte lines pushed to every peer, reduced by the receiver
  ALGO_P2P = 2,           // direct peer loads/stores (two-shot for all-reduce)
  ALGO_NVLS = 3,          // multimem.ld_reduce / multimem.st through the switch
  ALGO_RING = 4,          // neighbour ring over peer windows
  ALGO_TREE = 5,          // double binary tree over peer windows
  ALGO_CE = 6,            // copy engines (cudaMemcpyAsync + stream memory operations)
  ALGO_HOST = 7,          // staged through host memory and sockets
  ALGO_NVLS_ONESHOT = 8,  // all-reduce: every rank reads the whole vector with multimem.ld_reduce (small registered inputs)
  ALGO_COUNT = 9
};
const char* algoName(int a);

struct PeerInfo {
  int rank;
  int cudaDev;
  int nvmlDev;
  int64_t busId;
  uint64_t hostHash;
  uint64_t pidHash;
  int cudaCompCap;
  int mcSupport;       // device supports multicast objects
  int vmmSupport;      // device supports POSIX-fd shareable VMM handles
  uint64_t totalMem;
  int version;
  int hostOnly;        // rank has no GPU (host-memory communicator)
  FabricInfo fabric;   // NVLink fabric identity of the GPU (multi-node NVLink)
};

struct UserRedOp {
  bool used = false;
  ncclDataType_t type;
  ncclScalarResidence_t residence;
  uint64_t scalarBits;     // host-immediate scalar, widened to 8 bytes
  const void* devScalar;   // device-resident scalar
};

struct Task {
  int func;
  const void* send;
  void* recv;
  size_t count;
  ncclDataType_t type;
  int op;          // ncclRedOp_t or a user op handle
  int root;        // root rank or peer
  struct ::ncclComm* comm;
  cudaStream_t stream;
  // one-sided ops
  ncclWindow_vidmem* win = nullptr;
  size_t winOffset = 0;
  int sigIdx = 0, ctx = 0, opCnt = 0;
};

struct SymRuntime;    // mem/symmetric.h
struct HostPlane;     // host/hostcoll.cc
struct DevicePlane;   // comm/device_plane.h
struct Proxy;         // transport/proxy.h
struct RasState;
struct TopoState;
struct TunerState;
struct ProfilerState;
struct MemManager;

}  // namespace b200

struct ncclComm {
  uint64_t startMagic = b200::kCommMagic;
  int rank = 0, nRanks = 0;
  int cudaDev = -1, nvmlDev = -1;
  int compCap = 0;
  bool hostOnly = false;          // no GPU: buffers are host memory, data moves over sockets
  bool lsaAll = false;            // every rank is load/store reachable (one NVLink domain: one host, or one fabric clique across hosts)
  bool mnnvl = false;             // device memory is shared through fabric handles (the ranks' GPUs share an NVLink fabric across hosts)
  b200::Clique clique;                  // ranks of this rank's fabric clique (filled when the fabric is up on every rank)
  int node = 0, nNodes = 1, localRank = 0, localRanks = 1;
  uint64_t commHash = 0;
  ncclConfig_t config;
  std::string name;

  b200::Bootstrap* bootstrap = nullptr;
  std::vector<b200::PeerInfo> peers;

  volatile uint32_t* abortFlag = nullptr;   // host-mapped; kernels and socket loops poll it
  uint32_t* abortFlagDev = nullptr;
  volatile uint32_t* devStatus = nullptr;   // host-mapped words written by kernels on timeout
  uint32_t* devStatusDev = nullptr;
  bool revoked = false;
  bool finalized = false;

  // asynchronous state (non-blocking communicators)
  std::atomic<int> asyncResult{ncclSuccess};
  std::thread* initThread = nullptr;

  b200::HostPlane* hostPlane = nullptr;
  b200::DevicePlane* devPlane = nullptr;
  b200::SymRuntime* sym = nullptr;
  b200::Proxy* proxy = nullptr;
  b200::TopoState* topo = nullptr;
  b200::TunerState* tuner = nullptr;
  b200::ProfilerState* profiler = nullptr;
  b200::MemManager* memMgr = nullptr;

  std::vector<b200::UserRedOp> userOps;
  std::mutex lock;
  int childCount = 0;
  std::atomic<uint64_t> opCount{0};        // read by the RAS thread while the application issues work
  std::atomic<uintptr_t> launchOwner{0};   // thread that is issuing work on this communicator right now (0: none)
  ncclComm* parent = nullptr;

  // ncclCommInitAll: communicators created together in one process share a launch group
  std::vector<ncclComm*>* intraGroup = nullptr;

  uint64_t endMagic = b200::kCommMagic;
};

namespace b200 {

inline bool flagSet(const volatile uint32_t* f) { return f && __atomic_load_n((const uint32_t*)f, __ATOMIC_ACQUIRE) != 0; }   // abort flags are written by other threads
inline bool commValid(const ncclComm* c) { return c && c->startMagic == kCommMagic && c->endMagic == kCommMagic; }
ncclResult_t commEnsureReady(ncclComm* c);  // waits for / reports the state of a non-blocking init

// process-wide checkpoint calls walk the live communicators: contrib/checkpoint.cc
void checkpointCommAdd(ncclComm* comm);
void checkpointCommRemove(ncclComm* comm);

// host data plane ---------------------------------------------------------------------------
ncclResult_t hostPlaneCreate(ncclComm* comm);
void hostPlaneDestroy(ncclComm* comm);
void proxyQuiesce(ncclComm* comm);   // transport/proxy.cc: ends the progress thread of the network proxy, if there is one
ncclResult_t hostPlaneRun(ncclComm* comm, const Task& t);           // blocking, host pointers
ncclResult_t hostPlaneRunP2pGroup(ncclComm* comm, const std::vector<Task>& tasks);

// scheduler -----------------------------------------------------------------------------------
ncclResult_t enqueueTask(const Task& t);      // honours ncclGroupStart/End nesting
ncclResult_t groupStart();
ncclResult_t groupEnd(ncclSimInfo_t* sim = nullptr);
int groupDepth();
// Defers `fn` to ncclGroupEnd when called inside a group, otherwise runs it now (communicator
// creation inside groups, reference: src/group.cc:35-73).
ncclResult_t groupRunOrDefer(std::function<ncclResult_t()> fn);

// arg checks ---------------------------------------------------------------------------------
ncclResult_t argCheck(const Task& t, const char* opName);

}  // namespace b200
