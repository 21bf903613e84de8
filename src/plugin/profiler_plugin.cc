// External profiler plugin glue. Events sent to a plugin exporting ncclProfiler_v6:
//   GroupApi / CollApi / P2pApi   around each public call (and its group)
//   KernelLaunch                  around each kernel launch of the data plane
//   Group -> Coll / P2p           one per task that reaches the data plane, with algorithm names
//   KernelCh                      device-side execution window of the task's kernels: a pair of
//                                 CUDA events around the launches, polled at later API calls;
//                                 pTimer values are nanoseconds on the host clock of the start
//                                 event plus the measured device duration
// Reference parity: src/plugin/profiler.cc (load :46-113, init/finalize :245-263, API events
// :275-386, kernel launch :388-430, group/task :432-565, kernel channel :679-705).
#include <cuda_runtime.h>

#include <deque>
#include <mutex>

#include "../comm/device_plane.h"
#include "../kernels/args.h"
#include "plugin.h"
#include "profiler.h"

namespace b200 {

static const char* kTypeNames[] = {"ncclInt8", "ncclUint8", "ncclInt32", "ncclUint32", "ncclInt64", "ncclUint64", "ncclFloat16", "ncclFloat32",
                                   "ncclFloat64", "ncclBfloat16", "ncclFloat8e4m3", "ncclFloat8e5m2"};
static const char* typeName(int t) { return t >= 0 && t < 12 ? kTypeNames[t] : "unknown"; }

struct PendingKernel {
  cudaEvent_t start, stop;
  void* collHandle;
  void* groupHandle;
  uint64_t hostStartNs;
  int stampSlot;   // slot of the device time stamps (-1: none)
};

// Device time stamps: a ring of slots in pinned host memory that the kernels write through a device mapping
// ([kStampCtas][2] words per slot, see KernelStamp in kernels/common.cuh). A slot belongs to one task from its
// launch until its stop event has completed and the stamps have been turned into KernelCh events.
constexpr int kStampSlots = 256;
constexpr int kStampWords = 2 * kStampCtas;

struct ProfilerExtra {
  std::mutex lock;
  std::deque<PendingKernel> pending;
  std::vector<cudaEvent_t> pool;
  unsigned long long* stampHost = nullptr;
  unsigned long long* stampDev = nullptr;
  std::vector<int> freeSlots;
  bool stampTried = false;
};

static int takeStampSlot(ProfilerExtra* ex) {
  std::lock_guard<std::mutex> g(ex->lock);
  if (!ex->stampTried) {
    ex->stampTried = true;
    void* h = nullptr;
    void* d = nullptr;
    if (cudaHostAlloc(&h, sizeof(unsigned long long) * kStampSlots * kStampWords, cudaHostAllocMapped) == cudaSuccess &&
        cudaHostGetDevicePointer(&d, h, 0) == cudaSuccess) {
      ex->stampHost = (unsigned long long*)h;
      ex->stampDev = (unsigned long long*)d;
      for (int i = kStampSlots - 1; i >= 0; --i) ex->freeSlots.push_back(i);
    } else {
      (void)cudaGetLastError();
      if (h) cudaFreeHost(h);
    }
  }
  if (ex->freeSlots.empty()) return -1;
  int slot = ex->freeSlots.back();
  ex->freeSlots.pop_back();
  memset(ex->stampHost + (size_t)slot * kStampWords, 0, sizeof(unsigned long long) * kStampWords);
  return slot;
}
static std::mutex gExtraLock;
static std::map<ncclComm*, ProfilerExtra*> gExtra;

static ProfilerExtra* extraOf(ncclComm* comm, bool create) {
  std::lock_guard<std::mutex> g(gExtraLock);
  auto it = gExtra.find(comm);
  if (it != gExtra.end()) return it->second;
  if (!create) return nullptr;
  return gExtra[comm] = new ProfilerExtra;
}

ncclResult_t profilerLoad(ncclComm* comm) {
  std::string resolved;
  void* lib = pluginOpen(PLUGIN_PROFILER, &resolved);
  if (!lib) return ncclSuccess;
  ncclProfiler_v6_t* p = (ncclProfiler_v6_t*)pluginSymbol(lib, NCCL_PROFILER_PLUGIN_SYMBOL);
  bool v5 = false;
  if (!p) {
    // The v5 table has the same entry points and its event descriptor is the v6 one without the copy-engine events at the
    // end of the union: a v5 plugin is driven through the same calls with those three event types masked off.
    p = (ncclProfiler_v6_t*)pluginSymbol(lib, "ncclProfiler_v5");
    v5 = p != nullptr;
  }
  if (!p) { WARN("profiler plugin %s exports neither %s nor ncclProfiler_v5 (older interfaces are not supported)", resolved.c_str(), NCCL_PROFILER_PLUGIN_SYMBOL); return ncclSuccess; }
  ProfilerState* ps = new ProfilerState;
  ps->lib = lib;
  ps->prof = p;
  ps->name = p->name ? p->name : resolved;
  int mask = 0;
  const char* m = getEnv("NCCL_PROFILE_EVENT_MASK");
  if (m && *m) mask = (int)strtol(m, nullptr, 0);
  ncclResult_t r = p->init(&ps->ctx, comm->commHash, &mask, comm->name.c_str(), comm->nNodes, comm->nRanks, comm->rank, pluginLogger);
  if (r != ncclSuccess) { WARN("profiler plugin %s failed to initialise (%d)", ps->name.c_str(), (int)r); delete ps; return ncclSuccess; }
  if (v5) mask &= ~(ncclProfileCeColl | ncclProfileCeSync | ncclProfileCeBatch);
  ps->mask = mask;
  comm->profiler = ps;
  INFO(SUB_PROFILE, "profiler plugin %s (%s, interface v%d) attached, event mask 0x%x", ps->name.c_str(), resolved.c_str(), v5 ? 5 : 6, mask);
  return ncclSuccess;
}

void profilerPoll(ncclComm* comm, bool drain);

void profilerUnload(ncclComm* comm) {
  ProfilerState* ps = comm->profiler;
  if (!ps) return;
  profilerPoll(comm, true);
  if (ps->prof->finalize) ps->prof->finalize(ps->ctx);
  ProfilerExtra* ex = extraOf(comm, false);
  if (ex) {
    for (cudaEvent_t e : ex->pool) cudaEventDestroy(e);
    if (ex->stampHost) cudaFreeHost(ex->stampHost);
    (void)cudaGetLastError();
    {
      std::lock_guard<std::mutex> g(gExtraLock);
      gExtra.erase(comm);
    }
    delete ex;
  }
  delete ps;
  comm->profiler = nullptr;
}

void* profStart(ncclComm* comm, ncclProfilerEventDescr_t* d) {
  ProfilerState* ps = comm->profiler;
  if (!ps || !(ps->mask & (int)d->type)) return nullptr;
  d->rank = comm->rank;
  void* h = nullptr;
  if (ps->prof->startEvent(ps->ctx, &h, d) != ncclSuccess) return nullptr;
  return h;
}
void profStop(ncclComm* comm, void* h) {
  if (h && comm->profiler) comm->profiler->prof->stopEvent(h);
}
void profState(ncclComm* comm, void* h, ncclProfilerEventState_t st, ncclProfilerEventStateArgs_t* a) {
  if (h && comm->profiler && comm->profiler->prof->recordEventState) comm->profiler->prof->recordEventState(h, st, a);
}

// ---- events of network backends
// A handle of such an event remembers its communicator (stop and update arrive with the handle only).
struct NetEvent { ncclComm* comm; void* handle; };
ncclResult_t profilerNetCallback(void** eHandle, int type, void* pHandle, int64_t pluginId, void* extData) {
  if (!eHandle) return ncclSuccess;
  if (type == ncclProfilerNetEventStart) {
    *eHandle = nullptr;
    ProfNetParent* pp = (ProfNetParent*)pHandle;
    if (!pp || !pp->comm || !pp->comm->profiler) return ncclSuccess;
    ncclProfilerEventDescr_t d;
    memset(&d, 0, sizeof(d));
    d.type = ncclProfileNetPlugin;
    d.parentObj = pp->parent;
    d.netPlugin.id = pluginId;
    d.netPlugin.data = extData;
    void* h = profStart(pp->comm, &d);
    if (h) *eHandle = new NetEvent{pp->comm, h};
    return ncclSuccess;
  }
  NetEvent* ev = (NetEvent*)*eHandle;
  if (!ev) return ncclSuccess;
  if (type == ncclProfilerNetEventUpdate || type == ncclProfilerNetEventUpdateAndStop) {
    ncclProfilerEventStateArgs_t a;
    memset(&a, 0, sizeof(a));
    a.netPlugin.data = extData;
    profState(ev->comm, ev->handle, ncclProfilerNetPluginUpdate, &a);
  }
  if (type == ncclProfilerNetEventStop || type == ncclProfilerNetEventUpdateAndStop) {
    profStop(ev->comm, ev->handle);
    delete ev;
    *eHandle = nullptr;
  }
  return ncclSuccess;
}

// ---- copy-engine collectives
// Reference parity: CeColl / CeSync / CeBatch events of src/ce_coll.cc:133-285, :497-717.
void* profilerCeStart(ncclComm* comm, const Task& t, int what, void* parent, int numOps, size_t totalBytes) {
  ProfilerState* ps = comm->profiler;
  if (!ps) return nullptr;
  ncclProfilerEventDescr_t d;
  memset(&d, 0, sizeof(d));
  d.parentObj = parent;
  if (what == 0) {
    d.type = ncclProfileCeColl;
    d.ceColl.seqNumber = t.func < FUNC_COUNT ? ps->seq[t.func]++ : 0;
    d.ceColl.func = funcName(t.func);
    d.ceColl.sendBuff = t.send;
    d.ceColl.recvBuff = t.recv;
    d.ceColl.count = t.count;
    d.ceColl.root = t.root;
    d.ceColl.datatype = typeName(t.type);
    d.ceColl.syncStrategy = "stream memory operations";
    d.ceColl.intraBatchSync = false;
    d.ceColl.batchSize = (uint32_t)numOps;
    d.ceColl.numBatches = 1;
    d.ceColl.ceSeqNum = (uint32_t)(comm->devPlane ? comm->devPlane->ceEpoch / 2 : 0);
    d.ceColl.stream = (void*)t.stream;
  } else if (what == 1) {
    d.type = ncclProfileCeSync;
    d.ceCollSync.isComplete = numOps != 0;   // the closing barrier of the call
    d.ceCollSync.nRanks = comm->nRanks;
  } else {
    d.type = ncclProfileCeBatch;
    d.ceCollBatch.numOps = numOps;
    d.ceCollBatch.totalBytes = totalBytes;
    d.ceCollBatch.useIntraSync = false;
  }
  void* h = profStart(comm, &d);
  if (h) profState(comm, h, what == 0 ? ncclProfilerCeCollStart : what == 1 ? ncclProfilerCeSyncStart : ncclProfilerCeBatchStart, nullptr);
  return h;
}
void profilerCeStop(ncclComm* comm, void* h, int what) {
  if (!h) return;
  profState(comm, h, what == 0 ? ncclProfilerCeCollComplete : what == 1 ? ncclProfilerCeSyncComplete : ncclProfilerCeBatchComplete, nullptr);
  profStop(comm, h);
}

// ---- public-call events (called through ProfilerApiScope)
struct ApiPluginHandle {
  ncclComm* comm;
  void* group;
  void* api;
};

void* profilerPluginStart(ncclComm* comm, const Task& t) {
  if (!comm->profiler) return nullptr;
  profilerPoll(comm, false);
  ApiPluginHandle* h = new ApiPluginHandle{comm, nullptr, nullptr};
  ncclProfilerEventDescr_t d;
  memset(&d, 0, sizeof(d));
  d.type = ncclProfileGroupApi;
  d.groupApi.groupDepth = groupDepth();
  h->group = profStart(comm, &d);
  memset(&d, 0, sizeof(d));
  const bool p2p = t.func == FUNC_SEND || t.func == FUNC_RECV;
  d.parentObj = h->group;
  if (p2p) {
    d.type = ncclProfileP2pApi;
    d.p2pApi.func = funcName(t.func);
    d.p2pApi.count = t.count;
    d.p2pApi.datatype = typeName(t.type);
    d.p2pApi.stream = (void*)t.stream;
  } else {
    d.type = ncclProfileCollApi;
    d.collApi.func = funcName(t.func);
    d.collApi.count = t.count;
    d.collApi.datatype = typeName(t.type);
    d.collApi.root = t.root;
    d.collApi.stream = (void*)t.stream;
  }
  h->api = profStart(comm, &d);
  return h;
}

void profilerPluginStop(void* hv) {
  ApiPluginHandle* h = (ApiPluginHandle*)hv;
  profStop(h->comm, h->api);
  profStop(h->comm, h->group);
  delete h;
}

// ---- task events (data plane)
struct TaskProfile {
  void* group = nullptr;
  void* coll = nullptr;
  void* launch = nullptr;
  cudaEvent_t start = nullptr, stop = nullptr;
  uint64_t hostStartNs = 0;
  int stampSlot = -1;
};

static cudaEvent_t takeEvent(ProfilerExtra* ex) {
  {
    std::lock_guard<std::mutex> g(ex->lock);
    if (!ex->pool.empty()) { cudaEvent_t e = ex->pool.back(); ex->pool.pop_back(); return e; }
  }
  cudaEvent_t e = nullptr;
  if (cudaEventCreate(&e) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
  return e;
}

// Called before the data plane chooses and launches: records the device-side start marker.
void* profilerTaskStart(ncclComm* comm, const Task& t) {
  ProfilerState* ps = comm->profiler;
  if (!ps) return nullptr;
  TaskProfile* tp = new TaskProfile;
  tp->hostStartNs = nowNs();
  // device window: only outside stream capture (captured events cannot be queried)
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if ((ps->mask & ncclProfileKernelCh) && !comm->hostOnly && cudaStreamIsCapturing(t.stream, &cs) == cudaSuccess && cs == cudaStreamCaptureStatusNone) {
    ProfilerExtra* ex = extraOf(comm, true);
    tp->start = takeEvent(ex);
    tp->stop = takeEvent(ex);
    if (tp->start && tp->stop) {
      cudaEventRecord(tp->start, t.stream);
      tp->stampSlot = takeStampSlot(ex);
      if (tp->stampSlot >= 0 && comm->devPlane) comm->devPlane->curStamp = ex->stampDev + (size_t)tp->stampSlot * kStampWords;
    }
  }
  (void)cudaGetLastError();
  return tp;
}

// Called after the launches: by now the algorithm is known, so the task events carry its name.
void profilerTaskStop(ncclComm* comm, const Task& t, void* hv, const char* algo, const char* proto, int nCtas) {
  TaskProfile* tp = (TaskProfile*)hv;
  ProfilerState* ps = comm->profiler;
  if (comm->devPlane) comm->devPlane->curStamp = nullptr;
  if (!tp) return;
  if (!ps) { delete tp; return; }
  ncclProfilerEventDescr_t d;
  memset(&d, 0, sizeof(d));
  d.type = ncclProfileGroup;
  tp->group = profStart(comm, &d);
  memset(&d, 0, sizeof(d));
  d.parentObj = tp->group;
  if (t.func == FUNC_SEND || t.func == FUNC_RECV) {
    d.type = ncclProfileP2p;
    d.p2p.func = funcName(t.func);
    d.p2p.buff = t.func == FUNC_SEND ? (void*)t.send : t.recv;
    d.p2p.datatype = typeName(t.type);
    d.p2p.count = t.count;
    d.p2p.peer = t.root;
    d.p2p.nChannels = (uint8_t)std::min(nCtas, 255);
    d.p2p.parentGroup = tp->group;
  } else {
    d.type = ncclProfileColl;
    d.coll.seqNumber = t.func < FUNC_COUNT ? ps->seq[t.func]++ : 0;
    d.coll.func = funcName(t.func);
    d.coll.sendBuff = t.send;
    d.coll.recvBuff = t.recv;
    d.coll.count = t.count;
    d.coll.root = t.root;
    d.coll.datatype = typeName(t.type);
    d.coll.nChannels = (uint8_t)std::min(nCtas, 255);
    d.coll.nWarps = 16;
    d.coll.algo = algo;
    d.coll.proto = proto;
    d.coll.parentGroup = tp->group;
  }
  tp->coll = profStart(comm, &d);
  memset(&d, 0, sizeof(d));
  d.type = ncclProfileKernelLaunch;
  d.parentObj = tp->coll;
  d.kernelLaunch.stream = (void*)t.stream;
  tp->launch = profStart(comm, &d);
  profStop(comm, tp->launch);
  if (tp->start && tp->stop) {
    cudaEventRecord(tp->stop, t.stream);
    ProfilerExtra* ex = extraOf(comm, true);
    std::lock_guard<std::mutex> g(ex->lock);
    ex->pending.push_back(PendingKernel{tp->start, tp->stop, tp->coll, tp->group, tp->hostStartNs, tp->stampSlot});
  } else {
    profStop(comm, tp->coll);
    profStop(comm, tp->group);
  }
  (void)cudaGetLastError();
  delete tp;
}

// Closes the task events whose kernels have finished (all of them, waiting, when drain is set).
void profilerPoll(ncclComm* comm, bool drain) {
  ProfilerExtra* ex = extraOf(comm, false);
  if (!ex) return;
  for (;;) {
    PendingKernel pk;
    {
      std::lock_guard<std::mutex> g(ex->lock);
      if (ex->pending.empty()) return;
      pk = ex->pending.front();
      cudaError_t q = drain ? cudaEventSynchronize(pk.stop) : cudaEventQuery(pk.stop);
      if (q == cudaErrorNotReady) { (void)cudaGetLastError(); return; }
      ex->pending.pop_front();
    }
    // one KernelCh event per CTA that stamped its start and stop on the device (GPU global timer, nanoseconds)
    int stamped = 0;
    if (pk.stampSlot >= 0) {
      const unsigned long long* st = ex->stampHost + (size_t)pk.stampSlot * kStampWords;
      for (int c = 0; c < kStampCtas; ++c) {
        if (st[2 * c] == 0 || st[2 * c + 1] < st[2 * c]) continue;
        ncclProfilerEventDescr_t d;
        memset(&d, 0, sizeof(d));
        d.type = ncclProfileKernelCh;
        d.parentObj = pk.collHandle;
        d.kernelCh.channelId = (uint8_t)c;
        d.kernelCh.pTimer = st[2 * c];
        void* h = profStart(comm, &d);
        ncclProfilerEventStateArgs_t a;
        memset(&a, 0, sizeof(a));
        a.kernelCh.pTimer = st[2 * c + 1];
        profState(comm, h, ncclProfilerKernelChStop, &a);
        profStop(comm, h);
        ++stamped;
      }
    }
    if (stamped == 0) {
      // nothing stamped (copy engines, stream memory operations): one record from the bracketing events on the host clock
      float ms = 0;
      if (cudaEventElapsedTime(&ms, pk.start, pk.stop) != cudaSuccess) { (void)cudaGetLastError(); ms = 0; }
      ncclProfilerEventDescr_t d;
      memset(&d, 0, sizeof(d));
      d.type = ncclProfileKernelCh;
      d.parentObj = pk.collHandle;
      d.kernelCh.channelId = 0;
      d.kernelCh.pTimer = pk.hostStartNs;
      void* h = profStart(comm, &d);
      ncclProfilerEventStateArgs_t a;
      memset(&a, 0, sizeof(a));
      a.kernelCh.pTimer = pk.hostStartNs + (uint64_t)(ms * 1e6);
      profState(comm, h, ncclProfilerKernelChStop, &a);
      profStop(comm, h);
    }
    profStop(comm, pk.collHandle);
    profStop(comm, pk.groupHandle);
    std::lock_guard<std::mutex> g(ex->lock);
    ex->pool.push_back(pk.start);
    ex->pool.push_back(pk.stop);
    if (pk.stampSlot >= 0) ex->freeSlots.push_back(pk.stampSlot);
  }
}

void profilerCommInit(ncclComm* comm) { profilerLoad(comm); }
void profilerCommFini(ncclComm* comm) { profilerUnload(comm); }

}  // namespace b200
