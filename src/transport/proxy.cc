// Proxy: the service thread of a communicator that moves host-memory messages through the
// network backend. Callers post send / receive operations; the thread cuts each into slices,
// keeps several slices per operation in flight (isend / irecv), polls test(), and marks the
// operation done. proxyCreate wires a full mesh: every rank listens, handles are all-gathered
// through the bootstrap ring, lower ranks connect first to higher ones and accept afterwards.
// Reference parity: src/proxy.cc (ncclProxySaveOp :602, progress loop :954, service thread
// :1713), src/transport/net.cc (sendProxyProgress :1304-1468, recvProxyProgress :1470-1765).
#include <signal.h>

#include <ctype.h>
#include <limits.h>
#include <stdlib.h>

#include "net.h"

#include <sched.h>
#include <unistd.h>

#include "../plugin/plugin.h"

namespace b200 {

B200_PARAM(NetSliceKb, "B200_NET_SLICE_KB", 512, "slice size of proxy network operations, KiB");
B200_PARAM(NetInflight, "B200_NET_INFLIGHT", 8, "slices of one proxy operation kept in flight");

static constexpr int kTagNetMesh = BS_TAG_USER + 7;

static void profProxyOp(Proxy* p, ProxyOp* op, bool start) {
  ncclComm* comm = p->comm;
  if (!comm->profiler) return;
  if (start) {
    ncclProfilerEventDescr_t d;
    memset(&d, 0, sizeof(d));
    d.type = ncclProfileProxyOp;
    d.proxyOp.pid = getpid();
    d.proxyOp.peer = op->peer;
    d.proxyOp.nSteps = (int)((op->bytes + p->sliceBytes - 1) / p->sliceBytes);
    d.proxyOp.chunkSize = (int)std::min<size_t>(p->sliceBytes, op->bytes);
    d.proxyOp.isSend = op->isSend ? 1 : 0;
    op->profHandle = profStart(comm, &d);
  } else if (op->profHandle) {
    for (void*& h : op->stepHandle) if (h) { profStop(comm, h); h = nullptr; }
    if (op->nextStep) { profStop(comm, op->nextStep); op->nextStep = nullptr; }
    profStop(comm, op->profHandle);
    op->profHandle = nullptr;
  }
}

// The whole buffer of an operation is registered once with the backend (a no-op for sockets, a memory region for verbs), so
// that its slices do not register one by one.
static void opRegister(Proxy* p, ProxyOp* op) {
  op->regTried = true;
  void* comm = op->isSend ? p->sendComm[op->peer] : p->recvComm[op->peer];
  if (!p->net->regMr || !comm || op->bytes == 0) return;
  if (p->net->regMr(comm, op->data, op->bytes, NCCL_PTR_HOST, &op->mhandle) != ncclSuccess) op->mhandle = nullptr;
}
static void opRelease(Proxy* p, ProxyOp* op) {
  if (!op->mhandle) return;
  void* comm = op->isSend ? p->sendComm[op->peer] : p->recvComm[op->peer];
  if (p->net->deregMr && comm) p->net->deregMr(comm, op->mhandle);
  op->mhandle = nullptr;
}

static ncclResult_t progressOp(Proxy* p, ProxyOp* op) {
  ncclNet_t* net = p->net;
  if (!op->regTried) opRegister(p, op);
  // post new slices
  while (op->posted < op->bytes && op->tail - op->head < p->maxInflight) {
    size_t n = std::min(p->sliceBytes, op->bytes - op->posted);
    void* req = nullptr;
    char* ptr = op->data + op->posted;
    const int slot = op->tail % NCCL_NET_MAX_REQUESTS;
    if (op->profHandle && !op->nextStep) {
      ncclProfilerEventDescr_t d;
      memset(&d, 0, sizeof(d));
      d.type = ncclProfileProxyStep;
      d.parentObj = op->profHandle;
      d.proxyStep.step = op->stepsStarted++;
      op->nextStep = profStart(p->comm, &d);
    }
    op->stepParent[slot] = ProfNetParent{p->comm, op->nextStep ? op->nextStep : op->profHandle};
    void* ph = op->profHandle ? (void*)&op->stepParent[slot] : nullptr;
    if (op->isSend) {
      NCCLCHECK(net->isend(p->sendComm[op->peer], ptr, n, 0, op->mhandle, ph, &req));
    } else {
      void* ptrs[1] = {ptr};
      size_t sizes[1] = {n};
      int tags[1] = {0};
      void* mh[1] = {op->mhandle};
      void* phs[1] = {ph};
      NCCLCHECK(net->irecv(p->recvComm[op->peer], 1, ptrs, sizes, tags, mh, phs, &req));
    }
    if (!req) break;   // the backend is out of request slots: try again later
    op->requests[slot] = req;
    op->reqBytes[slot] = n;
    op->stepHandle[slot] = op->nextStep;
    op->nextStep = nullptr;
    if (op->stepHandle[slot]) {
      ncclProfilerEventStateArgs_t a;
      memset(&a, 0, sizeof(a));
      a.proxyStep.transSize = n;
      profState(p->comm, op->stepHandle[slot], op->isSend ? ncclProfilerProxyStepSendWait : ncclProfilerProxyStepRecvWait, &a);
    }
    op->tail++;
    op->posted += n;
    p->steps++;
  }
  // complete in order
  while (op->head < op->tail) {
    int slot = op->head % NCCL_NET_MAX_REQUESTS;
    int done = 0, size = 0;
    NCCLCHECK(net->test(op->requests[slot], &done, &size));
    if (!done) break;
    if (op->stepHandle[slot]) { profStop(p->comm, op->stepHandle[slot]); op->stepHandle[slot] = nullptr; }
    op->completed += op->reqBytes[slot];
    p->bytesMoved += op->reqBytes[slot];
    op->head++;
  }
  // zero-byte operations still exchange one empty message so that both sides match
  if (op->bytes == 0 && op->posted == 0 && op->tail == 0) {
    void* req = nullptr;
    static char dummy;
    if (op->isSend) NCCLCHECK(net->isend(p->sendComm[op->peer], &dummy, 0, 0, nullptr, nullptr, &req));
    else {
      void* ptrs[1] = {&dummy};
      size_t sizes[1] = {0};
      int tags[1] = {0};
      void* mh[1] = {nullptr};
      void* ph[1] = {nullptr};
      NCCLCHECK(net->irecv(p->recvComm[op->peer], 1, ptrs, sizes, tags, mh, ph, &req));
    }
    if (req) { op->requests[0] = req; op->reqBytes[0] = 0; op->tail = 1; }
  }
  return ncclSuccess;
}

static bool opFinished(const ProxyOp* op) { return op->head == op->tail && op->posted >= op->bytes && (op->bytes > 0 || op->tail > 0); }

// NCCL_PROXY_DUMP_SIGNAL=<signal number>: on that signal every proxy thread logs its operations in flight
// (reference: ncclDumpProxyState, src/proxy.cc:920-965, installed for the same variable). The handler only
// bumps a counter; the threads print from their own loop.
static std::atomic<unsigned> gDumpRequests{0};
static void proxyDumpHandler(int) { gDumpRequests.fetch_add(1, std::memory_order_relaxed); }
static void proxyInstallDumpSignal() {
  static std::once_flag once;
  std::call_once(once, [] {
    const char* e = getEnv("NCCL_PROXY_DUMP_SIGNAL");
    const int sig = e && *e ? atoi(e) : -1;
    if (sig <= 0) return;
    struct sigaction sa;
    memset(&sa, 0, sizeof(sa));
    sa.sa_handler = proxyDumpHandler;
    sa.sa_flags = SA_RESTART;
    if (sigaction(sig, &sa, nullptr) == 0) INFO(SUB_PROXY | SUB_INIT, "proxy state dump on signal %d", sig);
  });
}
static void proxyDump(Proxy* p, const std::vector<ProxyOp*>& active) {
  WARN("proxy state of rank %d: %zu operation(s) in flight, %llu completed", p->comm->rank, active.size(), (unsigned long long)p->opsDone);
  for (const ProxyOp* op : active)
    WARN("  %s peer %d: %zu of %zu bytes posted, %zu completed, %d request(s) outstanding", op->isSend ? "send to" : "recv from", op->peer, op->posted,
         op->bytes, op->completed, op->tail - op->head);
}

B200_PARAM(IgnoreCpuAffinity, "IGNORE_CPU_AFFINITY", 0, "1: the proxy thread may also use the CPUs near its GPU that are outside the affinity mask of the process")

// "0-15,32-47" -> CPU numbers. Returns how many were written (at most `max`).
static int parseCpuList(const char* text, int* out, int max) {
  int n = 0;
  const char* p = text;
  while (p && *p && n < max) {
    char* end = nullptr;
    long lo = strtol(p, &end, 10);
    if (end == p) break;
    long hi = lo;
    p = end;
    if (*p == '-') { hi = strtol(p + 1, &end, 10); if (end == p + 1) break; p = end; }
    for (long c = lo; c <= hi && n < max; ++c) if (c >= 0) out[n++] = (int)c;
    while (*p == ',' || *p == ' ' || *p == '\n') ++p;
  }
  return n;
}

// The proxy thread of a GPU rank runs on the CPUs next to that GPU (its PCI device's local_cpulist), restricted to the CPUs the
// process may use unless NCCL_IGNORE_CPU_AFFINITY=1: the staging copies and the network adapter then sit on one socket.
// Reference parity: ncclTopoGetCpuAffinity (src/graph/topo.cc) applied to the proxy threads (src/proxy.cc).
static void proxySetAffinity(Proxy* p) {
  ncclComm* comm = p->comm;
  char busId[32] = "", path[PATH_MAX], text[1024] = "";
  // NCCL_PROXY_CPUSET names the CPUs of every proxy thread outright (same list form as the kernel's cpulist files)
  if (const char* forced = getEnv("NCCL_PROXY_CPUSET")) {
    int cpus[1024];
    const int n = parseCpuList(forced, cpus, 1024);
    cpu_set_t want;
    CPU_ZERO(&want);
    for (int i = 0; i < n; ++i) if (cpus[i] < CPU_SETSIZE) CPU_SET(cpus[i], &want);
    if (n > 0 && pthread_setaffinity_np(pthread_self(), sizeof(want), &want) == 0) INFO(SUB_INIT | SUB_PROXY, "proxy of rank %d runs on the CPUs of NCCL_PROXY_CPUSET=%s", comm->rank, forced);
    return;
  }
  if (comm->hostOnly) return;
  int64ToBusId(comm->peers[comm->rank].busId, busId);
  for (char* c = busId; *c; ++c) *c = (char)tolower(*c);
  snprintf(path, sizeof(path), "/sys/bus/pci/devices/%s/local_cpulist", busId);
  FILE* f = fopen(path, "r");
  if (!f) return;
  if (!fgets(text, sizeof(text), f)) text[0] = 0;
  fclose(f);
  int cpus[1024];
  const int n = parseCpuList(text, cpus, 1024);
  cpu_set_t allowed, want;
  CPU_ZERO(&want);
  if (sched_getaffinity(0, sizeof(allowed), &allowed) != 0) return;
  int kept = 0;
  for (int i = 0; i < n; ++i)
    if (cpus[i] < CPU_SETSIZE && (paramIgnoreCpuAffinity() || CPU_ISSET(cpus[i], &allowed))) { CPU_SET(cpus[i], &want); ++kept; }
  if (!kept) return;
  if (pthread_setaffinity_np(pthread_self(), sizeof(want), &want) == 0)
    INFO(SUB_INIT | SUB_PROXY, "proxy of rank %d runs on %d CPU(s) next to GPU %s", comm->rank, kept, busId);
}

static void proxyMain(Proxy* p) {
  setThreadName("NCCL Proxy %d", p->comm->rank);
  proxySetAffinity(p);
  proxyInstallDumpSignal();
  std::vector<ProxyOp*> active;
  uint64_t idle = 0;
  unsigned dumpsSeen = gDumpRequests.load(std::memory_order_relaxed);
  // One ncclProfileProxyCtrl event spans the life of the thread; its states say when the thread slept for lack of work and
  // when operations were handed to it.
  void* ctrl = nullptr;
  bool ctrlTried = false;
  for (;;) {
    {
      std::unique_lock<std::mutex> lk(p->lock);
      if (active.empty() && p->ops.empty() && !p->stop) {
        if (ctrl) profState(p->comm, ctrl, ncclProfilerProxyCtrlSleep, nullptr);
        p->wake.wait(lk, [&] { return p->stop || !p->ops.empty(); });
      }
      // the profiler is attached to the communicator after this thread has started: look once work has arrived
      if (!ctrlTried && p->comm->profiler && (!p->ops.empty() || !active.empty())) {
        ctrlTried = true;
        ncclProfilerEventDescr_t d;
        memset(&d, 0, sizeof(d));
        d.type = ncclProfileProxyCtrl;
        ctrl = profStart(p->comm, &d);
      }
      int appended = 0;
      while (!p->ops.empty()) {
        active.push_back(p->ops.front());
        p->ops.pop_front();
        profProxyOp(p, active.back(), true);
        ++appended;
      }
      if (ctrl && appended) {
        ncclProfilerEventStateArgs_t a;
        memset(&a, 0, sizeof(a));
        a.proxyCtrl.appendedProxyOps = appended;
        profState(p->comm, ctrl, ncclProfilerProxyCtrlActive, &a);
      }
      if (p->stop && active.empty()) {
        if (ctrl) profStop(p->comm, ctrl);
        return;
      }
    }
    const bool aborted = p->comm->abortFlag && __atomic_load_n(p->comm->abortFlag, __ATOMIC_RELAXED);
    const unsigned dumps = gDumpRequests.load(std::memory_order_relaxed);
    if (dumps != dumpsSeen) { dumpsSeen = dumps; proxyDump(p, active); }
    bool progressed = false;
    // Two operations of one direction towards one peer share a byte stream: only the oldest may run.
    for (size_t i = 0; i < active.size();) {
      ProxyOp* op = active[i];
      bool blocked = false;
      for (size_t j = 0; j < i; ++j) if (active[j]->peer == op->peer && active[j]->isSend == op->isSend) blocked = true;
      ncclResult_t r = ncclSuccess;
      size_t before = op->completed + op->posted;
      if (aborted) r = ncclInternalError;
      else if (!blocked) r = progressOp(p, op);
      if (op->completed + op->posted != before) progressed = true;
      if (r != ncclSuccess) {
        opRelease(p, op);
        profProxyOp(p, op, false);
        op->state.store(-(int)r, std::memory_order_release);
        active.erase(active.begin() + i);
        p->wake.notify_all();
        continue;
      }
      if (!blocked && opFinished(op)) {
        opRelease(p, op);
        profProxyOp(p, op, false);
        p->opsDone++;
        op->state.store(1, std::memory_order_release);
        active.erase(active.begin() + i);
        p->wake.notify_all();
        progressed = true;
        continue;
      }
      ++i;
    }
    if (progressed) idle = 0;
    else if (++idle > 200) usleep(20);   // nothing moved for a while: stop burning the core
  }
}

// Which device of the backend this rank uses: the one whose PCI path shares the longest prefix with the GPU's (the NIC behind
// the same switch), and among equals the ranks of a host take turns, so that several NICs carry the traffic of several ranks.
// Ranks without a GPU, and devices without a PCI path (virtual interfaces), only take turns.
static int chooseNetDev(ncclComm* comm, ncclNet_t* net, int ndev) {
  if (ndev <= 1) return 0;
  char gpuPath[PATH_MAX] = "";
  if (!comm->hostOnly) {
    char busId[32], link[PATH_MAX];
    int64ToBusId(comm->peers[comm->rank].busId, busId);
    for (char* c = busId; *c; ++c) *c = (char)tolower(*c);
    snprintf(link, sizeof(link), "/sys/bus/pci/devices/%s", busId);
    if (!realpath(link, gpuPath)) gpuPath[0] = 0;
  }
  std::vector<int> score(ndev, 0);
  int best = 0;
  for (int d = 0; d < ndev; ++d) {
    ncclNetProperties_t props;
    memset(&props, 0, sizeof(props));
    if (net->getProperties(d, &props) != ncclSuccess || !props.pciPath || !gpuPath[0]) continue;
    int common = 0;
    while (props.pciPath[common] && props.pciPath[common] == gpuPath[common]) ++common;
    while (common > 0 && props.pciPath[common - 1] != '/') --common;   // whole path components only
    score[d] = common;
    best = std::max(best, common);
  }
  std::vector<int> nearest;
  for (int d = 0; d < ndev; ++d) if (score[d] == best) nearest.push_back(d);
  const int dev = nearest[(size_t)comm->localRank % nearest.size()];
  INFO(SUB_NET | SUB_INIT, "proxy of rank %d (local rank %d): network device %d of %d", comm->rank, comm->localRank, dev, ndev);
  return dev;
}

ncclResult_t proxyCreate(ncclComm* comm) {
  Proxy* p = new Proxy;
  p->comm = comm;
  ncclResult_t res = netSelect(&p->net, &p->external);
  if (res != ncclSuccess) { delete p; return res; }
  const int n = comm->nRanks, me = comm->rank;
  ncclNetCommConfig_t cfg = {NCCL_NET_TRAFFIC_CLASS_UNDEF};
  if (comm->config.trafficClass != NCCL_CONFIG_UNDEF_INT) cfg.trafficClass = comm->config.trafficClass;
  NCCLCHECKGOTO(p->net->init(&p->netCtx, comm->commHash, &cfg, pluginLogger, profilerNetCallback), res, fail);
  {
    int ndev = 0;
    NCCLCHECKGOTO(p->net->devices(&ndev), res, fail);
    if (ndev <= 0) { WARN("network backend %s has no device", p->net->name); res = ncclSystemError; goto fail; }
    p->dev = chooseNetDev(comm, p->net, ndev);
    p->sliceBytes = (size_t)std::max<int64_t>(paramNetSliceKb(), 4) << 10;
    p->maxInflight = (int)std::min<int64_t>(std::max<int64_t>(paramNetInflight(), 1), NCCL_NET_MAX_REQUESTS);
    std::vector<char> handles((size_t)n * NCCL_NET_HANDLE_MAXSIZE, 0);
    NCCLCHECKGOTO(p->net->listen(p->netCtx, p->dev, handles.data() + (size_t)me * NCCL_NET_HANDLE_MAXSIZE, &p->listenComm), res, fail);
    NCCLCHECKGOTO(bootstrapAllGather(comm->bootstrap, handles.data(), NCCL_NET_HANDLE_MAXSIZE), res, fail);
    p->sendComm.assign(n, nullptr);
    p->recvComm.assign(n, nullptr);
    // A backend may finish a connection only after several calls (connect / accept return no object until the other side has
    // answered), so dialling and accepting take turns until the whole mesh stands. Backends whose connect lands in the peer's
    // listen queue and whose accept waits (TCP) get through the same loop: every rank dials everybody before its first accept.
    {
      std::vector<int> toDial;
      std::vector<void*> accepted;
      for (int r = 0; r < n; ++r) if (r != me) toDial.push_back(r);
      while (!toDial.empty() || (int)accepted.size() < n - 1) {
        for (size_t i = 0; i < toDial.size();) {
          void* sc = nullptr;
          NCCLCHECKGOTO(p->net->connect(p->netCtx, p->dev, handles.data() + (size_t)toDial[i] * NCCL_NET_HANDLE_MAXSIZE, &sc, nullptr), res, fail);
          if (sc) { p->sendComm[toDial[i]] = sc; toDial.erase(toDial.begin() + i); } else ++i;
        }
        if ((int)accepted.size() < n - 1) {
          void* rc = nullptr;
          NCCLCHECKGOTO(p->net->accept(p->listenComm, &rc, nullptr), res, fail);
          if (rc) accepted.push_back(rc);
        }
        if (flagSet(comm->abortFlag)) { for (void* rc : accepted) p->net->closeRecv(rc); res = ncclInternalError; goto fail; }
      }
      // Each accepted connection says who dialled with a first 4-byte message (small enough to complete at the sender without a
      // matching receive on every backend).
      for (int r = 0; r < n; ++r) {
        if (r == me) continue;
        int hello = me, done = 0;
        void* req = nullptr;
        while (!req) NCCLCHECKGOTO(p->net->isend(p->sendComm[r], &hello, sizeof(hello), 0, nullptr, nullptr, &req), res, fail);
        while (!done) NCCLCHECKGOTO(p->net->test(req, &done, nullptr), res, fail);
      }
      for (size_t k = 0; k < accepted.size(); ++k) {
        void* rc = accepted[k];
        int hello = -1, done = 0;
        void* req = nullptr;
        void* ptrs[1] = {&hello};
        size_t sizes[1] = {sizeof(hello)};
        int tags[1] = {0};
        void* mh[1] = {nullptr};
        void* ph[1] = {nullptr};
        ncclResult_t hr = ncclSuccess;
        while (!req && hr == ncclSuccess) hr = p->net->irecv(rc, 1, ptrs, sizes, tags, mh, ph, &req);
        while (!done && hr == ncclSuccess) hr = p->net->test(req, &done, nullptr);
        if (hr == ncclSuccess && (hello < 0 || hello >= n || hello == me || p->recvComm[hello])) { WARN("proxy: unexpected peer %d on the network mesh", hello); hr = ncclInternalError; }
        if (hr != ncclSuccess) { for (size_t j = k; j < accepted.size(); ++j) p->net->closeRecv(accepted[j]); res = hr; goto fail; }
        p->recvComm[hello] = rc;
      }
    }
  }
  p->thread = std::thread(proxyMain, p);
  comm->proxy = p;
  INFO(SUB_PROXY | SUB_NET, "proxy of rank %d: %s mesh to %d peers, %zu KiB slices, %d in flight", me, p->net->name, n - 1, p->sliceBytes >> 10, p->maxInflight);
  return ncclSuccess;
fail:
  comm->proxy = p;
  proxyDestroy(comm);
  return res;
}

// Ends the proxy thread (its profiler events end with it) while the communicator's profiler is still attached; the
// connections stay until proxyDestroy.
void proxyQuiesce(ncclComm* comm) {
  Proxy* p = comm->proxy;
  if (!p || !p->thread.joinable()) return;
  {
    std::lock_guard<std::mutex> g(p->lock);
    p->stop = true;
  }
  p->wake.notify_all();
  p->thread.join();
}

void proxyDestroy(ncclComm* comm) {
  Proxy* p = comm->proxy;
  if (!p) return;
  if (p->thread.joinable()) {
    {
      std::lock_guard<std::mutex> g(p->lock);
      p->stop = true;
    }
    p->wake.notify_all();
    p->thread.join();
  }
  if (p->net) {
    for (void* c : p->sendComm) if (c) p->net->closeSend(c);
    for (void* c : p->recvComm) if (c) p->net->closeRecv(c);
    if (p->listenComm) p->net->closeListen(p->listenComm);
    if (p->net->finalize) p->net->finalize(p->netCtx);
  }
  delete p;
  comm->proxy = nullptr;
}

ProxyOp* proxyPost(Proxy* p, bool isSend, int peer, void* data, size_t bytes) {
  ProxyOp* op = new ProxyOp;
  op->isSend = isSend;
  op->peer = peer;
  op->data = (char*)data;
  op->bytes = bytes;
  {
    std::lock_guard<std::mutex> g(p->lock);
    p->ops.push_back(op);
  }
  p->wake.notify_all();
  return op;
}

ncclResult_t proxyWait(Proxy* p, ProxyOp** ops, int n) {
  ncclResult_t res = ncclSuccess;
  for (int i = 0; i < n; ++i) {
    ProxyOp* op = ops[i];
    int spins = 0;
    while (op->state.load(std::memory_order_acquire) == 0) {
      if (++spins < 2000) { sched_yield(); continue; }
      std::unique_lock<std::mutex> lk(p->lock);
      p->wake.wait_for(lk, std::chrono::milliseconds(1), [&] { return op->state.load(std::memory_order_acquire) != 0; });
    }
    int st = op->state.load(std::memory_order_acquire);
    if (st < 0 && res == ncclSuccess) res = (ncclResult_t)(-st);
    delete op;
  }
  return res;
}

}  // namespace b200

// Test hook: the CPU-list parser of the proxy's affinity set-up.
extern "C" int b200ParseCpuList(const char* text, int* out, int max) { return b200::parseCpuList(text, out, max); }
