// Group semantics and the enqueue path.
// ncclGroupStart/End nest per thread; calls made inside a group are queued and issued when the
// outermost group ends: deferred communicator jobs first, then, per communicator in order of
// first appearance, the collectives in program order with every run of consecutive send/recv
// tasks fused into one launch. Outside a group a call is a group of one.
// Reference parity: src/group.cc (:97-124 API, :309-384 launch loop, :598-760 groupLaunch,
// :766-887 group end), src/enqueue.cc:3014-3172 (taskAppend / ncclEnqueueCheck).
#include <algorithm>

#include "../plugin/plugin.h"
#include "device_plane.h"

namespace b200 {

struct GroupState {
  int depth = 0;
  std::vector<Task> tasks;
  std::vector<std::function<ncclResult_t()>> jobs;
  ncclResult_t error = ncclSuccess;
};
static thread_local GroupState tGroup;

int groupDepth() { return tGroup.depth; }

ncclResult_t groupStart() {
  tGroup.depth++;
  return ncclSuccess;
}

ncclResult_t groupRunOrDefer(std::function<ncclResult_t()> fn) {
  if (tGroup.depth == 0) return fn();
  tGroup.jobs.push_back(std::move(fn));
  return ncclSuccess;
}

static ncclResult_t runTask(ncclComm* comm, const Task& t) {
  comm->opCount++;
  INFO(SUB_COLL, "%s: opCount %llx sendbuff %p recvbuff %p count %zu datatype %d op %d root %d comm %p [nranks=%d] stream %p",
       funcName(t.func), (unsigned long long)comm->opCount.load(), t.send, t.recv, t.count, (int)t.type, t.op, t.root, (void*)comm,
       comm->nRanks, (void*)t.stream);
  if (comm->hostOnly) {
    if (comm->nRanks == 1) {
      // single host rank: copy (and scale for pre-multiplied sums) in place
      size_t bytes = t.count * typeSize(t.type);
      if (t.func == FUNC_ALLGATHER || t.func == FUNC_GATHER || t.func == FUNC_ALLTOALL || t.func == FUNC_SCATTER ||
          t.func == FUNC_BROADCAST || t.op < ncclNumOps) {
        if (t.send != t.recv && t.send && t.recv) memcpy(t.recv, t.send, bytes);
        return ncclSuccess;
      }
    }
    void* prof = comm->profiler ? profilerTaskStart(comm, t) : nullptr;
    ncclResult_t r = hostPlaneRun(comm, t);
    if (prof) profilerTaskStop(comm, t, prof, "RING", "SIMPLE", 1);
    return r;
  }
  return devPlaneRun(comm, t);
}

static ncclResult_t runP2p(ncclComm* comm, const std::vector<Task>& p2p) {
  if (p2p.empty()) return ncclSuccess;
  comm->opCount++;
  if (comm->hostOnly) {
    if (comm->nRanks == 1) {
      std::vector<const Task*> s, r;
      for (auto& t : p2p) (t.func == FUNC_SEND ? s : r).push_back(&t);
      if (s.size() != r.size()) return ncclInvalidUsage;
      for (size_t i = 0; i < s.size(); ++i) memcpy(r[i]->recv, s[i]->send, s[i]->count * typeSize(s[i]->type));
      return ncclSuccess;
    }
    std::vector<void*> prof;
    if (comm->profiler) for (auto& t : p2p) prof.push_back(profilerTaskStart(comm, t));
    ncclResult_t r = hostPlaneRunP2pGroup(comm, p2p);
    for (size_t i = 0; i < prof.size(); ++i) profilerTaskStop(comm, p2p[i], prof[i], "P2P", "SIMPLE", 1);
    return r;
  }
  std::vector<void*> prof;
  if (comm->profiler) for (auto& t : p2p) prof.push_back(profilerTaskStart(comm, t));
  ncclResult_t r = devPlaneRunP2pGroup(comm, p2p);
  for (size_t i = 0; i < prof.size(); ++i) profilerTaskStop(comm, p2p[i], prof[i], "P2P", "SIMPLE", 1);
  return r;
}

B200_PARAM(LaunchRaceFatal, "LAUNCH_RACE_FATAL", 1, "Two threads issuing work on one communicator at the same time: 1 = fail the later call, 0 = warn only");

// One thread at a time may issue work on a communicator (reference: NCCL_LAUNCH_RACE_FATAL, src/misc/strongstream.cc).
// The guard marks the communicator for the duration of the issue and notices a second thread.
struct LaunchGuard {
  ncclComm* comm;
  bool owner = false, raced = false;
  explicit LaunchGuard(ncclComm* c) : comm(c) {
    static thread_local char token;
    const uintptr_t me = (uintptr_t)&token;
    uintptr_t expected = 0;
    if (comm->launchOwner.compare_exchange_strong(expected, me, std::memory_order_acquire)) owner = true;
    else if (expected != me) raced = true;
  }
  ~LaunchGuard() { if (owner) comm->launchOwner.store(0, std::memory_order_release); }
};

static ncclResult_t launchAll(std::vector<Task>& tasks, ncclSimInfo_t* sim) {
  // communicators in order of first appearance
  std::vector<ncclComm*> comms;
  for (auto& t : tasks) if (std::find(comms.begin(), comms.end(), t.comm) == comms.end()) comms.push_back(t.comm);
  float simUs = 0;
  for (ncclComm* comm : comms) {
    LaunchGuard guard(comm);
    if (guard.raced && !sim) {
      WARN("communicator %p (rank %d) is being used by two threads at the same time; calls on one communicator must be serialised", (void*)comm, comm->rank);
      if (paramLaunchRaceFatal()) return ncclInvalidUsage;
    }
    std::vector<Task> p2p;
    std::vector<Task> batch;   // consecutive small all-reduces of one type / operator / stream: one launch
    auto flushBatch = [&]() -> ncclResult_t {
      size_t done = 0;
      while (done < batch.size()) {
        if (batch.size() - done == 1) { NCCLCHECK(runTask(comm, batch[done])); ++done; break; }
        int taken = 0;
        comm->opCount++;
        NCCLCHECK(devPlaneRunLLBatch(comm, batch.data() + done, (int)(batch.size() - done), &taken));
        if (comm->profiler)
          for (int i = 0; i < taken; ++i) profilerTaskStop(comm, batch[done + i], profilerTaskStart(comm, batch[done + i]), "ONESHOT", "LL", 0);
        done += taken;
      }
      batch.clear();
      return ncclSuccess;
    };
    float commUs = 0;
    for (auto& t : tasks) {
      if (t.comm != comm) continue;
      if (sim) { commUs += comm->hostOnly ? 0.f : devPlaneEstimateUs(comm, t); continue; }
      if (t.func == FUNC_SEND || t.func == FUNC_RECV) { NCCLCHECK(flushBatch()); p2p.push_back(t); continue; }
      NCCLCHECK(runP2p(comm, p2p));
      p2p.clear();
      if (!comm->hostOnly && devPlaneBatchable(comm, t)) {
        if (!batch.empty() && (batch[0].type != t.type || batch[0].op != t.op || batch[0].stream != t.stream)) NCCLCHECK(flushBatch());
        batch.push_back(t);
        continue;
      }
      NCCLCHECK(flushBatch());
      NCCLCHECK(runTask(comm, t));
    }
    if (!sim) { NCCLCHECK(flushBatch()); NCCLCHECK(runP2p(comm, p2p)); }
    simUs = std::max(simUs, commUs);  // communicators of one group run concurrently
  }
  if (sim) sim->estimatedTime = simUs;
  return ncclSuccess;
}

ncclResult_t groupEnd(ncclSimInfo_t* sim) {
  if (tGroup.depth == 0) { WARN("ncclGroupEnd: not in a group call."); return ncclInvalidUsage; }
  if (--tGroup.depth > 0) return ncclSuccess;
  ncclResult_t res = tGroup.error;
  std::vector<Task> tasks;
  std::vector<std::function<ncclResult_t()>> jobs;
  tasks.swap(tGroup.tasks);
  jobs.swap(tGroup.jobs);
  tGroup.error = ncclSuccess;
  if (res != ncclSuccess) return res;
  bool inProgress = false;
  if (jobs.size() > 1) {
    // communicator jobs of one group (e.g. one ncclCommInitRank per device) rendezvous with each
    // other, so they must run concurrently
    std::vector<std::thread> th;
    std::vector<ncclResult_t> rs(jobs.size(), ncclSuccess);
    int dev = -1;
    cudaGetDevice(&dev);
    (void)cudaGetLastError();
    for (size_t i = 0; i < jobs.size(); ++i) th.emplace_back([&, i] { rs[i] = jobs[i](); });
    for (auto& t : th) t.join();
    for (auto r : rs) { if (r == ncclInProgress) inProgress = true; else if (r != ncclSuccess) return r; }
  } else if (jobs.size() == 1) {
    ncclResult_t r = jobs[0]();
    if (r == ncclInProgress) inProgress = true; else if (r != ncclSuccess) return r;
  }
  NCCLCHECK(launchAll(tasks, sim));
  return inProgress ? ncclInProgress : ncclSuccess;
}

ncclResult_t enqueueTask(const Task& t) {
  ncclResult_t ready = commEnsureReady(t.comm);
  if (ready != ncclSuccess) {
    if (tGroup.depth > 0 && ready != ncclInProgress) tGroup.error = ready;
    return ready;
  }
  ncclResult_t chk = argCheck(t, funcName(t.func));
  if (chk != ncclSuccess) {
    if (tGroup.depth > 0) tGroup.error = chk;
    return chk;
  }
  if (tGroup.depth > 0) {
    tGroup.tasks.push_back(t);
    return ncclSuccess;
  }
  std::vector<Task> one{t};
  if ((t.func == FUNC_SEND || t.func == FUNC_RECV) && t.root == t.comm->rank) {
    WARN("%s to self outside of a group would never complete", funcName(t.func));
    return ncclInvalidUsage;
  }
  return launchAll(one, nullptr);
}

}  // namespace b200

extern "C" {
ncclResult_t ncclGroupStart(void) { return b200::groupStart(); }
ncclResult_t ncclGroupEnd(void) { return b200::groupEnd(nullptr); }
ncclResult_t ncclGroupSimulateEnd(ncclSimInfo_t* simInfo) {
  if (simInfo && simInfo->magic != 0x74685283) { WARN("ncclSimInfo_t was not initialised with NCCL_SIM_INFO_INITIALIZER"); return ncclInvalidArgument; }
  ncclSimInfo_t local = NCCL_SIM_INFO_INITIALIZER;
  ncclResult_t r = b200::groupEnd(simInfo ? simInfo : &local);
  return r;
}
ncclResult_t pncclGroupStart(void) { return ncclGroupStart(); }
ncclResult_t pncclGroupEnd(void) { return ncclGroupEnd(); }
ncclResult_t pncclGroupSimulateEnd(ncclSimInfo_t* s) { return ncclGroupSimulateEnd(s); }
}
