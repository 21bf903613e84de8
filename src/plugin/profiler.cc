// Built-in API event ring (the external plugin glue lives in profiler_plugin.cc).
#include "profiler.h"

#include <mutex>

namespace b200 {

static constexpr int kRing = 4096;
static ApiEvent gRing[kRing];
static uint64_t gHead = 0;
static std::mutex gLock;

void* profilerPluginStart(ncclComm* comm, const Task& t);   // profiler_plugin.cc
void profilerPluginStop(void* h);

struct ApiHandle {
  ApiEvent ev;
  void* plugin;
};

void* profilerApiStart(ncclComm* comm, const Task& t) {
  ApiHandle* h = new ApiHandle;
  h->ev = ApiEvent{nowNs(), 0, comm->commHash, comm->rank, t.func, t.root, t.count, (int)t.type, t.op, (void*)t.stream};
  h->plugin = profilerPluginStart(comm, t);
  nvtxRangeBegin(funcName(t.func), t.count * typeSize(t.type), comm->commHash, comm->rank);
  return h;
}

void profilerApiStop(void* hv) {
  ApiHandle* h = (ApiHandle*)hv;
  h->ev.tEndNs = nowNs();
  nvtxRangeEnd();
  if (h->plugin) profilerPluginStop(h->plugin);
  {
    std::lock_guard<std::mutex> g(gLock);
    gRing[gHead % kRing] = h->ev;
    ++gHead;
  }
  delete h;
}

int profilerRecentEvents(ApiEvent* out, int max) {
  std::lock_guard<std::mutex> g(gLock);
  uint64_t have = gHead < (uint64_t)kRing ? gHead : (uint64_t)kRing;
  int n = (int)(have < (uint64_t)max ? have : (uint64_t)max);
  for (int i = 0; i < n; ++i) out[i] = gRing[(gHead - n + i) % kRing];
  return n;
}

}  // namespace b200
