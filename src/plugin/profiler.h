// Profiling hooks of the host runtime: a built-in ring of API events (always on, cheap) and
// the external profiler plugin (events forwarded when a plugin is loaded).
// Reference parity: src/plugin/profiler.cc:245-938 (event start/stop from API, group and launch
// sites), src/include/plugin/nccl_profiler.h (event kinds).
#pragma once
#include "../comm/comm.h"

namespace b200 {

struct ApiEvent {
  uint64_t tStartNs, tEndNs;
  uint64_t commHash;
  int rank, func, root;
  size_t count;
  int type, op;
  void* stream;
};

void profilerCommInit(ncclComm* comm);
void profilerCommFini(ncclComm* comm);
// Returns a handle for profilerApiStop (null when nothing listens).
void* profilerApiStart(ncclComm* comm, const Task& t);
void profilerApiStop(void* h);
// Copies the most recent events (oldest first) into `out`; returns how many.
int profilerRecentEvents(ApiEvent* out, int max);

// Events of a copy-engine collective (plugin events CeColl / CeSync / CeBatch): the whole call, each of its two
// stream-memory-operation barriers, and the batch of copies. `what` 0 = the call, 1 = a barrier, 2 = the copies;
// the returned handle (null when no plugin listens) is closed with profilerCeStop.
void* profilerCeStart(ncclComm* comm, const Task& t, int what, void* parent, int numOps, size_t totalBytes);
void profilerCeStop(ncclComm* comm, void* h, int what);

struct ProfilerApiScope {
  void* h;
  ProfilerApiScope(ncclComm* c, const Task& t) : h(profilerApiStart(c, t)) {}
  ~ProfilerApiScope() { if (h) profilerApiStop(h); }
};

}  // namespace b200
