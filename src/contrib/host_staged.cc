// Chunked, overlapped host -> device -> all-reduce -> host pipeline (see include/nccl_host_staged.h).
// Three streams: copies in on one, the collectives on the caller's, copies out on a third; one event per chunk slot and
// stage orders them, across calls as well (a slot's staging memory is reused by the next call).
#include "nccl_host_staged.h"

#include <map>
#include <mutex>
#include <vector>

#include "../comm/comm.h"

namespace b200 {

struct HostStaged {
  cudaStream_t in = nullptr, out = nullptr;
  cudaEvent_t fork = nullptr;
  std::vector<cudaEvent_t> copied, reduced, returned;   // per chunk slot
};
static std::mutex gLock;
static std::map<ncclComm*, HostStaged*> gState;

static ncclResult_t stateOf(ncclComm* comm, size_t slots, HostStaged** out) {
  std::lock_guard<std::mutex> g(gLock);
  HostStaged*& s = gState[comm];
  if (!s) {
    s = new HostStaged;
    CUDACHECK(cudaStreamCreateWithFlags(&s->in, cudaStreamNonBlocking));
    CUDACHECK(cudaStreamCreateWithFlags(&s->out, cudaStreamNonBlocking));
    CUDACHECK(cudaEventCreateWithFlags(&s->fork, cudaEventDisableTiming));
  }
  while (s->copied.size() < slots) {
    cudaEvent_t e[3];
    for (auto& x : e) CUDACHECK(cudaEventCreateWithFlags(&x, cudaEventDisableTiming));
    s->copied.push_back(e[0]);
    s->reduced.push_back(e[1]);
    s->returned.push_back(e[2]);
  }
  *out = s;
  return ncclSuccess;
}

// Called when a communicator goes away.
void hostStagedRelease(ncclComm* comm) {
  std::lock_guard<std::mutex> g(gLock);
  auto it = gState.find(comm);
  if (it == gState.end()) return;
  HostStaged* s = it->second;
  for (auto* v : {&s->copied, &s->reduced, &s->returned}) for (cudaEvent_t e : *v) cudaEventDestroy(e);
  if (s->fork) cudaEventDestroy(s->fork);
  if (s->in) cudaStreamDestroy(s->in);
  if (s->out) cudaStreamDestroy(s->out);
  (void)cudaGetLastError();
  delete s;
  gState.erase(it);
}

}  // namespace b200

using namespace b200;

extern "C" ncclResult_t ncclAllReduceFromHost(const void* hostSend, void* hostRecv, void* devSend, void* devRecv, size_t count, ncclDataType_t type,
                                              ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream, size_t chunkBytes) {
  if (!commValid(comm) || !hostSend || !hostRecv || !devSend || !devRecv) return ncclInvalidArgument;
  if ((int)type < 0 || (int)type >= ncclNumTypes) return ncclInvalidArgument;
  if (count == 0) return ncclSuccess;
  NCCLCHECK(commEnsureReady(comm));
  if (comm->hostOnly) { WARN("ncclAllReduceFromHost: needs a GPU communicator (a host-memory communicator reduces host buffers with ncclAllReduce itself)"); return ncclInvalidUsage; }
  if (groupDepth() > 0) {
    WARN("ncclAllReduceFromHost: not available between ncclGroupStart and ncclGroupEnd (its collectives must launch where they are issued)");
    return ncclInvalidUsage;
  }
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cs) == cudaSuccess && cs != cudaStreamCaptureStatusNone) {
    WARN("ncclAllReduceFromHost: not available while the stream is being captured (it uses streams of its own)");
    return ncclInvalidUsage;
  }
  const size_t es = typeSize(type);
  size_t chunk = chunkBytes ? chunkBytes : ((size_t)32 << 20);
  chunk = std::max<size_t>(chunk / 4096 * 4096, 4096);
  const size_t chunkElems = chunk / es;
  const size_t nChunks = (count + chunkElems - 1) / chunkElems;
  HostStaged* s = nullptr;
  NCCLCHECK(stateOf(comm, nChunks, &s));
  CUDACHECK(cudaEventRecord(s->fork, stream));
  CUDACHECK(cudaStreamWaitEvent(s->in, s->fork, 0));
  for (size_t i = 0; i < nChunks; ++i) {
    const size_t off = i * chunkElems, len = std::min(chunkElems, count - off);
    const char* hs = (const char*)hostSend + off * es;
    char* hr = (char*)hostRecv + off * es;
    char* ds = (char*)devSend + off * es;
    char* dr = (char*)devRecv + off * es;
    // copy in: the previous user of this slot's staging memory (the collective of the last call that read it, the copy out
    // that read the result when both staging buffers are one) must be done
    CUDACHECK(cudaStreamWaitEvent(s->in, s->reduced[i], 0));
    CUDACHECK(cudaStreamWaitEvent(s->in, s->returned[i], 0));
    CUDACHECK(cudaMemcpyAsync(ds, hs, len * es, cudaMemcpyHostToDevice, s->in));
    CUDACHECK(cudaEventRecord(s->copied[i], s->in));
    // reduce: after its input has arrived and the last result of this slot has left
    CUDACHECK(cudaStreamWaitEvent(stream, s->copied[i], 0));
    CUDACHECK(cudaStreamWaitEvent(stream, s->returned[i], 0));
    NCCLCHECK(ncclAllReduce(ds, dr, len, type, op, comm, stream));
    CUDACHECK(cudaEventRecord(s->reduced[i], stream));
    // copy out
    CUDACHECK(cudaStreamWaitEvent(s->out, s->reduced[i], 0));
    CUDACHECK(cudaMemcpyAsync(hr, dr, len * es, cudaMemcpyDeviceToHost, s->out));
    CUDACHECK(cudaEventRecord(s->returned[i], s->out));
  }
  CUDACHECK(cudaStreamWaitEvent(stream, s->returned[nChunks - 1], 0));
  return ncclSuccess;
}
