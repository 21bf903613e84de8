// Copy-engine collectives: all-gather, all-to-all, broadcast, scatter and gather issued as
// cudaMemcpyAsync transfers into peer windows, bracketed by stream memory operations that play
// the role of the cross-rank barrier. They occupy no SM, which is what makes them attractive next
// to compute (FSDP parameter all-gathers). One cudaMemcpyAsync per peer: no batched-copy API.
// Synchronisation values come from a host-side counter, so this path is refused while the stream
// is being captured (a replay would present stale values); the SM kernels take over there.
// Reference parity: src/ce_coll.cc:93-131 (availability), :133-285 (flag synchronisation),
// :497-717 (all-gather / all-to-all / scatter / gather).
#include <vector>

#include "../comm/device_plane.h"
#include "../core/cudawrap.h"
#include "../plugin/profiler.h"

namespace b200 {

static constexpr int kCeSlot = kBarrierSlots - 1;   // barrier slot reserved for the copy engines

static ncclResult_t ceBarrier(ncclComm* comm, cudaStream_t stream, uint32_t value) {
  const CuApi* cu = cuApi();
  DevicePlane* dp = comm->devPlane;
  const int n = comm->nRanks, me = comm->rank;
  for (int j = 1; j < n; ++j) {
    int p = (me + j) % n;
    uint32_t* w = (uint32_t*)dp->resWin->host.peerPtr[p] + (size_t)kCeSlot * kMaxRanks + me;
    CUCHECK(cu->cuStreamWriteValue32((CUstream)stream, (CUdeviceptr)w, value, CU_STREAM_WRITE_VALUE_DEFAULT));
  }
  for (int j = 1; j < n; ++j) {
    int p = (me + j) % n;
    uint32_t* w = (uint32_t*)dp->resBase + (size_t)kCeSlot * kMaxRanks + p;
    CUCHECK(cu->cuStreamWaitValue32((CUstream)stream, (CUdeviceptr)w, value, CU_STREAM_WAIT_VALUE_GEQ));
  }
  return ncclSuccess;
}

// Stream waits of this path have no time limit of their own and do not look at the abort flag. ncclCommAbort and
// ncclCommRevoke therefore call this before they drain the device: it writes the newest value that any queued wait
// of this rank can be waiting for into every word of the copy engines' barrier row (from a stream of its own, since
// the caller's streams are blocked behind those waits), which releases them; the data behind them is abandoned.
void ceCollRelease(ncclComm* comm) {
  DevicePlane* dp = comm->devPlane;
  const CuApi* cu = cuApi();
  if (!dp || !cu || !dp->resBase || dp->ceEpoch == 0) return;
  cudaStream_t s = nullptr;
  if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) { (void)cudaGetLastError(); return; }
  for (int p = 0; p < comm->nRanks; ++p) {
    uint32_t* w = (uint32_t*)dp->resBase + (size_t)kCeSlot * kMaxRanks + p;
    cu->cuStreamWriteValue32((CUstream)s, (CUdeviceptr)w, (uint32_t)dp->ceEpoch, CU_STREAM_WRITE_VALUE_DEFAULT);
  }
  cudaStreamSynchronize(s);
  cudaStreamDestroy(s);
  (void)cudaGetLastError();
}

ncclResult_t ceCollRun(ncclComm* comm, const Task& t, bool* handled) {
  *handled = false;
  DevicePlane* dp = comm->devPlane;
  const CuApi* cu = cuApi();
  if (!cu || !comm->lsaAll || !dp->resWin) return ncclSuccess;
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(t.stream, &cs) != cudaSuccess) { (void)cudaGetLastError(); return ncclSuccess; }
  if (cs != cudaStreamCaptureStatusNone) return ncclSuccess;
  const int n = comm->nRanks, me = comm->rank;
  const size_t B = t.count * typeSize(t.type);
  // pushes need the destination inside a symmetric window (same offset on every rank)
  size_t recvBytes = (t.func == FUNC_ALLGATHER || t.func == FUNC_ALLTOALL) ? B * n : B;
  if (t.func == FUNC_GATHER) return ncclSuccess;   // the receive buffer is only defined on the root
  SymWindow* w = symFindWindow(comm, t.recv, recvBytes);
  if (!w || !w->symmetric) return ncclSuccess;
  const size_t off = (uintptr_t)t.recv - (uintptr_t)w->host.userPtr;
  auto peerRecv = [&](int p) { return (char*)w->host.peerPtr[p] + off; };
  // epoch values are even before / odd after, strictly increasing
  const uint32_t before = (uint32_t)(++dp->ceEpoch), after = (uint32_t)(++dp->ceEpoch);
  // the copies of this rank: one per block that it owns the source of
  struct Copy { const char* s; char* d; };
  std::vector<Copy> copies;
  const char* src = (const char*)t.send;
  for (int j = 0; j < n; ++j) {
    int p = (me + j) % n;
    const char* s = nullptr;
    char* d = nullptr;
    switch (t.func) {
      case FUNC_ALLGATHER: s = src; d = peerRecv(p) + (size_t)me * B; break;
      case FUNC_ALLTOALL: s = src + (size_t)p * B; d = peerRecv(p) + (size_t)me * B; break;
      case FUNC_BROADCAST: if (me == t.root) { s = src; d = peerRecv(p); } break;
      case FUNC_SCATTER: if (me == t.root) { s = src + (size_t)p * B; d = peerRecv(p); } break;
      default: break;
    }
    if (s && d && s != d) copies.push_back(Copy{s, d});
  }
  // profiler events cover the issue of the operations on the host (the stream runs them later)
  void* evColl = profilerCeStart(comm, t, 0, nullptr, (int)copies.size(), 0);
  void* evSync = profilerCeStart(comm, t, 1, evColl, 0, 0);
  ncclResult_t res = ceBarrier(comm, t.stream, before);   // every destination may be overwritten
  profilerCeStop(comm, evSync, 1);
  if (res != ncclSuccess) { profilerCeStop(comm, evColl, 0); return res; }
  void* evBatch = profilerCeStart(comm, t, 2, evColl, (int)copies.size(), copies.size() * B);
  for (const Copy& c : copies) {
    if (cudaMemcpyAsync(c.d, c.s, B, cudaMemcpyDeviceToDevice, t.stream) != cudaSuccess) {
      WARN("copy-engine collective: cudaMemcpyAsync failed: %s", cudaGetErrorString(cudaGetLastError()));
      profilerCeStop(comm, evBatch, 2);
      profilerCeStop(comm, evColl, 0);
      return ncclUnhandledCudaError;
    }
  }
  profilerCeStop(comm, evBatch, 2);
  evSync = profilerCeStart(comm, t, 1, evColl, 1, 0);
  res = ceBarrier(comm, t.stream, after);    // everything addressed to me has landed
  profilerCeStop(comm, evSync, 1);
  profilerCeStop(comm, evColl, 0);
  NCCLCHECK(res);
  *handled = true;
  return ncclSuccess;
}

}  // namespace b200
