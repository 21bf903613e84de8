// One-sided operations on windows: ncclPutSignal, ncclSignal, ncclWaitSignal.
// A signal is a 64-bit counter in the target's resource window, one per (source rank, index);
// the source adds 1 with a release-ordered reduction after its data has landed, the target waits
// until the counter has advanced by the expected number of operations (bounded wait).
// Reference parity: src/rma/rma.cc:24-138, src/rma/rma_ce.cc:19-384 (intra-node put + signal).
#include "../comm/device_plane.h"

namespace b200 {

static uint64_t* signalWord(ncclComm* comm, int owner, int src, int idx) {
  DevicePlane* dp = comm->devPlane;
  char* base = (char*)dp->resWin->host.peerPtr[owner];
  return (uint64_t*)(base + kOffSignals) + (size_t)src * kSignalsPerPeer + idx;
}

ncclResult_t signalRun(ncclComm* comm, const Task& t) {
  DevicePlane* dp = comm->devPlane;
  if (comm->nRanks > 1 && (!comm->lsaAll || !dp->resWin)) { WARN("one-sided operations need ranks that can map each other's memory"); return ncclInvalidUsage; }
  if (t.sigIdx < 0 || t.ctx < 0) return ncclInvalidArgument;
  const int idx = (t.ctx * 16 + t.sigIdx) % kSignalsPerPeer;
  if (t.func == FUNC_PUTSIGNAL || t.func == FUNC_SIGNAL) {
    if (t.func == FUNC_PUTSIGNAL && t.count) {
      if (!t.win || t.win->magic != kWindowMagic) { WARN("ncclPutSignal : invalid window"); return ncclInvalidArgument; }
      size_t bytes = t.count * typeSize(t.type);
      if (t.winOffset + bytes > t.win->size) { WARN("ncclPutSignal : %zu bytes at offset %zu exceed the window (%zu bytes)", bytes, t.winOffset, t.win->size); return ncclInvalidArgument; }
      char* dst = (char*)t.win->peerPtr[t.root] + t.winOffset;
      ScaleArgs ca{t.send, dst, bytes, 0, nullptr};
      size_t perCta = 512 * 4 * 16;
      int ctas = (int)std::min<size_t>((bytes + perCta - 1) / perCta, (size_t)dp->smCount * 2);
      dp->launches++;
      NCCLCHECK(launchKernel(localCopyKernelFn(4), dim3(std::max(ctas, 1)), dim3(512), 0, &ca, t.stream, false));
    }
    if (comm->nRanks == 1 && !dp->resWin) return ncclSuccess;
    OneSignalArgs sa{signalWord(comm, t.root, comm->rank, idx)};
    dp->launches++;
    return launchKernel(signalKernelFn(), dim3(1), dim3(32), 0, &sa, t.stream, false);
  }
  // wait
  if (comm->nRanks == 1 && !dp->resWin) return ncclSuccess;
  WaitSignalArgs wa;
  memset(&wa, 0, sizeof(wa));
  wa.nDesc = 1;
  wa.counter[0] = signalWord(comm, comm->rank, t.root, idx);
  wa.seen[0] = dp->sigSeen + (size_t)t.root * kSignalsPerPeer + idx;
  wa.opCnt[0] = (uint32_t)t.opCnt;
  wa.rank = comm->rank;
  memset(&wa.sync, 0, sizeof(wa.sync));
  wa.sync.status[comm->rank] = comm->devStatusDev;
  wa.sync.abortFlag = comm->abortFlagDev;
  wa.sync.timeoutNs = dp->timeoutNs;
  dp->launches++;
  return launchKernel(waitSignalKernelFn(), dim3(1), dim3(32), 0, &wa, t.stream, false);
}

}  // namespace b200
