// Memory accounting and suspend / resume of a communicator's own device memory.
// Suspend releases the resource window (flags, flagged-line buffers, mailboxes, staging area) after
// draining the device; resume allocates it again, maps it on every peer and restarts all epochs.
// Both are collective. User windows are not touched: their memory belongs to the caller.
// Reference parity: src/mem_manager.cc:395-525 (suspend), :527-924 (resume), :926-1010 (API).
#include "../comm/device_plane.h"

namespace b200 {

struct MemManager {
  bool suspended = false;
  size_t suspendedBytes = 0;
};

static MemManager* mgr(ncclComm* comm) {
  if (!comm->memMgr) comm->memMgr = new MemManager;
  return comm->memMgr;
}

ncclResult_t memSuspend(ncclComm* comm) {
  MemManager* m = mgr(comm);
  DevicePlane* dp = comm->devPlane;
  if (m->suspended) { WARN("ncclCommSuspend : communicator is already suspended"); return ncclInvalidUsage; }
  if (!dp || !dp->resBase) { m->suspended = true; return ncclSuccess; }
  int cur = -1;
  CUDACHECK(cudaGetDevice(&cur));
  if (cur != comm->cudaDev) CUDACHECK(cudaSetDevice(comm->cudaDev));
  CUDACHECK(cudaDeviceSynchronize());
  // nobody may still be writing into my window when its memory goes away
  NCCLCHECK(bootstrapBarrier(comm->bootstrap));
  m->suspendedBytes = dp->resSize;
  NCCLCHECK(symWindowDeregister(comm, dp->resWin));
  dp->resWin = nullptr;
  NCCLCHECK(memFree(dp->resBase));
  dp->resBase = nullptr;
  m->suspended = true;
  if (cur != comm->cudaDev) cudaSetDevice(cur);
  INFO(SUB_ALLOC, "rank %d suspended: released %zu bytes", comm->rank, m->suspendedBytes);
  return ncclSuccess;
}

ncclResult_t memResume(ncclComm* comm) {
  MemManager* m = mgr(comm);
  DevicePlane* dp = comm->devPlane;
  if (!m->suspended) { WARN("ncclCommResume : communicator is not suspended"); return ncclInvalidUsage; }
  if (!dp || dp->resSize == 0 || !comm->lsaAll) { m->suspended = false; return ncclSuccess; }
  int cur = -1;
  CUDACHECK(cudaGetDevice(&cur));
  if (cur != comm->cudaDev) CUDACHECK(cudaSetDevice(comm->cudaDev));
  NCCLCHECK(memAlloc(&dp->resBase, dp->resSize, comm->cudaDev));
  CUDACHECK(cudaMemset(dp->resBase, 0, dp->offMailbox));
  // epochs, sequence numbers and the consumed-signal table restart together with the flags and
  // counters of the new window they are compared against (same extent as devPlaneCreate allocates)
  const size_t privWords = kPrivWords + 2 * kMaxRanks * kSignalsPerPeer;
  CUDACHECK(cudaMemset(dp->priv, 0, privWords * sizeof(uint32_t)));
  CUDACHECK(cudaDeviceSynchronize());
  NCCLCHECK(symWindowRegister(comm, dp->resBase, dp->resSize, &dp->resWin, NCCL_WIN_COLL_SYMMETRIC));
  NCCLCHECK(bootstrapBarrier(comm->bootstrap));
  m->suspended = false;
  if (cur != comm->cudaDev) cudaSetDevice(cur);
  INFO(SUB_ALLOC, "rank %d resumed: %zu bytes mapped again", comm->rank, dp->resSize);
  return ncclSuccess;
}

ncclResult_t memStats(ncclComm* comm, int stat, uint64_t* value) {
  MemManager* m = mgr(comm);
  DevicePlane* dp = comm->devPlane;
  uint64_t scratch = dp && dp->resBase ? dp->resSize : 0;
  uint64_t persist = dp && dp->priv ? 4096 : 0;
  switch (stat) {
    case ncclStatGpuMemSuspend: *value = m->suspended ? 0 : scratch; break;
    case ncclStatGpuMemSuspended: *value = m->suspended ? 1 : 0; break;
    case ncclStatGpuMemPersist: *value = persist; break;
    case ncclStatGpuMemTotal: *value = scratch + persist; break;
    default: return ncclInvalidArgument;
  }
  return ncclSuccess;
}

void memMgrDestroy(ncclComm* comm) {
  delete comm->memMgr;
  comm->memMgr = nullptr;
}

}  // namespace b200
