// Memory manager of a communicator: every device allocation made on its behalf is tracked with a class
//   persist   small state that must survive (epoch words, window handles): never released;
//   scratch   working memory whose contents need not survive (the resource window, expert-parallel landing zones,
//             staging of the fused GEMMs): released on suspend, mapped again (zeroed where asked) on resume;
//   offload   memory whose contents must survive (activation windows handed to the caller): copied to pinned host
//             memory before it is released and copied back on resume.
// ncclCommSuspend drains the device, unregisters the windows over tracked memory (peers unmap it), and gives the
// physical memory back while the address ranges stay reserved, so every pointer stays valid; ncclCommResume maps
// new memory at the same addresses, restores / zeroes it, registers the windows again and runs the owners'
// callbacks (restart of epochs). Both are collective. ncclCommMemStats reports the totals per class.
// Reference parity: src/mem_manager.cc:129-330 (tracking), :395-525 (suspend), :527-924 (resume), :926-1010 (API).
#include <functional>

#include "../comm/device_plane.h"

namespace b200 {

struct MemRecord {
  void* ptr;
  size_t bytes;
  int cls;
  std::string what;
  SymWindow** win;                 // the owner's window over this memory (re-registered on resume), or null
  int winFlags;
  size_t zeroBytes;                // prefix to clear after new memory was mapped (scratch)
  std::function<void()> afterResume;
  void* hostCopy = nullptr;
  bool released = false;
};

struct MemManager {
  bool suspended = false;
  std::vector<MemRecord> records;   // in registration order: the same on every rank
  std::mutex lock;
};

static MemManager* mgr(ncclComm* comm) {
  if (!comm->memMgr) comm->memMgr = new MemManager;
  return comm->memMgr;
}

void memTrack(ncclComm* comm, void* ptr, size_t bytes, int cls, const char* what, SymWindow** win, int winFlags, size_t zeroBytes,
              std::function<void()> afterResume) {
  MemManager* m = mgr(comm);
  std::lock_guard<std::mutex> g(m->lock);
  m->records.push_back(MemRecord{ptr, bytes, cls, what ? what : "", win, winFlags, zeroBytes, std::move(afterResume)});
}

void memUntrack(ncclComm* comm, void* ptr) {
  if (!comm->memMgr) return;
  MemManager* m = comm->memMgr;
  std::lock_guard<std::mutex> g(m->lock);
  for (auto it = m->records.begin(); it != m->records.end(); ++it)
    if (it->ptr == ptr) {
      if (it->hostCopy) cudaFreeHost(it->hostCopy);
      m->records.erase(it);
      return;
    }
}

ncclResult_t memSuspend(ncclComm* comm) {
  MemManager* m = mgr(comm);
  if (m->suspended) { WARN("ncclCommSuspend : communicator is already suspended"); return ncclInvalidUsage; }
  int cur = -1;
  CUDACHECK(cudaGetDevice(&cur));
  if (cur != comm->cudaDev) CUDACHECK(cudaSetDevice(comm->cudaDev));
  CUDACHECK(cudaDeviceSynchronize());
  // nobody may still be writing into my windows when their memory goes away
  if (comm->nRanks > 1) NCCLCHECK(bootstrapBarrier(comm->bootstrap));
  size_t released = 0, offloaded = 0;
  for (auto& r : m->records) {
    if (r.cls == MEM_PERSIST || r.released) continue;
    MemAlloc a;
    if (!memLookup(r.ptr, &a) || !a.vmm) continue;   // memory from cudaMalloc cannot give its pages back and keep its address
    if (r.win && *r.win) { NCCLCHECK(symWindowDeregister(comm, *r.win)); *r.win = nullptr; }
    if (r.cls == MEM_OFFLOAD) {
      if (!r.hostCopy) CUDACHECK(cudaHostAlloc(&r.hostCopy, r.bytes, cudaHostAllocDefault));
      CUDACHECK(cudaMemcpy(r.hostCopy, r.ptr, r.bytes, cudaMemcpyDeviceToHost));
      offloaded += r.bytes;
    }
    NCCLCHECK(memDetachPhysical(r.ptr));
    r.released = true;
    released += a.size;
  }
  m->suspended = true;
  if (cur != comm->cudaDev) cudaSetDevice(cur);
  INFO(SUB_ALLOC, "rank %d suspended: released %zu bytes (%zu of them saved to host memory)", comm->rank, released, offloaded);
  return ncclSuccess;
}

ncclResult_t memResume(ncclComm* comm) {
  MemManager* m = mgr(comm);
  if (!m->suspended) { WARN("ncclCommResume : communicator is not suspended"); return ncclInvalidUsage; }
  int cur = -1;
  CUDACHECK(cudaGetDevice(&cur));
  if (cur != comm->cudaDev) CUDACHECK(cudaSetDevice(comm->cudaDev));
  size_t mapped = 0;
  for (auto& r : m->records) {
    if (!r.released) continue;
    NCCLCHECK(memAttachPhysical(r.ptr));
    if (r.cls == MEM_OFFLOAD && r.hostCopy) {
      CUDACHECK(cudaMemcpy(r.ptr, r.hostCopy, r.bytes, cudaMemcpyHostToDevice));
      cudaFreeHost(r.hostCopy);
      r.hostCopy = nullptr;
    } else if (r.zeroBytes) {
      CUDACHECK(cudaMemset(r.ptr, 0, std::min(r.zeroBytes, r.bytes)));
    }
    mapped += r.bytes;
  }
  CUDACHECK(cudaDeviceSynchronize());
  // windows in the order they were first registered (collective calls must line up across ranks)
  for (auto& r : m->records) {
    if (!r.released) continue;
    if (r.win && comm->nRanks > 1 && comm->lsaAll) NCCLCHECK(symWindowRegister(comm, r.ptr, r.bytes, r.win, r.winFlags));
    r.released = false;
  }
  for (auto& r : m->records) if (r.afterResume) r.afterResume();
  CUDACHECK(cudaDeviceSynchronize());
  if (comm->nRanks > 1) NCCLCHECK(bootstrapBarrier(comm->bootstrap));
  m->suspended = false;
  if (cur != comm->cudaDev) cudaSetDevice(cur);
  INFO(SUB_ALLOC, "rank %d resumed: %zu bytes mapped again", comm->rank, mapped);
  return ncclSuccess;
}

ncclResult_t memStats(ncclComm* comm, int stat, uint64_t* value) {
  MemManager* m = mgr(comm);
  std::lock_guard<std::mutex> g(m->lock);
  uint64_t persist = 0, releasable = 0, released = 0;
  for (auto& r : m->records) {
    if (r.cls == MEM_PERSIST) persist += r.bytes;
    else if (r.released) released += r.bytes;
    else releasable += r.bytes;
  }
  switch (stat) {
    case ncclStatGpuMemSuspend: *value = m->suspended ? 0 : releasable; break;      // what a suspend would give back now
    case ncclStatGpuMemSuspended: *value = m->suspended ? 1 : 0; break;
    case ncclStatGpuMemPersist: *value = persist; break;
    case ncclStatGpuMemTotal: *value = persist + releasable; break;                 // resident right now
    default: return ncclInvalidArgument;
  }
  (void)released;
  return ncclSuccess;
}

// Per class totals and the number of tracked allocations, for tools and tests: out[0..2] = bytes of persist / scratch /
// offload memory, out[3] = allocations tracked, out[4] = bytes currently released.
extern "C" __attribute__((visibility("default"))) int b200CommMemClasses(ncclComm_t comm, unsigned long long* out) {
  if (!commValid(comm) || !out) return 1;
  MemManager* m = mgr(comm);
  std::lock_guard<std::mutex> g(m->lock);
  for (int i = 0; i < 5; ++i) out[i] = 0;
  for (auto& r : m->records) {
    out[r.cls] += r.bytes;
    out[3]++;
    if (r.released) out[4] += r.bytes;
  }
  return 0;
}

void memMgrDestroy(ncclComm* comm) {
  if (comm->memMgr) for (auto& r : comm->memMgr->records) if (r.hostCopy) cudaFreeHost(r.hostCopy);
  delete comm->memMgr;
  comm->memMgr = nullptr;
}

}  // namespace b200
