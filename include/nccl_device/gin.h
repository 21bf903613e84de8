/*
 * GPU-initiated one-sided surface of the device API: put, signal, wait. The reference routes these
 * through a network backend (GDAKI / proxy); this build serves one NVLink domain, so for peers inside
 * the load/store team the operations are peer stores, `red.add` on signal words of the target's
 * resource window and bounded polls. Peers outside the team report ncclInvalidUsage (no RDMA
 * backend is linked).
 *   put(peer, dst, src, bytes [, signal])   copy, then optionally bump a signal on the peer
 *   signal(peer, id)                        bump signal `id` on the peer (release ordering)
 *   waitSignal(id, value) / readSignal(id)  bounded wait on / read of a local signal
 *   flush()                                 make earlier puts visible before what follows
 * Reference parity: src/include/nccl_device/gin.h:21-333 (ncclGin: put, signal, flush, wait*,
 * read*, reset*), impl/gin__funcs.h (abort-aware waits :774-1000).
 */
#ifndef NCCL_DEVICE_GIN_H_
#define NCCL_DEVICE_GIN_H_
#include "core.h"
#include "utility.h"
#if defined(__CUDACC__)
struct ncclGin {
  const ncclDevComm_t& comm;
  __device__ explicit ncclGin(const ncclDevComm_t& c, int /*context*/ = 0) : comm(c) {}

  __device__ unsigned long long* signalWord(int owner, int id) const {
    return (unsigned long long*)((char*)comm.resource.peerPtr[owner] + comm.ginSignalOffset) + id;
  }
  __device__ unsigned long long* counterWord(int id) const {
    return (unsigned long long*)((char*)comm.resource.peerPtr[comm.lsaRank] + comm.ginCounterOffset) + id;
  }

  /* Everything this thread (and, after a group sync, its group) wrote earlier is visible to the peer
   * once it observes the signal. */
  __device__ ncclResult_t signal(ncclTeam_t team, int peer, int id, unsigned long long add = 1) {
    const int world = ncclTeamRankToWorld(comm, team, peer);
    if (world < 0 || world >= comm.lsaSize || id < 0 || id >= comm.ginSignalCount) return ncclInvalidUsage;
    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(signalWord(world, id)), "l"(add) : "memory");
    return ncclSuccess;
  }

  template <typename Coop>
  __device__ ncclResult_t put(Coop coop, ncclTeam_t team, int peer, ncclWindow_t dstWin, size_t dstOffset, ncclWindow_t srcWin, size_t srcOffset,
                              size_t bytes, int signalId = -1, int counterId = -1) {
    const int world = ncclTeamRankToWorld(comm, team, peer);
    if (world < 0 || world >= comm.lsaSize) return ncclInvalidUsage;
    const char* s = (const char*)ncclGetLocalPointer(srcWin, srcOffset);
    char* d = (char*)ncclGetLsaPointer(dstWin, dstOffset, world);
    if ((((uintptr_t)s | (uintptr_t)d) & 15) == 0) {
      for (size_t i = (size_t)coop.thread_rank() * 16; i + 16 <= bytes; i += (size_t)coop.size() * 16) *(uint4*)(d + i) = *(const uint4*)(s + i);
      for (size_t b = bytes / 16 * 16 + coop.thread_rank(); b < bytes; b += coop.size()) d[b] = s[b];
    } else {
      for (size_t b = coop.thread_rank(); b < bytes; b += coop.size()) d[b] = s[b];
    }
    coop.sync();
    if (coop.thread_rank() == 0) {
      if (signalId >= 0) signal(team, peer, signalId);
      if (counterId >= 0 && counterId < comm.ginCounterCount) atomicAdd(counterWord(counterId), 1ull);
    }
    return ncclSuccess;
  }

  __device__ unsigned long long readSignal(int id) const {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(signalWord(comm.lsaRank, id)) : "memory");
    return v;
  }
  __device__ unsigned long long readCounter(int id) const { return *(volatile unsigned long long*)counterWord(id); }

  /* Returns ncclTimeout when the signal did not reach `value` within the budget (or the communicator was aborted). */
  __device__ ncclResult_t waitSignal(int id, unsigned long long value, unsigned long long timeoutCycles = 0) const {
    if (id < 0 || id >= comm.ginSignalCount) return ncclInvalidUsage;
    const unsigned long long budget = timeoutCycles ? timeoutCycles : comm.timeoutCycles;
    const long long start = clock64();
    unsigned spins = 0;
    while (readSignal(id) < value) {
      if ((++spins & 0xff) == 0 && ((unsigned long long)(clock64() - start) >= budget || ncclTestAbort(comm))) return ncclTimeout;
    }
    nccl_device::fenceAcqRelSys();
    return ncclSuccess;
  }
  __device__ void resetSignal(int id) { *(volatile unsigned long long*)signalWord(comm.lsaRank, id) = 0; }
  __device__ void resetCounter(int id) { *(volatile unsigned long long*)counterWord(id) = 0; }
  __device__ void flush() { nccl_device::fenceAcqRelSys(); }
};
#endif
#endif
