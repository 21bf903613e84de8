/*
 * Barrier among the ranks of the load/store team, executed by one cooperative group per rank.
 * Each barrier index owns one inbox word per peer in every rank's resource window and a private
 * epoch; arrive() release-stores the new epoch into every peer's inbox, wait() polls the local
 * inbox. Waits are bounded: after timeoutCycles (or when the communicator is aborted) they give
 * up and return ncclTimeout, leaving the kernel free to finish.
 * Reference parity: src/include/nccl_device/lsa_barrier.h, impl/lsa_barrier__funcs.h:55-175.
 */
#ifndef NCCL_DEVICE_LSA_BARRIER_H_
#define NCCL_DEVICE_LSA_BARRIER_H_
#include "coop.h"
#include "utility.h"
#if defined(__CUDACC__)
#include <cuda/atomic>
namespace nccl_device {
__host__ __device__ inline bool orderReleases(cuda::memory_order o) {
  return o == cuda::memory_order_release || o == cuda::memory_order_acq_rel || o == cuda::memory_order_seq_cst;
}
__host__ __device__ inline bool orderAcquires(cuda::memory_order o) {
  return o == cuda::memory_order_acquire || o == cuda::memory_order_consume || o == cuda::memory_order_acq_rel || o == cuda::memory_order_seq_cst;
}
}  // namespace nccl_device
template <typename Coop>
struct ncclLsaBarrierSession {
  Coop coop;
  const ncclDevComm_t& comm;
  int index;
  uint32_t epoch;
  bool autoFinish;   /* the tag constructor stores the epoch back when the session goes out of scope */
  __device__ ncclLsaBarrierSession(Coop coop_, const ncclDevComm_t& c, ncclTeam_t /*lsa team*/, int barrierIndex)
      : coop(coop_), comm(c), index(barrierIndex), epoch(c.barrierEpochs[barrierIndex]), autoFinish(false) {}
  /* The reference's spelling: team chosen by tag, scoped session (no finish() call), memory orders instead of flags. */
  __device__ ncclLsaBarrierSession(Coop coop_, const ncclDevComm_t& c, ncclTeamTagLsa, uint32_t barrierIndex, bool /*multimem*/ = false)
      : coop(coop_), comm(c), index((int)barrierIndex), epoch(c.barrierEpochs[barrierIndex]), autoFinish(true) {}
  __device__ ~ncclLsaBarrierSession() { if (autoFinish) finish(); }
  __device__ void arrive(Coop, cuda::memory_order order) { arrive(nccl_device::orderReleases(order)); }
  __device__ void wait(Coop, cuda::memory_order order) { (void)wait(0ull, nccl_device::orderAcquires(order)); }
  __device__ ncclResult_t wait(Coop, cuda::memory_order order, uint64_t timeoutCycles) { return wait((unsigned long long)timeoutCycles, nccl_device::orderAcquires(order)); }
  __device__ void sync(Coop, cuda::memory_order order) { (void)sync(0ull, nccl_device::orderReleases(order), nccl_device::orderAcquires(order)); }
  __device__ ncclResult_t sync(Coop, cuda::memory_order order, uint64_t timeoutCycles) {
    return sync((unsigned long long)timeoutCycles, nccl_device::orderReleases(order), nccl_device::orderAcquires(order));
  }
  __device__ uint32_t* inbox(int owner, int src) const {
    return (uint32_t*)((char*)comm.resource.peerPtr[owner] + comm.lsaBarrierOffset) + (size_t)index * NCCL_DEVICE_MAX_LSA + src;
  }
  /* With release, everything the group wrote before arrive() is visible to a peer after its matching
   * wait(acquire). A barrier that only announces "this kernel has started" needs neither (data
   * written by earlier kernels is already visible), and system-scope fences cost microseconds. */
  __device__ void arrive(bool release = true) {
    coop.sync();
    ++epoch;
    for (int p = coop.thread_rank(); p < comm.lsaSize; p += coop.size()) {
      if (p == comm.lsaRank) continue;
      if (release) nccl_device::fenceAcqRelSys();
      nccl_device::stRelaxedSys(inbox(p, comm.lsaRank), epoch);
    }
  }
  __device__ ncclResult_t wait(unsigned long long timeoutCycles = 0, bool acquire = true) {
    const unsigned long long budget = timeoutCycles ? timeoutCycles : comm.timeoutCycles;
    ncclResult_t res = ncclSuccess;
    for (int p = coop.thread_rank(); p < comm.lsaSize; p += coop.size()) {
      if (p == comm.lsaRank) continue;
      const uint32_t* w = inbox(comm.lsaRank, p);
      const long long start = clock64();
      unsigned spins = 0;
      while (nccl_device::rollingDiff(nccl_device::ldRelaxedSys(w), epoch) < 0) {
        if ((++spins & 0xff) == 0 && ((unsigned long long)(clock64() - start) >= budget || ncclTestAbort(comm))) { res = ncclTimeout; break; }
      }
      if (acquire) nccl_device::fenceAcqRelSys();
    }
    coop.sync();
    return res;
  }
  __device__ ncclResult_t sync(unsigned long long timeoutCycles = 0, bool release = true, bool acquire = true) { arrive(release); return wait(timeoutCycles, acquire); }
  /* Stores the epoch for the next kernel; call once, by the last user of this index in the kernel. */
  __device__ void finish() { if (coop.thread_rank() == 0) comm.barrierEpochs[index] = epoch; }
};
#endif
#endif
