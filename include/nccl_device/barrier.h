/*
 * Barrier over a whole communicator for device code. The reference combines an LSA barrier with a
 * rail barrier over network signals (ncclBarrierSession = LSA + GIN); here every rank of a device
 * communicator is inside one load/store team, so the session is the LSA barrier.
 * Reference parity: src/include/nccl_device/barrier.h, gin_barrier.h.
 */
#ifndef NCCL_DEVICE_BARRIER_H_
#define NCCL_DEVICE_BARRIER_H_
#include "lsa_barrier.h"
#include "gin.h"
#if defined(__CUDACC__)
/* What a network barrier would have to drain; with peer stores there is nothing queued in a NIC, the
 * barrier's release / acquire fences cover puts and gets alike. */
enum ncclGinFenceLevel : uint32_t { None = 0, Put = 1u << 0, Get = 1u << 1, Relaxed = None };
__host__ __device__ constexpr ncclGinFenceLevel operator|(ncclGinFenceLevel a, ncclGinFenceLevel b) { return (ncclGinFenceLevel)((uint32_t)a | (uint32_t)b); }
__host__ __device__ constexpr ncclGinFenceLevel operator&(ncclGinFenceLevel a, ncclGinFenceLevel b) { return (ncclGinFenceLevel)((uint32_t)a & (uint32_t)b); }
struct ncclGinAllContexts {
  const ncclDevComm_t& comm;
  __host__ __device__ constexpr ncclGinAllContexts(const ncclDevComm_t& c) : comm(c) {}
};

template <typename Coop>
struct ncclBarrierSession : ncclLsaBarrierSession<Coop> {
  typedef ncclLsaBarrierSession<Coop> Base;
  __device__ ncclBarrierSession(Coop coop, const ncclDevComm_t& c, ncclTeam_t team, int barrierIndex) : Base(coop, c, team, barrierIndex) {}
  /* the reference's tag constructors */
  __device__ ncclBarrierSession(Coop coop, ncclTeamTagLsa, const ncclDevComm_t& c, uint32_t index, bool multimem = false) : Base(coop, c, ncclTeamTagLsa(), index, multimem) {}
  __device__ ncclBarrierSession(Coop coop, ncclTeamTagWorld, const ncclGin& gin, uint32_t index, bool multimem = false) : Base(coop, gin.comm, ncclTeamTagLsa(), index, multimem) {}
  __device__ ncclBarrierSession(Coop coop, ncclTeamTagRail, const ncclGin& gin, uint32_t index) : Base(coop, gin.comm, ncclTeamTagLsa(), index) {}
  using Base::sync;
  __device__ void sync(Coop coop, cuda::memory_order order, ncclGinFenceLevel) { Base::sync(coop, order); }
  __device__ ncclResult_t sync(Coop coop, cuda::memory_order order, ncclGinFenceLevel, uint64_t timeoutCycles) { return Base::sync(coop, order, timeoutCycles); }
  __device__ Base& lsaBarrier() { return *this; }
};

/* Barrier over network signals in the reference; the same load/store barrier here. It uses the LSA barrier
 * slots of the device communicator: count them in lsaBarrierCount as well as in railGinBarrierCount. */
template <typename Coop>
struct ncclGinBarrierSession : ncclLsaBarrierSession<Coop> {
  typedef ncclLsaBarrierSession<Coop> Base;
  __device__ ncclGinBarrierSession(Coop coop, const ncclGin& gin, ncclTeamTagWorld, uint32_t index) : Base(coop, gin.comm, ncclTeamTagLsa(), index) {}
  __device__ ncclGinBarrierSession(Coop coop, const ncclGin& gin, ncclTeamTagRail, uint32_t index) : Base(coop, gin.comm, ncclTeamTagLsa(), index) {}
  __device__ ncclGinBarrierSession(Coop coop, ncclGinAllContexts all, ncclTeamTagWorld, uint32_t index) : Base(coop, all.comm, ncclTeamTagLsa(), index) {}
  __device__ ncclGinBarrierSession(Coop coop, ncclGinAllContexts all, ncclTeamTagRail, uint32_t index) : Base(coop, all.comm, ncclTeamTagLsa(), index) {}
  using Base::sync;
  __device__ void sync(Coop coop, cuda::memory_order order, ncclGinFenceLevel) { Base::sync(coop, order); }
  __device__ ncclResult_t sync(Coop coop, cuda::memory_order order, ncclGinFenceLevel, uint64_t timeoutCycles) { return Base::sync(coop, order, timeoutCycles); }
};
#endif
#endif
