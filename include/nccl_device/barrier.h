/*
 * Barrier over a whole communicator for device code. The reference combines an LSA barrier with a
 * rail barrier over network signals (ncclBarrierSession = LSA + GIN); here every rank of a device
 * communicator is inside one load/store team, so the session is the LSA barrier.
 * Reference parity: src/include/nccl_device/barrier.h, gin_barrier.h.
 */
#ifndef NCCL_DEVICE_BARRIER_H_
#define NCCL_DEVICE_BARRIER_H_
#include "lsa_barrier.h"
#if defined(__CUDACC__)
template <typename Coop>
struct ncclBarrierSession : ncclLsaBarrierSession<Coop> {
  __device__ ncclBarrierSession(Coop coop, const ncclDevComm_t& c, ncclTeam_t team, int barrierIndex)
      : ncclLsaBarrierSession<Coop>(coop, c, team, barrierIndex) {}
};
#endif
#endif
