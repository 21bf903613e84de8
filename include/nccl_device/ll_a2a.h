/*
 * Low-latency all-to-all session: 16-byte lines {data, epoch, data, epoch} stored straight into a
 * peer's slots; the receiver polls a slot until both epochs match. Slots are double-buffered by
 * epoch parity. 8 payload bytes per line.
 * Reference parity: src/include/nccl_device/ll_a2a.h, impl/ll_a2a__funcs.h:53-86.
 */
#ifndef NCCL_DEVICE_LL_A2A_H_
#define NCCL_DEVICE_LL_A2A_H_
#include "coop.h"
#include "utility.h"
#if defined(__CUDACC__)
template <typename Coop>
struct ncclLLA2ASession {
  Coop coop;
  const ncclDevComm_t& comm;
  int block;        /* which LLA2A block of the communicator this CTA uses */
  uint32_t epoch;
  __device__ ncclLLA2ASession(Coop coop_, const ncclDevComm_t& c, ncclTeam_t, int blockIndex)
      : coop(coop_), comm(c), block(blockIndex), epoch(c.llA2AEpochs[blockIndex] + 1) { if (epoch == 0) epoch = 1; }
  /* slot `slot` written by rank `src`, inside rank `owner`'s window */
  __device__ char* line(int owner, int src, int slot) const {
    size_t perBlock = (size_t)2 * NCCL_DEVICE_MAX_LSA * comm.llA2ASlotCount * 16;
    return (char*)comm.resource.peerPtr[owner] + comm.llA2AOffset + block * perBlock +
           ((size_t)((epoch & 1) * NCCL_DEVICE_MAX_LSA + src) * comm.llA2ASlotCount + slot) * 16;
  }
  __device__ void send(int peer, int slot, uint64_t value) {
    nccl_device::stVolatile16(line(peer, comm.lsaRank, slot), make_uint4((uint32_t)value, epoch, (uint32_t)(value >> 32), epoch));
  }
  __device__ void bcast(int slot, uint64_t value) {
    for (int p = 0; p < comm.lsaSize; ++p) if (p != comm.lsaRank) send(p, slot, value);
  }
  /* Returns ncclTimeout when the line did not arrive within the budget. */
  __device__ ncclResult_t recv(int src, int slot, uint64_t* value, unsigned long long timeoutCycles = 0) {
    const unsigned long long budget = timeoutCycles ? timeoutCycles : comm.timeoutCycles;
    const char* l = line(comm.lsaRank, src, slot);
    const long long start = clock64();
    unsigned spins = 0;
    uint4 v = nccl_device::ldVolatile16(l);
    while (v.y != epoch || v.w != epoch) {
      if ((++spins & 0xff) == 0 && ((unsigned long long)(clock64() - start) >= budget || ncclTestAbort(comm))) return ncclTimeout;
      v = nccl_device::ldVolatile16(l);
    }
    *value = (uint64_t)v.x | ((uint64_t)v.z << 32);
    return ncclSuccess;
  }
  /* Sum over the lines of every peer (and `mine`) as two packed floats. */
  __device__ ncclResult_t recvReduceFloat2(int slot, float2 mine, float2* out) {
    float2 acc = mine;
    for (int s = 0; s < comm.lsaSize; ++s) {
      if (s == comm.lsaRank) continue;
      uint64_t v;
      ncclResult_t r = recv(s, slot, &v);
      if (r != ncclSuccess) return r;
      acc.x += __uint_as_float((uint32_t)v);
      acc.y += __uint_as_float((uint32_t)(v >> 32));
    }
    *out = acc;
    return ncclSuccess;
  }
  __device__ void endEpoch() { coop.sync(); if (coop.thread_rank() == 0) comm.llA2AEpochs[block] = epoch; }
};
#endif
#endif
