/*
 * GPU-initiated networking surface of the device API. Ranks outside the load/store team are
 * reached through a network backend; this build serves one NVLink domain, so the put / signal
 * calls resolve to peer stores and counters in the resource window when the target is inside the
 * team and report ncclInvalidUsage otherwise (no RDMA backend is linked).
 * Reference parity: src/include/nccl_device/gin.h:21-333 (ncclGin: put, signal, wait, counters).
 */
#ifndef NCCL_DEVICE_GIN_H_
#define NCCL_DEVICE_GIN_H_
#include "core.h"
#include "utility.h"
#if defined(__CUDACC__)
struct ncclGin {
  const ncclDevComm_t& comm;
  __device__ explicit ncclGin(const ncclDevComm_t& c, int /*context*/ = 0) : comm(c) {}
  template <typename Coop>
  __device__ ncclResult_t put(Coop coop, ncclTeam_t team, int peer, ncclWindow_t dstWin, size_t dstOffset, ncclWindow_t srcWin, size_t srcOffset, size_t bytes) {
    int world = ncclTeamRankToWorld(comm, team, peer);
    if (world < 0 || world >= comm.lsaSize) return ncclInvalidUsage;
    const char* s = (const char*)ncclGetLocalPointer(srcWin, srcOffset);
    char* d = (char*)ncclGetLsaPointer(dstWin, dstOffset, world);
    for (size_t i = coop.thread_rank() * 16; i + 16 <= bytes; i += (size_t)coop.size() * 16) *(uint4*)(d + i) = *(const uint4*)(s + i);
    for (size_t b = bytes / 16 * 16 + coop.thread_rank(); b < bytes; b += coop.size()) d[b] = s[b];
    return ncclSuccess;
  }
  __device__ void flush() { nccl_device::fenceAcqRelSys(); }
};
#endif
#endif
