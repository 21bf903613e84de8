/*
 * Device API, core types: device communicator, windows, teams and pointer getters.
 * A kernel that includes <nccl_device.h> can address the memory of every rank of its load/store
 * team (the ranks whose memory is mapped here, NVLink domain) through registered windows, use the
 * NVLink-multicast alias of a window, and synchronise with the other ranks.
 * Reference parity: src/include/nccl_device/core.h (:78-142 requirements, :175-192 properties,
 * :210-255 teams, :267-275 pointer getters), impl/core__types.h.
 */
#ifndef NCCL_DEVICE_CORE_H_
#define NCCL_DEVICE_CORE_H_

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "nccl.h"

#define NCCL_DEVICE_MAX_LSA 8

/* Device-visible description of a registered window (ncclWindow_t points to one of these). */
struct ncclWindow_vidmem {
  void* peerPtr[NCCL_DEVICE_MAX_LSA]; /* peerPtr[p]: rank p's part of the window as mapped on this GPU */
  void* mcPtr;                        /* multicast alias of the window, or NULL */
  size_t size;
  int rank, nRanks;
  void* userPtr;
  struct ncclWindow_vidmem* devSelf;  /* device copy of this struct: what kernels receive */
  void* hostState;
  unsigned long long magic;
};

typedef struct ncclTeam {
  int nRanks;
  int rank;
  int stride;
} ncclTeam_t;

/* Byte offset of a requested buffer inside the communicator's resource window. */
typedef uint32_t ncclDevResourceHandle;
typedef ncclDevResourceHandle ncclDevResourceHandle_t;

/* Resources a kernel asks for when the device communicator is created. */
typedef struct ncclDevResourceRequirements {
  struct ncclDevResourceRequirements* next;
  size_t bufferSize;
  size_t bufferAlign;
  uint32_t* outBufferHandle;   /* receives the byte offset of the buffer inside the resource window */
  int ginSignalCount;
  int ginCounterCount;
  uint32_t* outGinSignalStart;
  uint32_t* outGinCounterStart;
} ncclDevResourceRequirements_t;

typedef struct ncclTeamRequirements {
  struct ncclTeamRequirements* next;
  ncclTeam_t team;
  int multimem;
  uint32_t* outMultimemHandle;
} ncclTeamRequirements_t;

typedef struct ncclDevCommRequirements {
  size_t size;
  unsigned int magic;
  unsigned int version;
  ncclDevResourceRequirements_t* resourceRequirementsList;
  ncclTeamRequirements_t* teamRequirementsList;
  int lsaMultimem;             /* want the multicast alias of the resource window */
  int barrierCount;            /* hybrid (LSA + rail) barriers */
  int lsaBarrierCount;         /* barriers among the load/store team, one per CTA that synchronises */
  int railGinBarrierCount;
  int lsaLLA2ABlockCount;      /* CTAs that run low-latency all-to-all sessions */
  int lsaLLA2ASlotCount;       /* 16-byte slots per CTA and peer */
  int ginForceEnable;
  int ginContextCount;
  int ginSignalCount;
  int ginCounterCount;
  int ginConnectionType;
  int ginExclusiveContexts;
  int ginQueueDepth;
  int ginTrafficClass;
  int worldGinBarrierCount;
  int ginStrongSignalsRequired;
  int ginVaSignalsRequired;
} ncclDevCommRequirements_t;

#define NCCL_DEV_COMM_REQUIREMENTS_MAGIC 0xdec0de01u
#define NCCL_DEV_COMM_REQUIREMENTS_INITIALIZER \
  { sizeof(ncclDevCommRequirements_t), NCCL_DEV_COMM_REQUIREMENTS_MAGIC, NCCL_VERSION_CODE, NULL, NULL, 0, 0, 0, 0, 0, 0, 0, 4, 0, 0, 0, 0, 0, 0, 0, 0, 0 }

typedef struct ncclCommProperties {
  size_t size;
  unsigned int magic;
  unsigned int version;
  int rank;
  int nRanks;
  int cudaDev;
  int nvmlDev;
  int deviceApiSupport;
  int multimemSupport;
  int ginType;
  int nLsaTeams;
  int hostRmaSupport;
  int railedGinType;
} ncclCommProperties_t;

#define NCCL_COMM_PROPERTIES_INITIALIZER \
  { sizeof(ncclCommProperties_t), 0xdec0de02u, NCCL_VERSION_CODE, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0 }

/* Passed by value to kernels. */
typedef struct ncclDevComm {
  int rank, nRanks;
  int lsaRank, lsaSize;
  struct ncclWindow_vidmem resource;   /* the communicator's resource window (barriers, LL slots, user buffers) */
  uint32_t lsaBarrierOffset;           /* byte offsets inside the resource window */
  int lsaBarrierCount;
  uint32_t llA2AOffset;
  int llA2ABlockCount, llA2ASlotCount;
  uint32_t* barrierEpochs;             /* private device words: one epoch per LSA barrier */
  uint32_t* llA2AEpochs;               /* private device words: one epoch per LLA2A block */
  uint32_t ginSignalOffset;            /* u64 signal words [ginSignalCount], in the resource window */
  int ginSignalCount;
  uint32_t ginCounterOffset;           /* u64 local completion counters [ginCounterCount] */
  int ginCounterCount;
  const uint32_t* abortFlag;           /* host-mapped: non-zero once the communicator is aborted */
  unsigned long long timeoutCycles;    /* default budget of device-side waits */
  /* Proxy mode of the put / signal surface: operations are queued for a host thread that runs them with the copy
   * engines (ncclGin in nccl_device/gin.h). All null / zero when puts are peer stores. */
  struct ncclGinProxyDesc* ginProxyRing;        /* host-mapped ring of descriptors */
  unsigned long long* ginProxyHead;             /* device word: next slot to claim */
  const volatile unsigned long long* ginProxyTail;   /* host-mapped: descriptors the host has taken */
  const volatile unsigned long long* ginProxyDone;   /* device word: operations completed (written in stream order) */
  unsigned int ginProxyMask;                    /* ring size - 1 */
} ncclDevComm_t;

/* One queued operation of the proxy mode: an optional copy followed by an optional add on a remote signal word and
 * on a local completion counter, all resolved to addresses by the issuing thread. `seq` is written last. */
typedef struct ncclGinProxyDesc {
  void* dst;
  const void* src;
  unsigned long long bytes;
  unsigned long long* signal;
  unsigned long long signalAdd;
  unsigned long long* counter;
  unsigned long long pad;
  volatile unsigned long long seq;     /* index of this operation + 1 once the descriptor is complete */
} ncclGinProxyDesc_t;

typedef enum { NCCL_GIN_TYPE_NONE = 0, NCCL_GIN_TYPE_PROXY = 2, NCCL_GIN_TYPE_GDAKI = 3, NCCL_GIN_TYPE_GPI = 4 } ncclGinType_t;

#ifdef __cplusplus
extern "C" {
#endif
ncclResult_t ncclCommQueryProperties(ncclComm_t comm, ncclCommProperties_t* props);
ncclResult_t ncclDevCommCreate(ncclComm_t comm, const ncclDevCommRequirements_t* reqs, ncclDevComm_t* devComm);
ncclResult_t ncclDevCommDestroy(ncclComm_t comm, const ncclDevComm_t* devComm);
/* Host-side pointer getters: where rank `peer`'s part of the window is mapped in this process. */
ncclResult_t ncclGetLsaDevicePointer(ncclWindow_t win, size_t offset, int peer, void** out);
ncclResult_t ncclGetLsaMultimemDevicePointer(ncclWindow_t win, size_t offset, void** out);
ncclResult_t ncclGetPeerDevicePointer(ncclWindow_t win, size_t offset, int peer, void** out);
/* The device copy of a window handle, to pass to kernels. */
ncclResult_t ncclWinGetDeviceHandle(ncclWindow_t win, ncclWindow_t* devHandle);
#ifdef __cplusplus
}
#endif

#if defined(__CUDACC__)
__host__ __device__ inline ncclTeam_t ncclTeamWorld(const ncclDevComm_t& c) { ncclTeam_t t = {c.nRanks, c.rank, 1}; return t; }
__host__ __device__ inline ncclTeam_t ncclTeamLsa(const ncclDevComm_t& c) { ncclTeam_t t = {c.lsaSize, c.lsaRank, 1}; return t; }
__host__ __device__ inline ncclTeam_t ncclTeamRail(const ncclDevComm_t& c) { ncclTeam_t t = {c.nRanks / c.lsaSize, c.rank / c.lsaSize, c.lsaSize}; return t; }
__host__ __device__ inline int ncclTeamRankToWorld(const ncclDevComm_t& c, ncclTeam_t t, int r) { return c.rank + (r - t.rank) * t.stride; }
/* Tags that select one of the three built-in teams in constructors. */
struct ncclTeamTagWorld {};
struct ncclTeamTagLsa {};
struct ncclTeamTagRail {};
/* Rank of team member r inside the load/store team (the team's ranks must lie in this rank's load/store team). */
__host__ __device__ inline int ncclTeamRankToLsa(const ncclDevComm_t& c, ncclTeam_t t, int r) { return c.lsaRank + (r - t.rank) * t.stride; }
/* Teams are arithmetic progressions of world ranks around the caller: member i of team t is world rank
 * self + (i - t.rank) * t.stride. The helpers below translate between two such teams. */
__host__ __device__ inline bool ncclTeamRankIsMember(ncclTeam_t a, ncclTeam_t b, int bPeer) {
  const int delta = (bPeer - b.rank) * b.stride;
  if (delta % a.stride) return false;
  const int i = a.rank + delta / a.stride;
  return i >= 0 && i < a.nRanks;
}
__host__ __device__ inline int ncclTeamRankToTeam(ncclTeam_t a, ncclTeam_t b, int bPeer) { return a.rank + (bPeer - b.rank) * b.stride / a.stride; }
/* Split a team of n ranks into blocks of innerSize consecutive members: the block this rank is in, and the team
 * of the ranks that hold the same position in every block. */
__host__ __device__ inline ncclTeam_t ncclTeamInnerFactor(ncclTeam_t parent, int innerSize) {
  ncclTeam_t t = {innerSize, parent.rank % innerSize, parent.stride};
  return t;
}
__host__ __device__ inline ncclTeam_t ncclTeamOuterFactor(ncclTeam_t parent, int innerSize) {
  ncclTeam_t t = {parent.nRanks / innerSize, parent.rank / innerSize, parent.stride * innerSize};
  return t;
}
/* The index-th member (as a rank of `parent`) of parent minus subset; subset must be a subset of parent. */
__host__ __device__ inline int ncclTeamRankInDifference(ncclTeam_t parent, ncclTeam_t subset, int index) {
  for (int i = 0; i < parent.nRanks; ++i) {
    if (ncclTeamRankIsMember(subset, parent, i)) continue;
    if (index-- == 0) return i;
  }
  return -1;
}

__device__ inline void* ncclGetLocalPointer(ncclWindow_t w, size_t offset) { return (char*)w->peerPtr[w->rank] + offset; }
__device__ inline void* ncclGetLsaPointer(ncclWindow_t w, size_t offset, int lsaPeer) { return (char*)w->peerPtr[lsaPeer] + offset; }
__device__ inline void* ncclGetPeerPointer(ncclWindow_t w, size_t offset, ncclTeam_t team, int peer) {
  return (char*)w->peerPtr[w->rank + (peer - team.rank) * team.stride] + offset;
}
__device__ inline void* ncclGetMultimemPointer(ncclWindow_t w, size_t offset) { return w->mcPtr ? (char*)w->mcPtr + offset : (void*)0; }
__device__ inline void* ncclGetLsaMultimemPointer(ncclWindow_t w, size_t offset, const ncclDevComm_t&) { return ncclGetMultimemPointer(w, offset); }
/* Pointers into the communicator's own resource window. */
__device__ inline void* ncclGetResourceBufferLocalPointer(const ncclDevComm_t& c, uint32_t handle) { return (char*)c.resource.peerPtr[c.lsaRank] + handle; }
__device__ inline void* ncclGetResourceBufferLsaPointer(const ncclDevComm_t& c, uint32_t handle, int peer) { return (char*)c.resource.peerPtr[peer] + handle; }
__device__ inline void* ncclGetResourceBufferMultimemPointer(const ncclDevComm_t& c, uint32_t handle) { return c.resource.mcPtr ? (char*)c.resource.mcPtr + handle : (void*)0; }
__device__ inline void* ncclGetResourceBufferLsaMultimemPointer(const ncclDevComm_t& c, ncclDevResourceHandle handle) { return ncclGetResourceBufferMultimemPointer(c, handle); }
__device__ inline void* ncclGetResourceBufferPeerPointer(const ncclDevComm_t& c, ncclDevResourceHandle handle, ncclTeam_t team, int peer) {
  return (char*)c.resource.peerPtr[c.lsaRank + (peer - team.rank) * team.stride] + handle;
}
__host__ __device__ inline size_t ncclGetResourceBufferOffset(ncclDevResourceHandle_t handle) { return handle; }
__device__ inline void* ncclGetPeerPointer(ncclWindow_t w, size_t offset, int worldPeer) { return (char*)w->peerPtr[worldPeer] + offset; }
#endif

#endif
