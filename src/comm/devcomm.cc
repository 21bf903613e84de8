// Host side of the device API: communicator properties, creation of device communicators (a
// zeroed symmetric resource window holding barrier inboxes, low-latency all-to-all slots and the
// buffers the caller asked for, plus private epoch words) and host-side pointer getters.
// Reference parity: src/dev_runtime.cc (ncclDevrInitOnce :221-292, ncclDevCommCreate :1063-1235,
// ncclCommQueryProperties, ncclGetLsaDevicePointer :1316-1370).
#include <map>
#include <strings.h>

#include "../mem/symmetric.h"
#include "comm.h"
#include "device_plane.h"
#include "../contrib/gin_proxy.h"
#include "../plugin/plugin.h"
#include "nccl_device/core.h"

namespace b200 {

ncclResult_t windowRegister(ncclComm_t comm, void* buff, size_t size, ncclWindow_t* win, int winFlags);   // mem/register.cc

B200_PARAM(DevCommTimeoutMs, "B200_DEVCOMM_TIMEOUT_MS", 10000, "default budget of device-API waits (barriers, low-latency receives), milliseconds");

struct DevCommState {
  void* buf = nullptr;
  size_t bytes = 0;
  ncclWindow_t win = nullptr;
  uint32_t* priv = nullptr;
  GinProxy* proxy = nullptr;
};
static std::mutex gDevLock;
static std::map<std::pair<ncclComm*, const uint32_t*>, DevCommState> gDevComms;

static size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace b200

using namespace b200;

extern "C" {

ncclResult_t ncclCommQueryProperties(ncclComm_t comm, ncclCommProperties_t* props) {
  if (!commValid(comm) || !props) return ncclInvalidArgument;
  NCCLCHECK(commEnsureReady(comm));
  props->rank = comm->rank;
  props->nRanks = comm->nRanks;
  props->cudaDev = comm->cudaDev;
  props->nvmlDev = comm->nvmlDev;
  const bool lsa = !comm->hostOnly && (comm->nRanks == 1 || (comm->lsaAll && comm->sym && comm->nRanks <= kMaxRanks));
  props->deviceApiSupport = lsa ? 1 : 0;
  props->multimemSupport = lsa && comm->sym && comm->sym->mcUsable ? 1 : 0;
  // the put / signal surface can be served by a host proxy thread (inside the load/store domain); no device-driven NIC backend
  props->ginType = lsa ? NCCL_GIN_TYPE_PROXY : NCCL_GIN_TYPE_NONE;
  // a network plugin with a table for GPU-initiated networking is reported here (its kind is the plugin's business: the
  // proxy kind is the conservative answer); nothing in this build hands traffic to it
  const GinPluginInfo* gp = comm->nNodes > 1 ? netGinPluginInfo() : nullptr;
  props->railedGinType = gp && gp->present && gp->devices > 0 ? NCCL_GIN_TYPE_PROXY : NCCL_GIN_TYPE_NONE;
  props->nLsaTeams = lsa ? 1 : comm->nNodes;
  props->hostRmaSupport = 1;   // ncclPutSignal / ncclSignal / ncclWaitSignal
  return ncclSuccess;
}

ncclResult_t ncclDevCommCreate(ncclComm_t comm, const ncclDevCommRequirements_t* reqs, ncclDevComm_t* out) {
  if (!commValid(comm) || !reqs || !out) return ncclInvalidArgument;
  NCCLCHECK(commEnsureReady(comm));
  if (reqs->magic != NCCL_DEV_COMM_REQUIREMENTS_MAGIC || reqs->size != sizeof(ncclDevCommRequirements_t)) {
    WARN("ncclDevCommCreate : requirements were not initialised with NCCL_DEV_COMM_REQUIREMENTS_INITIALIZER");
    return ncclInvalidArgument;
  }
  ncclCommProperties_t props = NCCL_COMM_PROPERTIES_INITIALIZER;
  NCCLCHECK(ncclCommQueryProperties(comm, &props));
  if (!props.deviceApiSupport) { WARN("ncclDevCommCreate : the ranks of this communicator do not share one load/store domain"); return ncclInvalidUsage; }
  if (reqs->railGinBarrierCount || reqs->worldGinBarrierCount) {
    WARN("ncclDevCommCreate : rail / world barriers were requested but this build serves one NVLink domain (use the load/store barriers)");
    return ncclInvalidUsage;
  }
  // put / signal through the host proxy thread instead of peer stores: asked for by the requirements or by NCCL_GIN_TYPE
  bool wantProxy = reqs->ginConnectionType > 0 || reqs->ginForceEnable != 0;
  if (const char* e = getEnv("NCCL_GIN_TYPE")) {
    if (!strcasecmp(e, "PROXY") || !strcmp(e, "2")) wantProxy = true;
    else if (!strcasecmp(e, "NONE") || !strcmp(e, "0")) wantProxy = false;
    else if (*e) { WARN("NCCL_GIN_TYPE=%s: only NONE and PROXY are available (no device-driven NIC backend)", e); return ncclInvalidUsage; }
  }
  if (reqs->lsaMultimem && !props.multimemSupport) { WARN("ncclDevCommCreate : multimem requested but NVLink multicast is not available"); return ncclInvalidUsage; }
  int cur = -1;
  CUDACHECK(cudaGetDevice(&cur));
  if (cur != comm->cudaDev) CUDACHECK(cudaSetDevice(comm->cudaDev));

  // layout of the resource window
  const int nBar = std::max(reqs->lsaBarrierCount + reqs->barrierCount, 1);
  const int llBlocks = reqs->lsaLLA2ABlockCount, llSlots = std::max(reqs->lsaLLA2ASlotCount, llBlocks ? 1 : 0);
  size_t off = 0;
  const size_t barOff = off;
  off = alignUp(off + (size_t)nBar * NCCL_DEVICE_MAX_LSA * sizeof(uint32_t), 256);
  const size_t llOff = off;
  off = alignUp(off + (size_t)llBlocks * 2 * NCCL_DEVICE_MAX_LSA * llSlots * 16, 256);
  // signals and counters of the GPU-initiated put / signal surface: served over NVLink inside the team
  int nSignals = reqs->ginSignalCount, nCounters = reqs->ginCounterCount;
  for (ncclDevResourceRequirements_t* r = reqs->resourceRequirementsList; r; r = r->next) {
    if (r->outGinSignalStart) *r->outGinSignalStart = (uint32_t)nSignals;
    if (r->outGinCounterStart) *r->outGinCounterStart = (uint32_t)nCounters;
    nSignals += r->ginSignalCount;
    nCounters += r->ginCounterCount;
  }
  const size_t sigOff = off;
  off = alignUp(off + (size_t)nSignals * 8, 256);
  const size_t cntOff = off;
  off = alignUp(off + (size_t)nCounters * 8, 256);
  for (ncclDevResourceRequirements_t* r = reqs->resourceRequirementsList; r; r = r->next) {
    size_t a = std::max<size_t>(r->bufferAlign, 16);
    if (a & (a - 1)) { WARN("ncclDevCommCreate : buffer alignment %zu is not a power of two", a); return ncclInvalidArgument; }
    off = alignUp(off, a);
    if (off + r->bufferSize > 0xffffffffull) { WARN("ncclDevCommCreate : resource buffers exceed 4 GiB"); return ncclInvalidArgument; }
    if (r->outBufferHandle) *r->outBufferHandle = (uint32_t)off;
    off += r->bufferSize;
  }
  for (ncclTeamRequirements_t* t = reqs->teamRequirementsList; t; t = t->next)
    if (t->outMultimemHandle) *t->outMultimemHandle = 0;   // the one multicast alias covers the whole team
  const size_t bytes = alignUp(std::max<size_t>(off, 4096), 4096);

  DevCommState st;
  st.bytes = bytes;
  ncclResult_t res = ncclMemAlloc(&st.buf, bytes);
  if (res != ncclSuccess) return res;
  if (cudaMemset(st.buf, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) { (void)cudaGetLastError(); ncclMemFree(st.buf); return ncclUnhandledCudaError; }
  res = windowRegister(comm, st.buf, bytes, &st.win, NCCL_WIN_COLL_SYMMETRIC);
  if (res != ncclSuccess || !st.win) { ncclMemFree(st.buf); return res != ncclSuccess ? res : ncclInternalError; }
  const size_t nPriv = (size_t)nBar + llBlocks + 4;
  if (cudaMalloc(&st.priv, nPriv * sizeof(uint32_t)) != cudaSuccess || cudaMemset(st.priv, 0, nPriv * sizeof(uint32_t)) != cudaSuccess) {
    (void)cudaGetLastError();
    ncclCommWindowDeregister(comm, st.win);
    ncclMemFree(st.buf);
    return ncclUnhandledCudaError;
  }
  cudaDeviceSynchronize();
  // nobody may store into a peer's window before that peer has zeroed it
  if (comm->nRanks > 1) NCCLCHECK(bootstrapBarrier(comm->bootstrap));

  memset(out, 0, sizeof(*out));
  out->rank = comm->rank;
  out->nRanks = comm->nRanks;
  out->lsaRank = comm->rank;
  out->lsaSize = comm->nRanks;
  out->resource = *st.win;
  out->resource.hostState = nullptr;
  out->lsaBarrierOffset = (uint32_t)barOff;
  out->lsaBarrierCount = nBar;
  out->llA2AOffset = (uint32_t)llOff;
  out->llA2ABlockCount = llBlocks;
  out->llA2ASlotCount = llSlots;
  out->ginSignalOffset = (uint32_t)sigOff;
  out->ginSignalCount = nSignals;
  out->ginCounterOffset = (uint32_t)cntOff;
  out->ginCounterCount = nCounters;
  out->barrierEpochs = st.priv;
  out->llA2AEpochs = st.priv + nBar;
  out->abortFlag = comm->abortFlagDev;
  int khz = 0;
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, comm->cudaDev);
  out->timeoutCycles = (unsigned long long)paramDevCommTimeoutMs() * (unsigned long long)std::max(khz, 1000000);
  if (wantProxy) {
    res = ginProxyCreate(comm->cudaDev, reqs->ginQueueDepth > 0 ? reqs->ginQueueDepth : 1024, &st.proxy, out);
    if (res != ncclSuccess) { cudaFree(st.priv); ncclCommWindowDeregister(comm, st.win); ncclMemFree(st.buf); return res; }
    INFO(SUB_INIT, "device communicator: put / signal run through the host proxy thread (%u descriptors)", out->ginProxyMask + 1);
  }
  {
    std::lock_guard<std::mutex> g(gDevLock);
    gDevComms[{comm, st.priv}] = st;
  }
  if (cur != comm->cudaDev) cudaSetDevice(cur);
  INFO(SUB_INIT, "device communicator: %zu bytes of resource window, %d barriers, %d x %d low-latency slots", bytes, nBar, llBlocks, llSlots);
  return ncclSuccess;
}

ncclResult_t ncclDevCommDestroy(ncclComm_t comm, const ncclDevComm_t* devComm) {
  if (!commValid(comm) || !devComm) return ncclInvalidArgument;
  DevCommState st;
  {
    std::lock_guard<std::mutex> g(gDevLock);
    auto it = gDevComms.find({comm, devComm->barrierEpochs});
    if (it == gDevComms.end()) { WARN("ncclDevCommDestroy : not a device communicator of this communicator"); return ncclInvalidArgument; }
    st = it->second;
    gDevComms.erase(it);
  }
  cudaDeviceSynchronize();
  ginProxyDestroy(st.proxy);
  ncclResult_t r = ncclCommWindowDeregister(comm, st.win);
  cudaFree(st.priv);
  ncclMemFree(st.buf);
  return r;
}

ncclResult_t ncclGetLsaDevicePointer(ncclWindow_t win, size_t offset, int peer, void** outPtr) {
  if (!win || !outPtr || win->magic != kWindowMagic) return ncclInvalidArgument;
  if (peer < 0 || peer >= win->nRanks || peer >= NCCL_DEVICE_MAX_LSA || offset > win->size) return ncclInvalidArgument;
  if (!win->peerPtr[peer]) { *outPtr = nullptr; return ncclInvalidUsage; }
  *outPtr = (char*)win->peerPtr[peer] + offset;
  return ncclSuccess;
}

ncclResult_t ncclGetLsaMultimemDevicePointer(ncclWindow_t win, size_t offset, void** outPtr) {
  if (!win || !outPtr || win->magic != kWindowMagic || offset > win->size) return ncclInvalidArgument;
  *outPtr = win->mcPtr ? (char*)win->mcPtr + offset : nullptr;
  return ncclSuccess;
}

// World ranks and load/store ranks coincide: every rank of a device communicator is in one load/store team.
ncclResult_t ncclGetPeerDevicePointer(ncclWindow_t win, size_t offset, int peer, void** outPtr) { return ncclGetLsaDevicePointer(win, offset, peer, outPtr); }

ncclResult_t ncclWinGetDeviceHandle(ncclWindow_t win, ncclWindow_t* devHandle) {
  if (!win || !devHandle || win->magic != kWindowMagic) return ncclInvalidArgument;
  *devHandle = win->devSelf;
  return ncclSuccess;
}

}  // extern "C"
