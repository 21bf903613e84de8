// Communicator lifecycle: creation (blocking or in a background thread), split / shrink / grow,
// finalize / destroy / abort / revoke, queries and error strings.
// Reference parity: src/init.cc (ncclGetUniqueId :183-196, ncclCommInitRankDev :2477-2559,
// initTransportsRank :965-1720, config parsing :1977-2470, ncclCommSplit :3392, ncclCommShrink :3177,
// ncclCommGrow :3224, ncclCommRevoke :2933-3022, ncclCommAbort :3025, error/query API :3415-3512).
#include <unistd.h>

#include <algorithm>
#include <set>

#include "../core/cudawrap.h"
#include "../plugin/plugin.h"
#include "../plugin/profiler.h"
#include "../ras/ras.h"
#include "../topo/topo.h"
#include "device_plane.h"

using namespace b200;

namespace b200 {
void hostStagedRelease(ncclComm* comm);   // contrib/host_staged.cc
void m2nCommRelease(ncclComm* comm);      // contrib/m2n.cc

B200_PARAM(CommBlocking, "COMM_BLOCKING", -1, "Override ncclConfig_t::blocking (-1 = keep the program's value)")
B200_PARAM(CheckMode, "CHECK_MODE", 1, "Argument checking: 0 none, 1 local, 2 local + cross-rank")
B200_PARAM(HostOnly, "B200_HOST_ONLY", 0, "Create host-memory communicators even when a GPU is present")
extern int64_t paramP2pDisable();
extern int64_t paramRasEnable();

const char* funcName(int f) {
  static const char* n[] = {"Broadcast", "Reduce", "AllGather", "ReduceScatter", "AllReduce", "SendRecv", "Send", "Recv",
                            "AlltoAll", "Scatter", "Gather", "AllGatherV", "PutSignal", "Signal", "WaitSignal"};
  return f >= 0 && f < FUNC_COUNT ? n[f] : "?";
}
const char* algoName(int a) {
  static const char* n[] = {"OneRank", "LL", "P2P", "NVLS", "Ring", "Tree", "CE", "Host"};
  return a >= 0 && a < ALGO_COUNT ? n[a] : "Auto";
}

static std::mutex gInitLock;
static bool gInitDone = false;
static ncclResult_t libInit() {
  std::lock_guard<std::mutex> g(gInitLock);
  if (gInitDone) return ncclSuccess;
  loadConfFiles();
  if (debugLevel() >= LOG_VERSION) {
    INFO(SUB_ALL, "NCCL version %d.%d.%d%s (B200-native implementation)", NCCL_MAJOR, NCCL_MINOR, NCCL_PATCH, NCCL_SUFFIX);
  }
  NCCLCHECK(bootstrapNetInit());
  gInitDone = true;
  return ncclSuccess;
}

static void applyConfig(ncclComm* comm, const ncclConfig_t* user) {
  ncclConfig_t def = NCCL_CONFIG_INITIALIZER;
  comm->config = def;
  if (user) {
    // Older programs pass a shorter struct: copy what they have, keep "undefined" for the rest.
    size_t n = std::min(user->size, sizeof(ncclConfig_t));
    memcpy(&comm->config, user, n);
    comm->config.size = sizeof(ncclConfig_t);
  }
  ncclConfig_t& c = comm->config;
  if (c.blocking == NCCL_CONFIG_UNDEF_INT) c.blocking = 1;
  if (paramCommBlocking() >= 0) c.blocking = (int)paramCommBlocking();
  if (c.cgaClusterSize == NCCL_CONFIG_UNDEF_INT) c.cgaClusterSize = 0;
  if (c.splitShare == NCCL_CONFIG_UNDEF_INT) c.splitShare = 0;
  if (c.shrinkShare == NCCL_CONFIG_UNDEF_INT) c.shrinkShare = 0;
  if (c.CTAPolicy == NCCL_CONFIG_UNDEF_INT) c.CTAPolicy = NCCL_CTA_POLICY_DEFAULT;
  if (c.commName) comm->name = c.commName;
}

static ncclResult_t checkConfig(const ncclConfig_t* c) {
  if (!c) return ncclSuccess;
  if (c->magic != NCCL_API_MAGIC) { WARN("ncclConfig_t was not initialised with NCCL_CONFIG_INITIALIZER"); return ncclInvalidArgument; }
  if (c->size < offsetof(ncclConfig_t, cgaClusterSize)) { WARN("ncclConfig_t: size %zu is too small", c->size); return ncclInvalidArgument; }
  if (c->blocking != NCCL_CONFIG_UNDEF_INT && c->blocking != 0 && c->blocking != 1) { WARN("ncclConfig_t: blocking must be 0 or 1"); return ncclInvalidArgument; }
  if (c->size > offsetof(ncclConfig_t, minCTAs) && c->minCTAs != NCCL_CONFIG_UNDEF_INT && c->minCTAs <= 0) { WARN("ncclConfig_t: minCTAs must be positive"); return ncclInvalidArgument; }
  if (c->size > offsetof(ncclConfig_t, maxCTAs) && c->maxCTAs != NCCL_CONFIG_UNDEF_INT && c->maxCTAs <= 0) { WARN("ncclConfig_t: maxCTAs must be positive"); return ncclInvalidArgument; }
  if (c->size > offsetof(ncclConfig_t, maxCTAs) && c->minCTAs != NCCL_CONFIG_UNDEF_INT && c->maxCTAs != NCCL_CONFIG_UNDEF_INT && c->minCTAs > c->maxCTAs) {
    WARN("ncclConfig_t: minCTAs %d exceeds maxCTAs %d", c->minCTAs, c->maxCTAs);
    return ncclInvalidArgument;
  }
  return ncclSuccess;
}

static void fillPeerInfo(ncclComm* comm, PeerInfo* pi) {
  memset(pi, 0, sizeof(*pi));
  pi->rank = comm->rank;
  pi->cudaDev = comm->cudaDev;
  pi->nvmlDev = comm->nvmlDev;
  pi->hostHash = hostHash();
  pi->pidHash = pidHash();
  pi->version = NCCL_VERSION_CODE;
  pi->hostOnly = comm->hostOnly;
  if (!comm->hostOnly) {
    char busId[32] = "";
    if (cudaDeviceGetPCIBusId(busId, sizeof(busId), comm->cudaDev) == cudaSuccess) pi->busId = busIdToInt64(busId);
    else (void)cudaGetLastError();
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, comm->cudaDev) == cudaSuccess) {
      pi->cudaCompCap = prop.major * 10 + prop.minor;
      pi->totalMem = prop.totalGlobalMem;
    }
    pi->vmmSupport = cuMemSupported(comm->cudaDev);
    pi->mcSupport = cuMulticastSupported(comm->cudaDev);
    fabricInfoQuery(busId[0] ? busId : nullptr, &pi->fabric);
  }
}

// Everything after the bootstrap ring exists: peer table, node layout, data planes.
static ncclResult_t commSetup(ncclComm* comm) {
  const int n = comm->nRanks;
  comm->peers.resize(n);
  fillPeerInfo(comm, &comm->peers[comm->rank]);
  NCCLCHECK(bootstrapAllGather(comm->bootstrap, comm->peers.data(), sizeof(PeerInfo)));
  bool mixed = false, anyHost = false;
  for (auto& p : comm->peers) {
    if (p.version != NCCL_VERSION_CODE) {
      WARN("rank %d runs library version %d, rank %d runs %d: all ranks must use the same library", p.rank, p.version, comm->rank, NCCL_VERSION_CODE);
      return ncclInvalidUsage;
    }
    anyHost = anyHost || p.hostOnly;
    mixed = mixed || (p.hostOnly != comm->hostOnly);
  }
  if (mixed) { WARN("some ranks have a GPU and some do not: all ranks must be of one kind"); return ncclInvalidUsage; }
  // node layout
  std::vector<uint64_t> hosts;
  for (auto& p : comm->peers) if (std::find(hosts.begin(), hosts.end(), p.hostHash) == hosts.end()) hosts.push_back(p.hostHash);
  comm->nNodes = (int)hosts.size();
  comm->node = (int)(std::find(hosts.begin(), hosts.end(), comm->peers[comm->rank].hostHash) - hosts.begin());
  comm->localRanks = 0;
  for (auto& p : comm->peers) {
    if (p.hostHash != comm->peers[comm->rank].hostHash) continue;
    if (p.rank == comm->rank) comm->localRank = comm->localRanks;
    comm->localRanks++;
  }
  uint64_t h = bootstrapMagic(comm->bootstrap);
  comm->commHash = hashCombine(h, (uint64_t)n);
  if (!comm->hostOnly) {
    for (auto& p : comm->peers) {
      if (p.rank != comm->rank && p.hostHash == comm->peers[comm->rank].hostHash && p.busId == comm->peers[comm->rank].busId) {
        WARN("Duplicate GPU detected : rank %d and rank %d both on CUDA device %lx", comm->rank, p.rank, (long)p.busId);
        return ncclInvalidUsage;
      }
    }
    comm->compCap = comm->peers[comm->rank].cudaCompCap;
    NCCLCHECK(mnnvlCheck(comm));
    const bool oneDomain = comm->nNodes == 1 || (comm->mnnvl && (int)comm->clique.ranks.size() == n);
    comm->lsaAll = oneDomain && n <= kMaxRanks && !paramP2pDisable();
    NCCLCHECK(topoInit(comm));   // topology detection + graphs (feeds the model, the dumps and fallbacks)
  }
  if (comm->hostOnly) {
    if (n > 1) NCCLCHECK(hostPlaneCreate(comm));
  } else {
    NCCLCHECK(devPlaneCreate(comm));
  }
  NCCLCHECK(tunerLoad(comm));
  profilerCommInit(comm);
  if (paramRasEnable()) rasCommAdd(comm);
  checkpointCommAdd(comm);
  INFO(SUB_INIT, "comm %p rank %d nranks %d cudaDev %d nodes %d localRanks %d %s - Init COMPLETE", (void*)comm, comm->rank, n, comm->cudaDev,
       comm->nNodes, comm->localRanks, comm->hostOnly ? "(host memory)" : (comm->lsaAll ? "(symmetric data plane)" : "(socket fallback)"));
  return ncclSuccess;
}

static ncclResult_t allocFlags(ncclComm* comm) {
  if (comm->hostOnly) {
    comm->abortFlag = new uint32_t[8]();
    comm->devStatus = comm->abortFlag + 4;
    return ncclSuccess;
  }
  uint32_t* host = nullptr;
  CUDACHECK(cudaHostAlloc((void**)&host, 8 * sizeof(uint32_t), cudaHostAllocMapped));
  memset(host, 0, 8 * sizeof(uint32_t));
  uint32_t* dev = nullptr;
  CUDACHECK(cudaHostGetDevicePointer((void**)&dev, host, 0));
  comm->abortFlag = host;
  comm->abortFlagDev = dev;
  comm->devStatus = host + 4;
  comm->devStatusDev = dev + 4;
  return ncclSuccess;
}

static void freeComm(ncclComm* comm) {
  if (!comm) return;
  if (comm->initThread) { if (comm->initThread->joinable()) comm->initThread->join(); delete comm->initThread; }
  rasCommRemove(comm);
  checkpointCommRemove(comm);
  proxyQuiesce(comm);   // its events belong to the profiler that goes next
  profilerCommFini(comm);
  tunerUnload(comm);
  hostStagedRelease(comm);
  m2nCommRelease(comm);
  if (comm->devPlane) {
    int cur = -1;
    cudaGetDevice(&cur);
    if (comm->cudaDev >= 0 && cur != comm->cudaDev) cudaSetDevice(comm->cudaDev);
    devPlaneDestroy(comm);
    if (cur >= 0 && cur != comm->cudaDev) cudaSetDevice(cur);
  }
  hostPlaneDestroy(comm);
  topoDestroy(comm);
  if (comm->bootstrap) bootstrapClose(comm->bootstrap);
  if (comm->hostOnly) delete[] comm->abortFlag;
  else if (comm->abortFlag) cudaFreeHost((void*)comm->abortFlag);
  (void)cudaGetLastError();
  comm->startMagic = comm->endMagic = 0;
  delete comm;
}

struct InitArgs {
  int nranks, rank, nIds;
  std::vector<ncclUniqueId> ids;
  ncclComm* parent = nullptr;       // split/shrink
  std::vector<int> parentRanks;
  uint64_t splitMagic = 0;
};

static ncclResult_t initBody(ncclComm* comm, InitArgs ia) {
  ncclResult_t res = ncclSuccess;
  if (!comm->hostOnly) CUDACHECKGOTO(cudaSetDevice(comm->cudaDev), res, fail);
  NCCLCHECKGOTO(allocFlags(comm), res, fail);
  if (ia.parent) {
    NCCLCHECKGOTO(bootstrapSplit(ia.splitMagic, ia.parent->bootstrap, ia.rank, ia.nranks, ia.parentRanks.data(), comm->abortFlag, &comm->bootstrap), res, fail);
  } else {
    BootstrapInitArgs ba;
    ba.cudaDev = comm->cudaDev;
    ba.nvmlDev = comm->nvmlDev;
    ba.abortFlag = comm->abortFlag;
    NCCLCHECKGOTO(bootstrapInit(ia.nIds, ia.ids.data(), ia.rank, ia.nranks, ba, &comm->bootstrap), res, fail);
  }
  NCCLCHECKGOTO(commSetup(comm), res, fail);
  comm->asyncResult = ncclSuccess;
  return ncclSuccess;
fail:
  comm->asyncResult = res;
  return res;
}

static ncclResult_t commCreate(ncclComm** out, const InitArgs& ia, const ncclConfig_t* config) {
  NCCLCHECK(libInit());
  NCCLCHECK(checkConfig(config));
  if (ia.nranks < 1 || ia.rank < 0 || ia.rank >= ia.nranks) { WARN("Invalid rank requested : %d/%d", ia.rank, ia.nranks); return ncclInvalidArgument; }
  ncclComm* comm = new ncclComm;
  comm->rank = ia.rank;
  comm->nRanks = ia.nranks;
  comm->parent = nullptr;
  applyConfig(comm, config ? config : (ia.parent ? &ia.parent->config : nullptr));
  int ndev = 0;
  if (paramHostOnly() || cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    (void)cudaGetLastError();
    comm->hostOnly = true;
    comm->cudaDev = -1;
  } else {
    if (cudaGetDevice(&comm->cudaDev) != cudaSuccess) { (void)cudaGetLastError(); delete comm; return ncclUnhandledCudaError; }
    comm->nvmlDev = comm->cudaDev;
  }
  *out = comm;
  if (comm->config.blocking) {
    ncclResult_t r = initBody(comm, ia);
    if (r != ncclSuccess) { *out = nullptr; freeComm(comm); }
    return r;
  }
  comm->asyncResult = ncclInProgress;
  comm->initThread = new std::thread([comm, ia] { setThreadName("b200 Init"); initBody(comm, ia); });
  return ncclInProgress;
}

ncclResult_t commEnsureReady(ncclComm* c) {
  if (!commValid(c)) { WARN("invalid communicator handle"); return ncclInvalidArgument; }
  int r = c->asyncResult.load();
  if (r == ncclInProgress) return ncclInProgress;
  if (r != ncclSuccess) return (ncclResult_t)r;
  if (c->revoked) { WARN("communicator was revoked"); return ncclInvalidUsage; }
  if (flagSet(c->abortFlag)) return ncclInternalError;
  return ncclSuccess;
}

}  // namespace b200

// ====================================================================================== C API
extern "C" {

ncclResult_t ncclGetVersion(int* version) {
  if (!version) return ncclInvalidArgument;
  *version = NCCL_VERSION_CODE;
  return ncclSuccess;
}

ncclResult_t ncclGetUniqueId(ncclUniqueId* out) {
  NCCLCHECK(libInit());
  if (!out) return ncclInvalidArgument;
  memset(out, 0, sizeof(*out));
  BootstrapHandle h;
  NCCLCHECK(bootstrapGetUniqueId(&h));
  memcpy(out->internal, &h, sizeof(h));
  return ncclSuccess;
}

static ncclResult_t initRankCommon(ncclComm_t* newcomm, int nranks, int myrank, int nId, ncclUniqueId* ids, ncclConfig_t* config) {
  if (!newcomm || !ids || nId < 1 || nId > nranks) { WARN("invalid arguments to communicator creation"); return ncclInvalidArgument; }
  *newcomm = nullptr;
  InitArgs ia;
  ia.nranks = nranks;
  ia.rank = myrank;
  ia.nIds = nId;
  ia.ids.assign(ids, ids + nId);
  // With NCCL_COMM_ID every process derives the id from the environment; rank 0 serves as root.
  const char* env = getEnv("NCCL_COMM_ID");
  if (env && *env && myrank == 0) {
    BootstrapHandle h;
    memcpy(&h, ids[0].internal, sizeof(h));
    NCCLCHECK(libInit());
    NCCLCHECK(bootstrapCreateRoot(&h, true));
  }
  ncclComm* c = nullptr;
  ncclResult_t r = commCreate(&c, ia, config);
  *newcomm = c;
  return r;
}

ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank, ncclConfig_t* config) {
  return groupRunOrDefer([=]() mutable { return initRankCommon(comm, nranks, rank, 1, &commId, config); });
}
ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank) {
  return groupRunOrDefer([=]() mutable { return initRankCommon(comm, nranks, rank, 1, &commId, nullptr); });
}
ncclResult_t ncclCommInitRankScalable(ncclComm_t* newcomm, int nranks, int myrank, int nId, ncclUniqueId* commIds, ncclConfig_t* config) {
  std::vector<ncclUniqueId> ids(commIds, commIds + (nId > 0 ? nId : 0));
  return groupRunOrDefer([=]() mutable { return initRankCommon(newcomm, nranks, myrank, nId, ids.data(), config); });
}

ncclResult_t ncclCommInitAll(ncclComm_t* comms, int ndev, const int* devlist) {
  NCCLCHECK(libInit());
  if (!comms || ndev < 1) { WARN("ncclCommInitAll: invalid arguments"); return ncclInvalidArgument; }
  int total = 0;
  if (cudaGetDeviceCount(&total) != cudaSuccess) { (void)cudaGetLastError(); total = 0; }
  std::vector<int> devs(ndev);
  std::set<int> seen;
  for (int i = 0; i < ndev; ++i) {
    devs[i] = devlist ? devlist[i] : i;
    if (total && (devs[i] < 0 || devs[i] >= total)) { WARN("ncclCommInitAll: invalid device %d", devs[i]); return ncclInvalidArgument; }
    if (!seen.insert(devs[i]).second) { WARN("ncclCommInitAll: device %d listed twice", devs[i]); return ncclInvalidUsage; }
  }
  ncclUniqueId id;
  NCCLCHECK(ncclGetUniqueId(&id));
  int saved = -1;
  cudaGetDevice(&saved);
  (void)cudaGetLastError();
  std::vector<std::thread> th;
  std::vector<ncclResult_t> res(ndev, ncclSuccess);
  for (int i = 0; i < ndev; ++i) {
    th.emplace_back([&, i] {
      if (total) cudaSetDevice(devs[i]);
      res[i] = initRankCommon(&comms[i], ndev, i, 1, &id, nullptr);
    });
  }
  for (auto& t : th) t.join();
  if (saved >= 0) cudaSetDevice(saved);
  for (int i = 0; i < ndev; ++i) if (res[i] != ncclSuccess) return res[i];
  return ncclSuccess;
}

ncclResult_t ncclCommFinalize(ncclComm_t comm) {
  if (!commValid(comm)) return ncclInvalidArgument;
  if (comm->revoked) { WARN("ncclCommFinalize after ncclCommRevoke is invalid"); return ncclInvalidUsage; }
  if (comm->initThread && comm->initThread->joinable()) comm->initThread->join();
  if (!comm->hostOnly && comm->devPlane) {
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != comm->cudaDev) cudaSetDevice(comm->cudaDev);
    cudaError_t e = cudaDeviceSynchronize();   // every enqueued collective has completed
    if (cur >= 0 && cur != comm->cudaDev) cudaSetDevice(cur);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return ncclUnhandledCudaError; }
    NCCLCHECK(devPlaneCheckStatus(comm));
  }
  comm->finalized = true;
  return ncclSuccess;
}

ncclResult_t ncclCommDestroy(ncclComm_t comm) {
  if (comm == nullptr) return ncclSuccess;
  if (!commValid(comm)) { WARN("ncclCommDestroy: invalid communicator"); return ncclInvalidArgument; }
  if (!comm->finalized && !comm->revoked && comm->asyncResult.load() == ncclSuccess) {
    ncclResult_t r = ncclCommFinalize(comm);
    if (r != ncclSuccess) INFO(SUB_INIT, "finalize during destroy returned %d", (int)r);
  }
  INFO(SUB_INIT, "comm %p rank %d nranks %d - Destroy COMPLETE", (void*)comm, comm->rank, comm->nRanks);
  freeComm(comm);
  return ncclSuccess;
}

ncclResult_t ncclCommAbort(ncclComm_t comm) {
  if (comm == nullptr) return ncclSuccess;
  if (!commValid(comm)) return ncclInvalidArgument;
  if (comm->abortFlag) __atomic_store_n((uint32_t*)comm->abortFlag, 1u, __ATOMIC_SEQ_CST);
  if (comm->initThread && comm->initThread->joinable()) comm->initThread->join();
  // A thread blocked inside a call on this communicator leaves it once it sees the flag; its objects must outlive it.
  for (int ms = 0; comm->launchOwner.load(std::memory_order_acquire) != 0 && ms < 30000; ++ms) std::this_thread::sleep_for(std::chrono::milliseconds(1));
  if (comm->launchOwner.load(std::memory_order_acquire) != 0) WARN("ncclCommAbort: another thread is still inside a call on communicator %p after 30 s", (void*)comm);
  if (!comm->hostOnly && comm->devPlane) {
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != comm->cudaDev) cudaSetDevice(comm->cudaDev);
    ceCollRelease(comm);       // stream waits of the copy-engine collectives do not see the flag: release them
    cudaDeviceSynchronize();   // kernels leave their waits once they see the flag
    (void)cudaGetLastError();
    if (cur >= 0 && cur != comm->cudaDev) cudaSetDevice(cur);
  }
  INFO(SUB_INIT, "comm %p rank %d nranks %d - Abort COMPLETE", (void*)comm, comm->rank, comm->nRanks);
  freeComm(comm);
  return ncclSuccess;
}

ncclResult_t ncclCommRevoke(ncclComm_t comm, int revokeFlags) {
  if (!commValid(comm)) return ncclInvalidArgument;
  if (revokeFlags != NCCL_REVOKE_DEFAULT) { WARN("ncclCommRevoke: flags must be NCCL_REVOKE_DEFAULT"); return ncclInvalidArgument; }
  // Stop what is in flight, keep the object: shrink/split/destroy stay legal afterwards.
  if (comm->abortFlag) __atomic_store_n((uint32_t*)comm->abortFlag, 1u, __ATOMIC_SEQ_CST);
  if (!comm->hostOnly && comm->devPlane) {
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != comm->cudaDev) cudaSetDevice(comm->cudaDev);
    ceCollRelease(comm);
    cudaDeviceSynchronize();
    (void)cudaGetLastError();
    if (cur >= 0 && cur != comm->cudaDev) cudaSetDevice(cur);
  }
  comm->revoked = true;
  // quiescent: the control plane may be used again (bootstrap sockets poll the same flag)
  if (comm->abortFlag) __atomic_store_n((uint32_t*)comm->abortFlag, 0u, __ATOMIC_SEQ_CST);
  return ncclSuccess;
}

static ncclResult_t childCreate(ncclComm* parent, const std::vector<int>& members, int newRank, ncclComm_t* newcomm, ncclConfig_t* config,
                                uint64_t salt) {
  InitArgs ia;
  ia.nranks = (int)members.size();
  ia.rank = newRank;
  ia.nIds = 0;
  ia.parent = parent;
  ia.parentRanks = members;
  ia.splitMagic = hashCombine(hashCombine(bootstrapMagic(parent->bootstrap), (uint64_t)parent->childCount), salt);
  ncclComm* c = nullptr;
  int cur = -1;
  if (!parent->hostOnly) { cudaGetDevice(&cur); if (cur != parent->cudaDev) cudaSetDevice(parent->cudaDev); }
  ncclResult_t r = commCreate(&c, ia, config);
  if (cur >= 0 && cur != parent->cudaDev) cudaSetDevice(cur);
  *newcomm = c;
  return r;
}

ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, ncclConfig_t* config) {
  if (!newcomm) return ncclInvalidArgument;
  *newcomm = nullptr;
  if (!commValid(comm)) return ncclInvalidArgument;
  int st = comm->asyncResult.load();
  if (st != ncclSuccess) return (ncclResult_t)st;
  if (color < 0 && color != NCCL_SPLIT_NOCOLOR) { WARN("ncclCommSplit: invalid color %d", color); return ncclInvalidArgument; }
  return groupRunOrDefer([=]() -> ncclResult_t {
    const int n = comm->nRanks;
    std::vector<int> ck(2 * n);
    ck[2 * comm->rank] = color;
    ck[2 * comm->rank + 1] = key;
    NCCLCHECK(bootstrapAllGather(comm->bootstrap, ck.data(), 2 * sizeof(int)));
    comm->childCount++;
    if (color == NCCL_SPLIT_NOCOLOR) return ncclSuccess;
    std::vector<std::pair<int, int>> mem;  // (key, parent rank)
    for (int r = 0; r < n; ++r) if (ck[2 * r] == color) mem.push_back({ck[2 * r + 1], r});
    std::stable_sort(mem.begin(), mem.end());
    std::vector<int> members;
    int newRank = -1;
    for (auto& m : mem) { if (m.second == comm->rank) newRank = (int)members.size(); members.push_back(m.second); }
    return childCreate(comm, members, newRank, newcomm, config, (uint64_t)color + 1);
  });
}

ncclResult_t ncclCommShrink(ncclComm_t comm, int* excludeRanksList, int excludeRanksCount, ncclComm_t* newcomm, ncclConfig_t* config, int shrinkFlags) {
  if (!newcomm) return ncclInvalidArgument;
  *newcomm = nullptr;
  if (!commValid(comm)) return ncclInvalidArgument;
  if (excludeRanksCount <= 0 || !excludeRanksList || excludeRanksCount >= comm->nRanks) { WARN("ncclCommShrink: invalid exclude list"); return ncclInvalidArgument; }
  std::set<int> ex(excludeRanksList, excludeRanksList + excludeRanksCount);
  for (int r : ex) if (r < 0 || r >= comm->nRanks) { WARN("ncclCommShrink: rank %d out of range", r); return ncclInvalidArgument; }
  if (ex.count(comm->rank)) { WARN("ncclCommShrink: an excluded rank must not call"); return ncclInvalidArgument; }
  if (shrinkFlags & NCCL_SHRINK_ABORT) {
    // peers may be gone: stop what is in flight on the parent first
    if (comm->abortFlag) __atomic_store_n((uint32_t*)comm->abortFlag, 1u, __ATOMIC_SEQ_CST);
    if (!comm->hostOnly) { cudaDeviceSynchronize(); (void)cudaGetLastError(); }
    if (comm->abortFlag) __atomic_store_n((uint32_t*)comm->abortFlag, 0u, __ATOMIC_SEQ_CST);
  }
  std::vector<int> members;
  int newRank = -1;
  for (int r = 0; r < comm->nRanks; ++r) {
    if (ex.count(r)) continue;
    if (r == comm->rank) newRank = (int)members.size();
    members.push_back(r);
  }
  comm->childCount++;
  // survivors derive the member list locally: nothing is sent to excluded (possibly dead) ranks
  return childCreate(comm, members, newRank, newcomm, config, 0x5348524eull);
}

ncclResult_t ncclCommGetUniqueId(ncclComm_t comm, ncclUniqueId* uniqueId) {
  if (!commValid(comm) || !uniqueId) return ncclInvalidArgument;
  return ncclGetUniqueId(uniqueId);
}

ncclResult_t ncclCommGrow(ncclComm_t comm, int nRanks, const ncclUniqueId* uniqueId, int rank, ncclComm_t* newcomm, ncclConfig_t* config) {
  if (!newcomm) return ncclInvalidArgument;
  *newcomm = nullptr;
  ncclUniqueId id;
  int myRank = rank;
  if (comm) {
    // existing member: keeps its rank; the root (the member that holds the id) shares it with the others
    if (!commValid(comm)) return ncclInvalidArgument;
    if (nRanks <= comm->nRanks) { WARN("ncclCommGrow: new size %d must exceed the current size %d", nRanks, comm->nRanks); return ncclInvalidArgument; }
    myRank = comm->rank;
    std::vector<char> gathered((size_t)comm->nRanks * (sizeof(ncclUniqueId) + sizeof(int)), 0);
    char* mine = gathered.data() + (size_t)comm->rank * (sizeof(ncclUniqueId) + sizeof(int));
    int have = uniqueId ? 1 : 0;
    memcpy(mine, &have, sizeof(int));
    if (uniqueId) memcpy(mine + sizeof(int), uniqueId, sizeof(ncclUniqueId));
    NCCLCHECK(bootstrapAllGather(comm->bootstrap, gathered.data(), (int)(sizeof(ncclUniqueId) + sizeof(int))));
    bool found = false;
    for (int r = 0; r < comm->nRanks && !found; ++r) {
      char* slot = gathered.data() + (size_t)r * (sizeof(ncclUniqueId) + sizeof(int));
      int h;
      memcpy(&h, slot, sizeof(int));
      if (h) { memcpy(&id, slot + sizeof(int), sizeof(ncclUniqueId)); found = true; }
    }
    if (!found) { WARN("ncclCommGrow: no existing rank supplied the unique id"); return ncclInvalidArgument; }
  } else {
    if (!uniqueId || rank < 0) { WARN("ncclCommGrow: a new rank needs the unique id and its rank"); return ncclInvalidArgument; }
    id = *uniqueId;
  }
  return initRankCommon(newcomm, nRanks, myRank, 1, &id, config ? config : (comm ? &comm->config : nullptr));
}

const char* ncclGetErrorString(ncclResult_t code) {
  switch (code) {
    case ncclSuccess: return "no error";
    case ncclUnhandledCudaError: return "unhandled cuda error (run with NCCL_DEBUG=INFO for details)";
    case ncclSystemError: return "unhandled system error (run with NCCL_DEBUG=INFO for details)";
    case ncclInternalError: return "internal error - please report this issue to the NCCL developers";
    case ncclInvalidArgument: return "invalid argument (run with NCCL_DEBUG=WARN for details)";
    case ncclInvalidUsage: return "invalid usage (run with NCCL_DEBUG=WARN for details)";
    case ncclRemoteError: return "remote process exited or there was a network error";
    case ncclInProgress: return "NCCL operation in progress";
    case ncclTimeout: return "operation timed out";
    default: return "unknown result code";
  }
}

const char* ncclGetLastError(ncclComm_t) { return lastErrorString(); }

ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* asyncError) {
  if (!commValid(comm) || !asyncError) return ncclInvalidArgument;
  int st = comm->asyncResult.load();
  if (st == ncclSuccess && !comm->hostOnly && comm->devPlane) {
    ncclResult_t d = devPlaneCheckStatus(comm);
    if (d != ncclSuccess) { comm->asyncResult = d; st = d; }
  }
  *asyncError = (ncclResult_t)st;
  return ncclSuccess;
}

ncclResult_t ncclCommCount(const ncclComm_t comm, int* count) {
  if (!commValid(comm) || !count) return ncclInvalidArgument;
  *count = comm->nRanks;
  return ncclSuccess;
}
ncclResult_t ncclCommCuDevice(const ncclComm_t comm, int* device) {
  if (!commValid(comm) || !device) return ncclInvalidArgument;
  *device = comm->cudaDev;
  return ncclSuccess;
}
ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank) {
  if (!commValid(comm) || !rank) return ncclInvalidArgument;
  *rank = comm->rank;
  return ncclSuccess;
}

ncclResult_t ncclRedOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t datatype, ncclScalarResidence_t residence, ncclComm_t comm) {
  if (!commValid(comm) || !op || !scalar) return ncclInvalidArgument;
  if ((int)datatype < 0 || datatype >= ncclNumTypes) return ncclInvalidArgument;
  std::lock_guard<std::mutex> g(comm->lock);
  size_t idx = 0;
  for (; idx < comm->userOps.size(); ++idx) if (!comm->userOps[idx].used) break;
  if (idx == comm->userOps.size()) comm->userOps.emplace_back();
  UserRedOp& u = comm->userOps[idx];
  u.used = true;
  u.type = datatype;
  u.residence = residence;
  u.scalarBits = 0;
  u.devScalar = nullptr;
  if (residence == ncclScalarHostImmediate) memcpy(&u.scalarBits, scalar, typeSize(datatype));
  else u.devScalar = scalar;
  *op = (ncclRedOp_t)(ncclNumOps + (int)idx);
  return ncclSuccess;
}

ncclResult_t ncclRedOpDestroy(ncclRedOp_t op, ncclComm_t comm) {
  if (!commValid(comm)) return ncclInvalidArgument;
  int idx = (int)op - ncclNumOps;
  std::lock_guard<std::mutex> g(comm->lock);
  if (idx < 0 || idx >= (int)comm->userOps.size() || !comm->userOps[idx].used) { WARN("ncclRedOpDestroy: operator %d was not created by ncclRedOpCreatePreMulSum", (int)op); return ncclInvalidArgument; }
  comm->userOps[idx].used = false;
  return ncclSuccess;
}

// profiling twins
ncclResult_t pncclGetVersion(int* v) { return ncclGetVersion(v); }
ncclResult_t pncclGetUniqueId(ncclUniqueId* u) { return ncclGetUniqueId(u); }
ncclResult_t pncclCommInitRankConfig(ncclComm_t* c, int n, ncclUniqueId id, int r, ncclConfig_t* cfg) { return ncclCommInitRankConfig(c, n, id, r, cfg); }
ncclResult_t pncclCommInitRank(ncclComm_t* c, int n, ncclUniqueId id, int r) { return ncclCommInitRank(c, n, id, r); }
ncclResult_t pncclCommInitAll(ncclComm_t* c, int n, const int* d) { return ncclCommInitAll(c, n, d); }
ncclResult_t pncclCommInitRankScalable(ncclComm_t* c, int n, int r, int k, ncclUniqueId* ids, ncclConfig_t* cfg) { return ncclCommInitRankScalable(c, n, r, k, ids, cfg); }
ncclResult_t pncclCommFinalize(ncclComm_t c) { return ncclCommFinalize(c); }
ncclResult_t pncclCommDestroy(ncclComm_t c) { return ncclCommDestroy(c); }
ncclResult_t pncclCommAbort(ncclComm_t c) { return ncclCommAbort(c); }
ncclResult_t pncclCommRevoke(ncclComm_t c, int f) { return ncclCommRevoke(c, f); }
ncclResult_t pncclCommSplit(ncclComm_t c, int col, int key, ncclComm_t* n, ncclConfig_t* cfg) { return ncclCommSplit(c, col, key, n, cfg); }
ncclResult_t pncclCommShrink(ncclComm_t c, int* l, int n, ncclComm_t* nc, ncclConfig_t* cfg, int f) { return ncclCommShrink(c, l, n, nc, cfg, f); }
ncclResult_t pncclCommGetUniqueId(ncclComm_t c, ncclUniqueId* u) { return ncclCommGetUniqueId(c, u); }
ncclResult_t pncclCommGrow(ncclComm_t c, int n, const ncclUniqueId* u, int r, ncclComm_t* nc, ncclConfig_t* cfg) { return ncclCommGrow(c, n, u, r, nc, cfg); }
const char* pncclGetErrorString(ncclResult_t r) { return ncclGetErrorString(r); }
const char* pncclGetLastError(ncclComm_t c) { return ncclGetLastError(c); }
ncclResult_t pncclCommGetAsyncError(ncclComm_t c, ncclResult_t* e) { return ncclCommGetAsyncError(c, e); }
ncclResult_t pncclCommCount(const ncclComm_t c, int* n) { return ncclCommCount(c, n); }
ncclResult_t pncclCommCuDevice(const ncclComm_t c, int* d) { return ncclCommCuDevice(c, d); }
ncclResult_t pncclCommUserRank(const ncclComm_t c, int* r) { return ncclCommUserRank(c, r); }
ncclResult_t pncclRedOpCreatePreMulSum(ncclRedOp_t* o, void* s, ncclDataType_t t, ncclScalarResidence_t r, ncclComm_t c) { return ncclRedOpCreatePreMulSum(o, s, t, r, c); }
ncclResult_t pncclRedOpDestroy(ncclRedOp_t o, ncclComm_t c) { return ncclRedOpDestroy(o, c); }

}  // extern "C"
