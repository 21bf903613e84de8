// Checkpoint support: see include/nccl_checkpoint.h.
#include "nccl_checkpoint.h"

#include <algorithm>
#include <mutex>

#include "../comm/comm.h"
#include "../comm/device_plane.h"
#include "../mem/symmetric.h"

using namespace b200;

struct ncclCheckpointState {
  struct Win { uint64_t ptr, size; int flags; };
  uint32_t version = 1;
  int nRanks = 0, rank = 0;
  int hostOnly = 0;
  ncclConfig_t config;
  char name[128] = "";
  std::vector<Win> windows;
};

// Live communicators of this process in creation order (init.cc adds and removes them), and the ones the
// process-wide prepare call suspended.
static std::mutex gCommsLock;
static std::vector<ncclComm*> gComms, gSuspended;

namespace b200 {
void checkpointCommAdd(ncclComm* comm) {
  std::lock_guard<std::mutex> g(gCommsLock);
  gComms.push_back(comm);
}
void checkpointCommRemove(ncclComm* comm) {
  std::lock_guard<std::mutex> g(gCommsLock);
  gComms.erase(std::remove(gComms.begin(), gComms.end(), comm), gComms.end());
  gSuspended.erase(std::remove(gSuspended.begin(), gSuspended.end(), comm), gSuspended.end());
}
}  // namespace b200

static constexpr uint64_t kCkptMagic = 0x434b50544232303ull;

extern "C" {

ncclResult_t ncclCommCheckpointPrepare(ncclComm_t comm, ncclCheckpoint_t* out) {
  if (!commValid(comm) || !out) return ncclInvalidArgument;
  NCCLCHECK(commEnsureReady(comm));
  if (comm->parent || comm->childCount) INFO(SUB_INIT, "ncclCommCheckpointPrepare: split relations are not recorded; re-split after the restore");
  ncclCheckpointState* st = new ncclCheckpointState;
  st->nRanks = comm->nRanks;
  st->rank = comm->rank;
  st->hostOnly = comm->hostOnly ? 1 : 0;
  st->config = comm->config;
  st->config.commName = nullptr;   // pointers do not survive; the name is kept as text
  st->config.netName = nullptr;
  snprintf(st->name, sizeof(st->name), "%s", comm->name.c_str());
  std::vector<SymWindow*> userWins;
  if (comm->sym) {
    std::lock_guard<std::mutex> g(comm->sym->lock);
    for (SymWindow* w : comm->sym->windows) {
      if (comm->devPlane && w == comm->devPlane->resWin) continue;   // the library's own window comes back with the communicator
      st->windows.push_back({(uint64_t)(uintptr_t)w->host.userPtr, (uint64_t)w->host.size, w->flags});
      userWins.push_back(w);
    }
  }
  if (!comm->hostOnly) {
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != comm->cudaDev) cudaSetDevice(comm->cudaDev);
    cudaDeviceSynchronize();
    if (cur >= 0 && cur != comm->cudaDev) cudaSetDevice(cur);
  }
  for (SymWindow* w : userWins) NCCLCHECK(ncclCommWindowDeregister(comm, &w->host));
  NCCLCHECK(ncclCommDestroy(comm));
  *out = st;
  return ncclSuccess;
}

ncclResult_t ncclCommCheckpointSave(ncclCheckpoint_t st, void* buf, size_t* bytes) {
  if (!st || !bytes) return ncclInvalidArgument;
  const size_t need = 8 + 4 + 4 * 3 + sizeof(ncclConfig_t) + sizeof(st->name) + 4 + st->windows.size() * sizeof(ncclCheckpointState::Win);
  if (!buf || *bytes < need) { bool query = !buf; *bytes = need; return query ? ncclSuccess : ncclInvalidArgument; }
  char* p = (char*)buf;
  auto put = [&](const void* src, size_t n) { memcpy(p, src, n); p += n; };
  put(&kCkptMagic, 8);
  put(&st->version, 4);
  put(&st->nRanks, 4);
  put(&st->rank, 4);
  put(&st->hostOnly, 4);
  put(&st->config, sizeof(ncclConfig_t));
  put(st->name, sizeof(st->name));
  uint32_t nw = (uint32_t)st->windows.size();
  put(&nw, 4);
  if (nw) put(st->windows.data(), nw * sizeof(ncclCheckpointState::Win));
  *bytes = need;
  return ncclSuccess;
}

ncclResult_t ncclCommCheckpointLoad(const void* buf, size_t bytes, ncclCheckpoint_t* out) {
  if (!buf || !out || bytes < 8 + 4 + 12 + sizeof(ncclConfig_t) + 128 + 4) return ncclInvalidArgument;
  const char* p = (const char*)buf;
  auto get = [&](void* dst, size_t n) { memcpy(dst, p, n); p += n; };
  uint64_t magic;
  get(&magic, 8);
  if (magic != kCkptMagic) { WARN("ncclCommCheckpointLoad: not a checkpoint record"); return ncclInvalidArgument; }
  ncclCheckpointState* st = new ncclCheckpointState;
  get(&st->version, 4);
  get(&st->nRanks, 4);
  get(&st->rank, 4);
  get(&st->hostOnly, 4);
  get(&st->config, sizeof(ncclConfig_t));
  get(st->name, sizeof(st->name));
  uint32_t nw;
  get(&nw, 4);
  if (st->version != 1 || (size_t)(p - (const char*)buf) + (size_t)nw * sizeof(ncclCheckpointState::Win) > bytes) { delete st; return ncclInvalidArgument; }
  st->windows.resize(nw);
  if (nw) get(st->windows.data(), nw * sizeof(ncclCheckpointState::Win));
  st->config.commName = nullptr;
  st->config.netName = nullptr;
  *out = st;
  return ncclSuccess;
}

ncclResult_t ncclCommCheckpointRestore(ncclCheckpoint_t st, ncclUniqueId uid, ncclComm_t* comm, ncclWindow_t* windows, int maxWindows) {
  if (!st || !comm) return ncclInvalidArgument;
  ncclConfig_t cfg = st->config;
  cfg.commName = st->name[0] ? st->name : nullptr;
  NCCLCHECK(ncclCommInitRankConfig(comm, st->nRanks, uid, st->rank, &cfg));
  for (size_t i = 0; i < st->windows.size(); ++i) {
    ncclWindow_t w = nullptr;
    NCCLCHECK(ncclCommWindowRegister(*comm, (void*)(uintptr_t)st->windows[i].ptr, (size_t)st->windows[i].size, &w, st->windows[i].flags));
    if (windows && (int)i < maxWindows) windows[i] = w;
  }
  return ncclSuccess;
}

ncclResult_t ncclCommCheckpointFree(ncclCheckpoint_t st) {
  delete st;
  return ncclSuccess;
}

// ---- process-wide calls with the reference's signatures (contrib/nccl_checkpoint/nccl_checkpoint.h:22-24).
// Every communicator keeps its handle. Prepare drains each GPU communicator and releases the device memory and
// peer mappings the library owns (the collective suspend of ncclCommSuspend), in creation order, which is the same
// on every rank; Restore maps everything again. Communicators the application suspended itself are left alone.
ncclResult_t ncclCheckpointPrepare(void) {
  std::vector<ncclComm*> comms;
  {
    std::lock_guard<std::mutex> g(gCommsLock);
    if (!gSuspended.empty()) { WARN("ncclCheckpointPrepare: already prepared; call ncclCheckpointRestore first"); return ncclInvalidUsage; }
    comms = gComms;
  }
  std::vector<ncclComm*> done;
  for (ncclComm* c : comms) {
    if (!commValid(c) || c->hostOnly || c->revoked || c->finalized) continue;
    NCCLCHECK(commEnsureReady(c));
    uint64_t already = 0;
    if (memStats(c, ncclStatGpuMemSuspended, &already) == ncclSuccess && already) continue;
    ncclResult_t r = memSuspend(c);
    if (r != ncclSuccess) {
      for (ncclComm* d : done) memResume(d);
      return r;
    }
    done.push_back(c);
  }
  std::lock_guard<std::mutex> g(gCommsLock);
  gSuspended = done;
  INFO(SUB_INIT, "ncclCheckpointPrepare: %zu communicator(s) suspended", done.size());
  return ncclSuccess;
}

ncclResult_t ncclCheckpointRestore(void) {
  std::vector<ncclComm*> comms;
  {
    std::lock_guard<std::mutex> g(gCommsLock);
    comms.swap(gSuspended);
  }
  ncclResult_t res = ncclSuccess;
  for (ncclComm* c : comms) {
    ncclResult_t r = commValid(c) ? memResume(c) : ncclSuccess;
    if (r != ncclSuccess && res == ncclSuccess) res = r;
  }
  INFO(SUB_INIT, "ncclCheckpointRestore: %zu communicator(s) resumed", comms.size());
  return res;
}

ncclResult_t ncclCheckpointGetVersion(int* checkpointVersion, int* ncclVersion) {
  if (checkpointVersion) *checkpointVersion = NCCL_CHECKPOINT_VERSION;
  if (ncclVersion) *ncclVersion = NCCL_VERSION_CODE;
  return ncclSuccess;
}

}  // extern "C"
