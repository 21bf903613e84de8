// Collective network: whole collectives handed to a fabric that reduces / gathers on its own,
// through the ncclCollNet table a net plugin may export (SHARP-style in-network reduction).
// Bring-up: every rank opens a listen object, the handles travel over the bootstrap all-gather,
// connect() forms the group. The group is used only when EVERY rank could join, so that all ranks
// take the same path for a collective. Data: the user's host buffers are registered around each
// call and the request is polled to completion (abort-aware).
// Reference parity: src/transport/coll_net.cc (set-up through listen / connect over the bootstrap,
// reduceSupport check, iallreduce / iallgather / ireducescatter driven by the proxy),
// NCCL_COLLNET_ENABLE (src/init.cc). There the network moves GPU memory for multi-node jobs; here the
// path serves host-memory communicators, which is where a network backend can be exercised.
#include <chrono>
#include <thread>

#include "net.h"
#include "../plugin/plugin.h"

namespace b200 {

B200_PARAM(CollNetEnable, "COLLNET_ENABLE", 0, "1: use the collective network of the net plugin (in-network reduction) when every rank can join it");

struct CollNet {
  ncclCollNet_t* api = nullptr;
  void* ctx = nullptr;
  void* listenComm = nullptr;
  void* collComm = nullptr;
  uint64_t calls = 0;
};

struct JoinInfo {
  int ok;
  char handle[NCCL_NET_HANDLE_MAXSIZE];
};

void collNetDestroy(CollNet* c) {
  if (!c) return;
  if (c->collComm && c->api->closeColl) c->api->closeColl(c->collComm);
  if (c->listenComm && c->api->closeListen) c->api->closeListen(c->listenComm);
  if (c->ctx && c->api->finalize) c->api->finalize(c->ctx);
  delete c;
}

ncclResult_t collNetCreate(ncclComm* comm, CollNet** out) {
  *out = nullptr;
  if (!paramCollNetEnable() || comm->nRanks < 2) return ncclSuccess;
  // From here on every rank takes part in the all-gather below, whatever it found locally.
  ncclCollNet_t* api = netCollNetTable();
  CollNet* c = new CollNet;
  c->api = api;
  std::vector<JoinInfo> all(comm->nRanks);
  JoinInfo& mine = all[comm->rank];
  memset(&mine, 0, sizeof(mine));
  int ndev = 0;
  if (api && api->init && api->init(&c->ctx, comm->commHash, pluginLogger) == ncclSuccess && api->devices(&ndev) == ncclSuccess && ndev > 0 &&
      api->listen(c->ctx, 0, mine.handle, &c->listenComm) == ncclSuccess)
    mine.ok = 1;
  ncclResult_t res = bootstrapAllGather(comm->bootstrap, all.data(), sizeof(JoinInfo));
  if (res != ncclSuccess) { collNetDestroy(c); return res; }
  int joined = 0;
  for (auto& j : all) joined += j.ok;
  if (joined != comm->nRanks) {
    if (comm->rank == 0) INFO(SUB_NET | SUB_INIT, "collective network: %d of %d ranks can join; not used", joined, comm->nRanks);
    collNetDestroy(c);
    return ncclSuccess;
  }
  std::vector<void*> handles(comm->nRanks);
  for (int r = 0; r < comm->nRanks; ++r) handles[r] = all[r].handle;
  ncclResult_t cr = api->connect(handles.data(), comm->nRanks, comm->rank, c->listenComm, &c->collComm);
  // connect can fail on one rank only: agree on the outcome before anybody relies on the group
  std::vector<int> okAll(comm->nRanks, 0);
  okAll[comm->rank] = cr == ncclSuccess && c->collComm ? 1 : 0;
  res = bootstrapAllGather(comm->bootstrap, okAll.data(), sizeof(int));
  int connected = 0;
  for (int v : okAll) connected += v;
  if (res != ncclSuccess || connected != comm->nRanks) {
    if (comm->rank == 0) WARN("collective network %s: only %d of %d ranks connected; not used", api->name, connected, comm->nRanks);
    collNetDestroy(c);
    return res;
  }
  if (api->closeListen && c->listenComm) { api->closeListen(c->listenComm); c->listenComm = nullptr; }
  INFO(SUB_NET | SUB_INIT, "collective network %s: rank %d of %d connected", api->name, comm->rank, comm->nRanks);
  *out = c;
  return ncclSuccess;
}

bool collNetSupports(CollNet* c, ncclDataType_t type, ncclRedOp_t op) {
  int yes = 0;
  return c && c->api->reduceSupport && c->api->reduceSupport(type, op, &yes) == ncclSuccess && yes;
}

// Registers [p, p + bytes) as host memory; nullptr handle when the plugin has no registration.
static ncclResult_t reg(CollNet* c, const void* p, size_t bytes, void** mh) {
  *mh = nullptr;
  if (!c->api->regMr || bytes == 0) return ncclSuccess;
  return c->api->regMr(c->collComm, (void*)p, bytes, NCCL_PTR_HOST, mh);
}
static void dereg(CollNet* c, void* mh) {
  if (mh && c->api->deregMr) c->api->deregMr(c->collComm, mh);
}

// Polls a request to completion. A nullptr request means "cannot post now": the caller posts again.
static ncclResult_t waitRequest(ncclComm* comm, CollNet* c, void* request) {
  int done = 0, spins = 0;
  while (!done) {
    NCCLCHECK(c->api->test(request, &done, nullptr));
    if (done) break;
    if (flagSet(comm->abortFlag)) return ncclInternalError;
    if (++spins > 1000) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  return ncclSuccess;
}

template <typename Post>
static ncclResult_t postAndWait(ncclComm* comm, CollNet* c, Post post) {
  void* request = nullptr;
  for (int tries = 0; !request; ++tries) {
    NCCLCHECK(post(&request));
    if (request) break;
    if (flagSet(comm->abortFlag)) return ncclInternalError;
    if (tries > 1000) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  c->calls++;
  return waitRequest(comm, c, request);
}

ncclResult_t collNetAllReduce(ncclComm* comm, CollNet* c, const void* send, void* recv, size_t count, ncclDataType_t type, ncclRedOp_t op) {
  const size_t bytes = count * typeSize(type);
  void *smh = nullptr, *rmh = nullptr;
  NCCLCHECK(reg(c, send, bytes, &smh));
  ncclResult_t res = send == recv ? ncclSuccess : reg(c, recv, bytes, &rmh);
  if (send == recv) rmh = smh;
  if (res == ncclSuccess)
    res = postAndWait(comm, c, [&](void** rq) { return c->api->iallreduce(c->collComm, (void*)send, recv, count, type, op, smh, rmh, rq); });
  if (rmh != smh) dereg(c, rmh);
  dereg(c, smh);
  return res;
}

// One receive part covering the whole output: rank p's block lands at recv + p * bytesPerRank.
ncclResult_t collNetAllGather(ncclComm* comm, CollNet* c, const void* send, void* recv, size_t bytesPerRank) {
  if (!c->api->iallgather) return ncclInvalidUsage;
  void *smh = nullptr, *rmh = nullptr;
  NCCLCHECK(reg(c, send, bytesPerRank, &smh));
  ncclResult_t res = reg(c, recv, bytesPerRank * comm->nRanks, &rmh);
  if (res == ncclSuccess) {
    ncclNetSGE_t part = {rmh, recv, bytesPerRank * comm->nRanks};
    res = postAndWait(comm, c, [&](void** rq) { return c->api->iallgather(c->collComm, (void*)send, 1, &part, bytesPerRank, 0, bytesPerRank, smh, rq); });
  }
  dereg(c, rmh);
  dereg(c, smh);
  return res;
}

// One send part covering the whole input: the block for rank p starts at send + p * bytesPerRank.
ncclResult_t collNetReduceScatter(ncclComm* comm, CollNet* c, const void* send, void* recv, size_t countPerRank, ncclDataType_t type, ncclRedOp_t op) {
  if (!c->api->ireducescatter) return ncclInvalidUsage;
  const size_t bytesPerRank = countPerRank * typeSize(type);
  void *smh = nullptr, *rmh = nullptr;
  NCCLCHECK(reg(c, send, bytesPerRank * comm->nRanks, &smh));
  ncclResult_t res = reg(c, recv, bytesPerRank, &rmh);
  if (res == ncclSuccess) {
    ncclNetSGE_t part = {smh, (void*)send, bytesPerRank * comm->nRanks};
    res = postAndWait(comm, c, [&](void** rq) {
      return c->api->ireducescatter(c->collComm, 1, &part, recv, bytesPerRank, 0, bytesPerRank, type, op, rmh, rq);
    });
  }
  dereg(c, rmh);
  dereg(c, smh);
  return res;
}

}  // namespace b200
