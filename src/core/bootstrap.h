// Out-of-band rendezvous and control-plane collectives over TCP.
// The byte layout of the unique id, of the rank->root check-in, of the root->rank reply,
// of the first ring all-gather payload and of tagged point-to-point messages follows the
// reference (src/bootstrap.cc, src/include/bootstrap.h:14-19) so that a rank of this
// library can rendezvous through a reference root and the other way round.
#pragma once
#include "socket.h"

namespace b200 {

struct BootstrapHandle {
  uint64_t magic;
  SockAddr addr;
  int nRanks;
};
static_assert(sizeof(BootstrapHandle) == 40, "bootstrap handle is 40 bytes inside the 128-byte unique id");
static_assert(sizeof(BootstrapHandle) <= NCCL_UNIQUE_ID_BYTES, "handle must fit the unique id");

union RingConnectInfo {
  SockAddr addr;
  char handle[128];
};
static_assert(sizeof(RingConnectInfo) == 128, "ring connect info is 128 bytes");

struct ExtInfo {
  int rank, nranks, iroot, nroots, offset;
  SockAddr listenRootAddress;
  RingConnectInfo connectInfo;
};
static_assert(sizeof(ExtInfo) == 176, "rank check-in message is 176 bytes");

struct RasRankInit {
  SockAddr addr;
  int pid;
  int cudaDev;
  int nvmlDev;
  uint64_t hostHash;
  uint64_t pidHash;
};
static_assert(sizeof(RasRankInit) == 56, "RAS rank record is 56 bytes");

struct BootstrapRingData {
  SockAddr peerAddress;
  SockAddr peerProxy;
  uint64_t peerUDS;
  RasRankInit rasRank;
};
static_assert(sizeof(BootstrapRingData) == 120, "first ring all-gather slot is 120 bytes");

enum BootstrapTag : int {
  BS_TAG_COMMSPLIT = 1 << 16,
  BS_TAG_INTRANODE_AG = (1 << 16) + 1,
  BS_TAG_BARRIER = (1 << 16) + 2,
  BS_TAG_BCAST = (1 << 16) + 3,
  BS_TAG_USER = (1 << 16) + 16,
};

struct Bootstrap;  // opaque per-communicator state

// Root side ---------------------------------------------------------------
// Fills `h` with a fresh magic and the address of a listening socket served by a detached
// root thread. With NCCL_COMM_ID set, the address comes from the environment and only the
// process that calls bootstrapCreateRoot(h, true) serves it.
ncclResult_t bootstrapNetInit();
ncclResult_t bootstrapGetUniqueId(BootstrapHandle* h);
ncclResult_t bootstrapCreateRoot(BootstrapHandle* h, bool idFromEnv);

// Rank side ---------------------------------------------------------------
struct BootstrapInitArgs {
  int cudaDev = -1;
  int nvmlDev = -1;
  volatile uint32_t* abortFlag = nullptr;
};
// handles: nHandles unique ids at a 128-byte stride (multi-root when nHandles > 1).
ncclResult_t bootstrapInit(int nHandles, const void* handles, int rank, int nranks, const BootstrapInitArgs& args,
                           Bootstrap** out);
// New ring among `nranks` ranks of `parent`; parentRanks[i] is the parent rank of new rank i.
ncclResult_t bootstrapSplit(uint64_t magic, Bootstrap* parent, int rank, int nranks, const int* parentRanks,
                            volatile uint32_t* abortFlag, Bootstrap** out);
ncclResult_t bootstrapAllGather(Bootstrap* b, void* allData, int size);
ncclResult_t bootstrapSend(Bootstrap* b, int peer, int tag, const void* data, int size);
ncclResult_t bootstrapRecv(Bootstrap* b, int peer, int tag, void* data, int size);
// Persistent tagged connections (the data plane of host-memory communicators, proxy links).
ncclResult_t bootstrapConnect(Bootstrap* b, int peer, int tag, Socket* out);
ncclResult_t bootstrapAccept(Bootstrap* b, int peer, int tag, Socket* out);
ncclResult_t bootstrapBarrier(Bootstrap* b, int tag = BS_TAG_BARRIER);
// Sub-group helpers: `ranks` lists the members (comm ranks), `rank` is my index in it.
ncclResult_t bootstrapIntraNodeBarrier(Bootstrap* b, const int* ranks, int rank, int nranks, int tag);
ncclResult_t bootstrapIntraNodeAllGather(Bootstrap* b, const int* ranks, int rank, int nranks, void* allData, int size);
ncclResult_t bootstrapIntraNodeBroadcast(Bootstrap* b, const int* ranks, int rank, int nranks, int root, void* data, int size);
ncclResult_t bootstrapBroadcast(Bootstrap* b, int root, void* data, int size);
ncclResult_t bootstrapClose(Bootstrap* b);
ncclResult_t bootstrapAbort(Bootstrap* b);

int bootstrapRank(const Bootstrap* b);
int bootstrapNRanks(const Bootstrap* b);
uint64_t bootstrapMagic(const Bootstrap* b);
const BootstrapRingData* bootstrapPeers(const Bootstrap* b);  // nranks entries (addresses, UDS ids, RAS records)
Socket* bootstrapProxyListenSocket(Bootstrap* b);             // may be null (split children sharing the parent's)

// Multi-root rank distribution (exposed for tests).
int bsRootIdFromRank(int rank, int nRanks, int nRoots, int offset);
int bsFirstRankFromRoot(int root, int nRanks, int nRoots, int offset);
int bsNRankFromRoot(int root, int nRanks, int nRoots, int offset);

}  // namespace b200
