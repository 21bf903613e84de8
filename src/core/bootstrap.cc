// Bootstrap: root rendezvous thread, TCP ring, control-plane collectives.
// Protocol (reference: src/bootstrap.cc:288-403 root, :674-883 rank, :980-1105 tagged p2p,
// :1144-1193 ring all-gather, :1221-1236 dissemination barrier):
//   1. every rank opens a ring listen socket and a root-reply listen socket, connects to
//      its root and sends  int 176 + ExtInfo;
//   2. once a root has heard from all of its ranks (plus, with several roots, the first rank
//      of the next root) it connects back to each rank and sends  int 128 + the ring
//      address of that rank's successor;
//   3. each rank connects to its successor, accepts its predecessor, and the ring
//      all-gathers one BootstrapRingData per rank;
//   4. later messages are either ring all-gathers or tagged one-shot connections that begin
//      with {int rank; int tag}.  Every message is an int length followed by the payload.
#include "bootstrap.h"

#include <pthread.h>
#include <unistd.h>

#include <algorithm>
#include <list>
#include <mutex>
#include <thread>

namespace b200 {

bool rasListenAddr(SockAddr* out);   // ras/ras.cc


B200_PARAM(StaggerRate, "UID_STAGGER_RATE", 7000, "Rank check-ins per second above the stagger threshold")
B200_PARAM(StaggerThreshold, "UID_STAGGER_THRESHOLD", 256, "Ranks per root above which check-ins are staggered")
B200_PARAM(RasEnable, "RAS_ENABLE", 1, "Start the reliability/availability/serviceability thread")

static SockAddr gIfAddr;
static char gIfName[64];
static std::once_flag gNetOnce;
static ncclResult_t gNetResult = ncclSuccess;

ncclResult_t bootstrapNetInit() {
  std::call_once(gNetOnce, [] {
    const char* env = getEnv("NCCL_COMM_ID");
    gNetResult = bootstrapInterface(&gIfAddr, gIfName);
    if (gNetResult == ncclSuccess)
      INFO(SUB_BOOTSTRAP, "Bootstrap: Using %s:%s%s", gIfName, sockAddrToString(&gIfAddr).c_str(), env ? " (NCCL_COMM_ID set)" : "");
  });
  return gNetResult;
}

// ---- length-prefixed messages -------------------------------------------------------------
static ncclResult_t msgSend(Socket* s, const void* data, int size) {
  NCCLCHECK(sockSend(s, &size, sizeof(int)));
  if (size > 0) NCCLCHECK(sockSend(s, data, size));
  return ncclSuccess;
}
static ncclResult_t msgRecv(Socket* s, void* data, int size) {
  int got = 0;
  NCCLCHECK(sockRecv(s, &got, sizeof(int)));
  if (got > size) {
    WARN("Bootstrap: message truncated: peer sent %d bytes, expected at most %d", got, size);
    return ncclInternalError;
  }
  if (got > 0) NCCLCHECK(sockRecv(s, data, got));
  return ncclSuccess;
}

// ---- multi-root rank distribution ------------------------------------------------------------
int bsFirstRankFromRoot(int root, int nRanks, int nRoots, int offset) {
  if (root == -1) return 0;
  int n = nRanks - offset;
  return offset + root * (n / nRoots) + std::min(root, n % nRoots);
}
int bsRootIdFromRank(int rank, int nRanks, int nRoots, int offset) {
  if (nRoots == 0 || rank < offset) return -1;
  int n = nRanks - offset, r = rank - offset;
  int big = n % nRoots, per = n / nRoots;
  int boundary = big * (per + 1);
  return r < boundary ? r / (per + 1) : (r - boundary) / per + big;
}
int bsNRankFromRoot(int root, int nRanks, int nRoots, int offset) {
  if (root == -1) return 0;
  int n = nRanks - offset;
  int ir = ((root % nRoots) + nRoots) % nRoots;
  return n / nRoots + (ir < n % nRoots ? 1 : 0);
}

// ---- root thread ---------------------------------------------------------------------------
struct RootArgs {
  Socket* listenSock;
  uint64_t magic;
};

static ncclResult_t rootReply(const SockAddr* to, uint64_t magic, const RingConnectInfo* info) {
  Socket s;
  NCCLCHECK(sockInit(&s, to, magic, SOCK_BOOTSTRAP));
  ncclResult_t r = sockConnect(&s);
  if (r == ncclSuccess) r = msgSend(&s, info, sizeof(*info));
  sockClose(&s);
  return r;
}

static void* rootMain(void* p) {
  RootArgs* a = (RootArgs*)p;
  setThreadName("b200 BootRoot");
  std::vector<RingConnectInfo> ringInfo;
  std::vector<SockAddr> replyAddr;
  std::vector<char> seen;
  int nranks = 0, iroot = 0, nroots = 0, offset = 0, toServe = 0, toHear = 0, heard = 0;
  do {
    Socket s;
    ExtInfo info;
    sockInit(&s, nullptr, a->magic, SOCK_BOOTSTRAP);
    if (sockAccept(&s, a->listenSock) != ncclSuccess) goto out;
    ncclResult_t r = msgRecv(&s, &info, sizeof(info));
    sockClose(&s);
    if (r != ncclSuccess) goto out;
    if (heard == 0) {
      nranks = info.nranks; iroot = info.iroot; nroots = info.nroots; offset = info.offset;
      if (nranks <= 0 || nroots <= 0 || iroot < 0) { WARN("Bootstrap root: malformed check-in"); goto out; }
      toServe = bsNRankFromRoot(iroot, nranks, nroots, offset);
      // With several roots (or a grow offset) the first rank of the next root checks in here too.
      toHear = toServe + ((offset > 0 || nroots > 1) ? 1 : 0);
      ringInfo.resize(toHear);
      replyAddr.resize(toHear);
      seen.assign(toHear, 0);
    }
    if (nranks != info.nranks || nroots != info.nroots || iroot != info.iroot || offset != info.offset) {
      WARN("Bootstrap root: ranks disagree: nranks %d/%d nroots %d/%d iroot %d/%d offset %d/%d", nranks,
           info.nranks, nroots, info.nroots, iroot, info.iroot, offset, info.offset);
      goto out;
    }
    int local = info.rank - bsFirstRankFromRoot(iroot % nroots, nranks, nroots, offset);
    if (local < 0 || local >= toHear) { WARN("Bootstrap root: rank %d does not belong to root %d", info.rank, iroot); goto out; }
    if (seen[local]) { WARN("Bootstrap root: rank %d of %d checked in twice", info.rank, nranks); goto out; }
    seen[local] = 1;
    ringInfo[local] = info.connectInfo;
    replyAddr[local] = info.listenRootAddress;
    ++heard;
    TRACE(SUB_BOOTSTRAP, "root %d: rank %d checked in (%d/%d)", iroot, info.rank, heard, toHear);
  } while (heard < toHear);
  // Everyone is here: tell each served rank where its ring successor listens.
  for (int r = 0; r < toServe; ++r) {
    if (rootReply(&replyAddr[r], a->magic, &ringInfo[(r + 1) % toHear]) != ncclSuccess) {
      WARN("Bootstrap root: could not reach local rank %d at %s", r, sockAddrToString(&replyAddr[r]).c_str());
    }
  }
out:
  sockClose(a->listenSock);
  delete a->listenSock;
  delete a;
  return nullptr;
}

ncclResult_t bootstrapCreateRoot(BootstrapHandle* h, bool idFromEnv) {
  NCCLCHECK(bootstrapNetInit());
  Socket* ls = new Socket;
  sockInit(ls, idFromEnv ? &h->addr : &gIfAddr, h->magic, SOCK_BOOTSTRAP);
  if (!idFromEnv) {
    if (ls->addr.sa.sa_family == AF_INET) ls->addr.sin.sin_port = 0; else ls->addr.sin6.sin6_port = 0;
  }
  ncclResult_t r = sockListen(ls);
  if (r != ncclSuccess) { delete ls; return r; }
  h->addr = ls->addr;
  RootArgs* a = new RootArgs{ls, h->magic};
  pthread_t t;
  if (pthread_create(&t, nullptr, rootMain, a) != 0) { WARN("pthread_create failed"); return ncclSystemError; }
  pthread_detach(t);
  return ncclSuccess;
}

ncclResult_t bootstrapGetUniqueId(BootstrapHandle* h) {
  memset(h, 0, sizeof(*h));
  NCCLCHECK(bootstrapNetInit());
  const char* env = getEnv("NCCL_COMM_ID");
  if (env && *env) {
    INFO(SUB_ENV, "NCCL_COMM_ID set by environment to %s", env);
    NCCLCHECK(sockAddrFromString(&h->addr, env));
    h->magic = kSocketMagic;  // every process derives the same id from the environment
  } else {
    h->magic = randomU64();
    NCCLCHECK(bootstrapCreateRoot(h, false));
  }
  return ncclSuccess;
}

// ---- per-communicator state ------------------------------------------------------------------
struct Unexpected {
  int peer, tag;
  Socket sock;
};

struct Bootstrap {
  int rank = 0, nranks = 0;
  uint64_t magic = 0;
  volatile uint32_t* abortFlag = nullptr;
  Socket ringListen, ringSend, ringRecv, peerListen;
  Socket* proxyListen = nullptr;
  std::vector<BootstrapRingData> peers;
  std::list<Unexpected> unexpected;
  std::mutex lock;  // serialises tagged traffic of one communicator
};

int bootstrapRank(const Bootstrap* b) { return b->rank; }
int bootstrapNRanks(const Bootstrap* b) { return b->nranks; }
uint64_t bootstrapMagic(const Bootstrap* b) { return b->magic; }
const BootstrapRingData* bootstrapPeers(const Bootstrap* b) { return b->peers.data(); }
Socket* bootstrapProxyListenSocket(Bootstrap* b) { return b->proxyListen; }

static ncclResult_t listenOn(Socket* s, uint64_t magic, SockType type, volatile uint32_t* abortFlag, SockAddr* out) {
  NCCLCHECK(bootstrapNetInit());
  SockAddr a = gIfAddr;
  if (a.sa.sa_family == AF_INET) a.sin.sin_port = 0; else a.sin6.sin6_port = 0;
  NCCLCHECK(sockInit(s, &a, magic, type, abortFlag));
  NCCLCHECK(sockListen(s));
  if (out) *out = s->addr;
  return ncclSuccess;
}

static ncclResult_t ringConnect(Bootstrap* b, const SockAddr* next) {
  NCCLCHECK(sockInit(&b->ringSend, next, b->magic, SOCK_BOOTSTRAP, b->abortFlag));
  NCCLCHECK(sockConnect(&b->ringSend));
  NCCLCHECK(sockInit(&b->ringRecv, nullptr, b->magic, SOCK_BOOTSTRAP, b->abortFlag));
  NCCLCHECK(sockAccept(&b->ringRecv, &b->ringListen));
  return ncclSuccess;
}

static ncclResult_t checkIn(const BootstrapHandle* h, volatile uint32_t* abortFlag, const ExtInfo* info) {
  Socket s;
  NCCLCHECK(sockInit(&s, &h->addr, h->magic, SOCK_BOOTSTRAP, abortFlag));
  ncclResult_t r = sockConnect(&s);
  if (r == ncclSuccess) r = msgSend(&s, info, sizeof(*info));
  sockClose(&s);
  return r;
}

static ncclResult_t exchangePeerTable(Bootstrap* b, const SockAddr* proxyAddr, const RasRankInit* ras) {
  b->peers.assign(b->nranks, BootstrapRingData{});
  BootstrapRingData& me = b->peers[b->rank];
  me.peerAddress = b->peerListen.addr;
  if (proxyAddr) me.peerProxy = *proxyAddr;
  me.peerUDS = randomU64();
  if (ras) me.rasRank = *ras;
  return bootstrapAllGather(b, b->peers.data(), sizeof(BootstrapRingData));
}

ncclResult_t bootstrapInit(int nHandles, const void* handles, int rank, int nranks, const BootstrapInitArgs& args,
                           Bootstrap** out) {
  auto handleAt = [&](int i) { return (const BootstrapHandle*)((const char*)handles + (size_t)i * NCCL_UNIQUE_ID_BYTES); };
  if (nHandles < 1 || !handles || rank < 0 || rank >= nranks) return ncclInvalidArgument;
  Bootstrap* b = new Bootstrap;
  ncclResult_t ret = ncclSuccess;
  b->rank = rank;
  b->nranks = nranks;
  b->abortFlag = args.abortFlag;
  b->magic = handleAt(0)->magic;
  ExtInfo info;
  memset(&info, 0, sizeof(info));
  RingConnectInfo nextPeer;
  memset(&nextPeer, 0, sizeof(nextPeer));
  Socket rootReplyListen, reply;
  const int offset = 0;
  int root = bsRootIdFromRank(rank, nranks, nHandles, offset);
  SockAddr proxyAddr;
  RasRankInit ras;

  NCCLCHECKGOTO(listenOn(&b->ringListen, b->magic, SOCK_BOOTSTRAP, b->abortFlag, &info.connectInfo.addr), ret, fail);
  NCCLCHECKGOTO(listenOn(&rootReplyListen, handleAt(root)->magic, SOCK_BOOTSTRAP, b->abortFlag, &info.listenRootAddress), ret, fail);
  info.nranks = nranks;
  info.nroots = nHandles;
  info.offset = offset;

  {  // spread check-ins of very large jobs over time so the root's accept queue never overflows
    int perRoot = bsNRankFromRoot(root, nranks, nHandles, offset);
    if (perRoot > paramStaggerThreshold()) {
      double perUs = paramStaggerRate() / 1.0e6;
      long us = (long)((rank - bsFirstRankFromRoot(root, nranks, nHandles, offset)) / perUs);
      std::this_thread::sleep_for(std::chrono::microseconds(us));
    }
  }
  info.rank = rank;
  info.iroot = root;
  NCCLCHECKGOTO(checkIn(handleAt(root), b->abortFlag, &info), ret, fail);
  if (nHandles > 1 && rank == bsFirstRankFromRoot(root, nranks, nHandles, offset)) {
    // The previous root owns the link from its last rank to me: check in there too, numbered
    // one past its last rank.
    int prevRank = (rank - 1 + nranks) % nranks;
    int prevRoot = bsRootIdFromRank(prevRank, nranks, nHandles, offset);
    ExtInfo extra = info;
    extra.rank = prevRank + 1;
    extra.iroot = prevRoot;
    NCCLCHECKGOTO(checkIn(handleAt(prevRoot), b->abortFlag, &extra), ret, fail);
  }
  sockInit(&reply, nullptr, handleAt(root)->magic, SOCK_BOOTSTRAP, b->abortFlag);
  NCCLCHECKGOTO(sockAccept(&reply, &rootReplyListen), ret, fail);
  ret = msgRecv(&reply, &nextPeer, sizeof(nextPeer));
  sockClose(&reply);
  sockClose(&rootReplyListen);
  if (ret != ncclSuccess) goto fail;

  NCCLCHECKGOTO(ringConnect(b, &nextPeer.addr), ret, fail);
  b->proxyListen = new Socket;
  NCCLCHECKGOTO(listenOn(b->proxyListen, b->magic, SOCK_PROXY, b->abortFlag, &proxyAddr), ret, fail);
  NCCLCHECKGOTO(listenOn(&b->peerListen, b->magic, SOCK_BOOTSTRAP, b->abortFlag, nullptr), ret, fail);
  memset(&ras, 0, sizeof(ras));
  ras.addr = gIfAddr;
  if (paramRasEnable()) {
    SockAddr ra;
    if (rasListenAddr(&ra)) ras.addr = ra;   // port 0 (the bare interface address) tells peers that this rank runs without RAS
  }
  ras.pid = (int)getpid();
  ras.cudaDev = args.cudaDev;
  ras.nvmlDev = args.nvmlDev;
  ras.hostHash = hostHash();
  ras.pidHash = pidHash();
  NCCLCHECKGOTO(exchangePeerTable(b, &proxyAddr, &ras), ret, fail);
  INFO(SUB_BOOTSTRAP, "Bootstrap: rank %d/%d ready (magic 0x%llx)", rank, nranks, (unsigned long long)b->magic);
  *out = b;
  return ncclSuccess;
fail:
  sockClose(&rootReplyListen);
  bootstrapClose(b);
  return ret;
}

ncclResult_t bootstrapSplit(uint64_t magic, Bootstrap* parent, int rank, int nranks, const int* parentRanks,
                            volatile uint32_t* abortFlag, Bootstrap** out) {
  Bootstrap* b = new Bootstrap;
  ncclResult_t ret = ncclSuccess;
  b->rank = rank;
  b->nranks = nranks;
  b->magic = magic;
  b->abortFlag = abortFlag;
  RingConnectInfo mine, next;
  memset(&mine, 0, sizeof(mine));
  memset(&next, 0, sizeof(next));
  SockAddr proxyAddr;
  int prev = parentRanks[(rank - 1 + nranks) % nranks];
  int nxt = parentRanks[(rank + 1) % nranks];
  NCCLCHECKGOTO(listenOn(&b->ringListen, magic, SOCK_BOOTSTRAP, abortFlag, &mine.addr), ret, fail);
  NCCLCHECKGOTO(listenOn(&b->peerListen, magic, SOCK_BOOTSTRAP, abortFlag, nullptr), ret, fail);
  // My predecessor in the new ring needs my listen address; I need my successor's.
  NCCLCHECKGOTO(bootstrapSend(parent, prev, BS_TAG_COMMSPLIT, &mine, sizeof(mine)), ret, fail);
  NCCLCHECKGOTO(bootstrapRecv(parent, nxt, BS_TAG_COMMSPLIT, &next, sizeof(next)), ret, fail);
  NCCLCHECKGOTO(ringConnect(b, &next.addr), ret, fail);
  b->proxyListen = new Socket;
  NCCLCHECKGOTO(listenOn(b->proxyListen, magic, SOCK_PROXY, abortFlag, &proxyAddr), ret, fail);
  {
    RasRankInit ras = parent->peers[parent->rank].rasRank;
    NCCLCHECKGOTO(exchangePeerTable(b, &proxyAddr, &ras), ret, fail);
  }
  *out = b;
  return ncclSuccess;
fail:
  bootstrapClose(b);
  return ret;
}

// ---- ring all-gather -------------------------------------------------------------------------
// Two rings run at once (clockwise and counter-clockwise) so that n ranks finish in n/2 steps.
ncclResult_t bootstrapAllGather(Bootstrap* b, void* allData, int size) {
  int n = b->nranks, rank = b->rank;
  char* data = (char*)allData;
  if (n == 1) return ncclSuccess;
  int steps = n / 2;
  for (int step = 0; step < steps; ++step) {
    bool lastOneWay = (step == steps - 1) && (n % 2 == 0);
    int cwSend = (rank - step + n) % n, cwRecv = (rank - step - 1 + n) % n;
    int ccwSend = (rank + step) % n, ccwRecv = (rank + step + 1) % n;
    int szOut = size, szInCw = 0, szInCcw = 0;
    NCCLCHECK(sockSendRecv(&b->ringSend, &szOut, sizeof(int), &b->ringRecv, &szInCw, sizeof(int)));
    if (!lastOneWay) NCCLCHECK(sockSendRecv(&b->ringRecv, &szOut, sizeof(int), &b->ringSend, &szInCcw, sizeof(int)));
    if (szInCw > size || szInCcw > size) {
      WARN("Bootstrap all-gather: peer slot is %d/%d bytes, expected %d", szInCw, szInCcw, size);
      return ncclInternalError;
    }
    SockOp ops[4] = {{SOCK_OP_SEND, &b->ringSend, data + (size_t)cwSend * size, size, 0},
                     {SOCK_OP_RECV, &b->ringRecv, data + (size_t)cwRecv * size, szInCw, 0},
                     {SOCK_OP_SEND, &b->ringRecv, data + (size_t)ccwSend * size, size, 0},
                     {SOCK_OP_RECV, &b->ringSend, data + (size_t)ccwRecv * size, szInCcw, 0}};
    NCCLCHECK(sockMultiOp(ops, lastOneWay ? 2 : 4));
  }
  return ncclSuccess;
}

// ---- tagged point-to-point ---------------------------------------------------------------------
struct AckInfo { int rank, tag; };

ncclResult_t bootstrapConnect(Bootstrap* b, int peer, int tag, Socket* s) {
  AckInfo ack{b->rank, tag};
  NCCLCHECK(sockInit(s, &b->peers[peer].peerAddress, b->magic, SOCK_BOOTSTRAP, b->abortFlag));
  ncclResult_t r = sockConnect(s);
  if (r == ncclSuccess) r = msgSend(s, &ack, sizeof(ack));
  if (r != ncclSuccess) sockClose(s);
  return r;
}

ncclResult_t bootstrapAccept(Bootstrap* b, int peer, int tag, Socket* s) {
  std::lock_guard<std::mutex> g(b->lock);
  for (auto it = b->unexpected.begin(); it != b->unexpected.end(); ++it) {
    if ((peer < 0 || it->peer == peer) && it->tag == tag) {
      *s = it->sock;
      b->unexpected.erase(it);
      return ncclSuccess;
    }
  }
  for (;;) {
    AckInfo ack{0, 0};
    sockInit(s, nullptr, b->magic, SOCK_BOOTSTRAP, b->abortFlag);
    NCCLCHECK(sockAccept(s, &b->peerListen));
    ncclResult_t r = msgRecv(s, &ack, sizeof(ack));
    if (r != ncclSuccess) { sockClose(s); return r; }
    if (ack.tag == tag && (peer < 0 || ack.rank == peer)) return ncclSuccess;
    b->unexpected.push_back(Unexpected{ack.rank, ack.tag, *s});  // someone else's message: park it
  }
}

ncclResult_t bootstrapSend(Bootstrap* b, int peer, int tag, const void* data, int size) {
  Socket s;
  NCCLCHECK(bootstrapConnect(b, peer, tag, &s));
  ncclResult_t r = msgSend(&s, data, size);
  sockClose(&s);
  return r;
}

ncclResult_t bootstrapRecv(Bootstrap* b, int peer, int tag, void* data, int size) {
  Socket s;
  NCCLCHECK(bootstrapAccept(b, peer, tag, &s));
  ncclResult_t r = msgRecv(&s, data, size);
  sockClose(&s, r == ncclSuccess);
  return r;
}

// Dissemination barrier: log2(n) rounds, round k talks to rank +/- 2^k.
static ncclResult_t p2pBarrier(Bootstrap* b, const int* ranks, int rank, int nranks, int tag) {
  int token = 0;
  for (int mask = 1; mask < nranks; mask <<= 1) {
    int src = (rank - mask + nranks) % nranks, dst = (rank + mask) % nranks;
    NCCLCHECK(bootstrapSend(b, ranks ? ranks[dst] : dst, tag, &token, sizeof(token)));
    NCCLCHECK(bootstrapRecv(b, ranks ? ranks[src] : src, tag, &token, sizeof(token)));
  }
  return ncclSuccess;
}
ncclResult_t bootstrapBarrier(Bootstrap* b, int tag) { return p2pBarrier(b, nullptr, b->rank, b->nranks, tag); }
ncclResult_t bootstrapIntraNodeBarrier(Bootstrap* b, const int* ranks, int rank, int nranks, int tag) {
  return p2pBarrier(b, ranks, rank, nranks, tag);
}

ncclResult_t bootstrapIntraNodeAllGather(Bootstrap* b, const int* ranks, int rank, int nranks, void* allData, int size) {
  if (nranks == 1) return ncclSuccess;
  char* data = (char*)allData;
  int prev = ranks[(rank - 1 + nranks) % nranks], next = ranks[(rank + 1) % nranks];
  // plain ring over tagged messages; slot moving at step i originated at rank - i
  for (int i = 1; i < nranks; ++i) {
    int sslice = (rank - i + 1 + nranks) % nranks, rslice = (rank - i + nranks) % nranks;
    NCCLCHECK(bootstrapSend(b, next, BS_TAG_INTRANODE_AG, data + (size_t)sslice * size, size));
    NCCLCHECK(bootstrapRecv(b, prev, BS_TAG_INTRANODE_AG, data + (size_t)rslice * size, size));
  }
  return ncclSuccess;
}

ncclResult_t bootstrapIntraNodeBroadcast(Bootstrap* b, const int* ranks, int rank, int nranks, int root, void* data, int size) {
  if (nranks == 1) return ncclSuccess;
  if (rank == root) {
    for (int i = 0; i < nranks; ++i)
      if (i != root) NCCLCHECK(bootstrapSend(b, ranks ? ranks[i] : i, BS_TAG_BCAST, data, size));
  } else {
    NCCLCHECK(bootstrapRecv(b, ranks ? ranks[root] : root, BS_TAG_BCAST, data, size));
  }
  return ncclSuccess;
}
ncclResult_t bootstrapBroadcast(Bootstrap* b, int root, void* data, int size) {
  return bootstrapIntraNodeBroadcast(b, nullptr, b->rank, b->nranks, root, data, size);
}

ncclResult_t bootstrapClose(Bootstrap* b) {
  if (!b) return ncclSuccess;
  for (auto& u : b->unexpected) sockClose(&u.sock);
  sockClose(&b->ringListen);
  sockClose(&b->ringSend);
  sockClose(&b->ringRecv);
  sockClose(&b->peerListen);
  if (b->proxyListen) { sockClose(b->proxyListen); delete b->proxyListen; }
  delete b;
  return ncclSuccess;
}
ncclResult_t bootstrapAbort(Bootstrap* b) { return bootstrapClose(b); }

}  // namespace b200
