// Host-memory data plane: every collective executed by the calling thread over a full mesh of
// persistent TCP connections between the ranks. It serves communicators created on machines
// without a GPU (buffers are host pointers) and is the fallback that GPU communicators stage
// through when ranks are not load/store reachable (different hosts, P2P disabled).
// Schedules: ring reduce-scatter + ring all-gather for all-reduce (the classic 2(n-1)-step
// schedule, reference: src/device/all_reduce.h:14-83 runs the same steps on the GPU), rings for
// all-gather / reduce-scatter, chains for broadcast / reduce, pairwise exchange for all-to-all.
#include <algorithm>
#include <functional>

#include "../comm/comm.h"
#include "hosttypes.h"

#include <sched.h>

#include "../transport/net.h"
#include "../transport/shm.h"

namespace b200 {

struct HostPlane {
  std::vector<Socket> peer;   // peer[r] connected to rank r (unused for r == rank)
  std::vector<char> tmp;
  Proxy* proxy = nullptr;     // set when messages travel through the network backend instead
  std::vector<ShmLink> shmOut, shmIn;   // set when every rank is on this host and NCCL_B200_HOST_SHM=1
  bool shm = false;
  CollNet* collnet = nullptr;   // in-network collectives of the net plugin, when every rank joined (NCCL_COLLNET_ENABLE=1)
  volatile uint32_t* abortFlag = nullptr;
};

B200_PARAM(HostShm, "B200_HOST_SHM", 0, "1: ranks of one host exchange host-memory messages through shared-memory rings instead of TCP");
B200_PARAM(HostShmKb, "B200_HOST_SHM_KB", 4096, "capacity of one shared-memory ring, KiB");

struct ShmOp { ShmLink* link; char* p; size_t n, off; bool send; };

// Progresses all operations together; two operations on one link and direction run in posting order.
static ncclResult_t shmRun(HostPlane* hp, std::vector<ShmOp>& ops) {
  uint64_t last = nowNs();
  const uint64_t budget = 120ull * 1000000000ull;
  size_t left = 0;
  for (auto& o : ops) if (o.off < o.n) ++left;
  while (left) {
    bool moved = false;
    for (size_t i = 0; i < ops.size(); ++i) {
      ShmOp& o = ops[i];
      if (o.off >= o.n) continue;
      bool blocked = false;
      for (size_t j = 0; j < i; ++j) if (ops[j].off < ops[j].n && ops[j].link == o.link && ops[j].send == o.send) blocked = true;
      if (blocked) continue;
      size_t m = o.send ? shmLinkSend(o.link, o.p + o.off, o.n - o.off) : shmLinkRecv(o.link, o.p + o.off, o.n - o.off);
      if (m) { o.off += m; moved = true; if (o.off >= o.n) --left; }
    }
    if (moved) { last = nowNs(); continue; }
    if (hp->abortFlag && __atomic_load_n(hp->abortFlag, __ATOMIC_RELAXED)) return ncclInternalError;
    if (nowNs() - last > budget) { WARN("shared-memory link made no progress for 120 s"); return ncclSystemError; }
    sched_yield();
  }
  return ncclSuccess;
}

B200_PARAM(HostNet, "B200_HOST_NET", 0, "1: host-memory messages go through the network backend (plugin or built-in Socket) and the proxy thread; 0: direct TCP mesh");

static constexpr int kTagHostMesh = BS_TAG_USER + 1;

static ncclResult_t hostPlaneCreateLinks(ncclComm* comm) {
  HostPlane* hp = new HostPlane;
  int n = comm->nRanks, me = comm->rank;
  hp->peer.resize(n);
  hp->abortFlag = comm->abortFlag;
  const char* shmOff = getEnv("NCCL_SHM_DISABLE");
  if (paramHostShm() && comm->nNodes == 1 && !(shmOff && atoi(shmOff) == 1)) {
    hp->shmIn.resize(n);
    hp->shmOut.resize(n);
    char base[96];
    snprintf(base, sizeof(base), "/nccl-b200-%llx", (unsigned long long)comm->commHash);
    ncclResult_t res = ncclSuccess;
    for (int r = 0; r < n && res == ncclSuccess; ++r)
      if (r != me) res = shmLinkCreate(std::string(base) + "-" + std::to_string(r) + "-" + std::to_string(me), (size_t)paramHostShmKb() << 10, &hp->shmIn[r]);
    if (res == ncclSuccess) res = bootstrapBarrier(comm->bootstrap);
    for (int r = 0; r < n && res == ncclSuccess; ++r)
      if (r != me) res = shmLinkOpen(std::string(base) + "-" + std::to_string(me) + "-" + std::to_string(r), &hp->shmOut[r]);
    if (res == ncclSuccess) res = bootstrapBarrier(comm->bootstrap);
    for (auto& l : hp->shmIn) shmLinkUnlink(&l);   // everybody has attached: the names can go
    if (res != ncclSuccess) { delete hp; return res; }
    hp->shm = true;
    comm->hostPlane = hp;
    INFO(SUB_SHM | SUB_INIT, "host plane of rank %d: shared-memory rings to %d local peers (%lld KiB each)", me, n - 1, (long long)paramHostShmKb());
    return ncclSuccess;
  }
  bool ext = false;
  ncclNet_t* net = nullptr;
  if (netSelect(&net, &ext) == ncclSuccess && (ext || paramHostNet())) {
    ncclResult_t res = proxyCreate(comm);
    if (res != ncclSuccess) { delete hp; return res; }
    hp->proxy = comm->proxy;
    comm->hostPlane = hp;
    return ncclSuccess;
  }
  // Higher ranks listen, lower ranks dial: connects land in the listen backlog, so dialling
  // everything first and accepting afterwards cannot deadlock.
  for (int r = me + 1; r < n; ++r) {
    ncclResult_t res = bootstrapConnect(comm->bootstrap, r, kTagHostMesh, &hp->peer[r]);
    if (res != ncclSuccess) { delete hp; return res; }
  }
  for (int r = 0; r < me; ++r) {
    ncclResult_t res = bootstrapAccept(comm->bootstrap, r, kTagHostMesh, &hp->peer[r]);
    if (res != ncclSuccess) { delete hp; return res; }
  }
  comm->hostPlane = hp;
  return ncclSuccess;
}

ncclResult_t hostPlaneCreate(ncclComm* comm) {
  NCCLCHECK(hostPlaneCreateLinks(comm));
  return collNetCreate(comm, &comm->hostPlane->collnet);
}

void hostPlaneDestroy(ncclComm* comm) {
  if (!comm->hostPlane) return;
  collNetDestroy(comm->hostPlane->collnet);
  proxyDestroy(comm);
  for (auto& l : comm->hostPlane->shmIn) shmLinkClose(&l);
  for (auto& l : comm->hostPlane->shmOut) shmLinkClose(&l);
  for (auto& s : comm->hostPlane->peer) sockClose(&s);
  delete comm->hostPlane;
  comm->hostPlane = nullptr;
}

static ncclResult_t exchange(HostPlane* hp, int to, const void* sbuf, size_t sbytes, int from, void* rbuf, size_t rbytes) {
  if (hp->shm) {
    std::vector<ShmOp> ops;
    if (sbytes > 0) ops.push_back(ShmOp{&hp->shmOut[to], (char*)sbuf, sbytes, 0, true});
    if (rbytes > 0) ops.push_back(ShmOp{&hp->shmIn[from], (char*)rbuf, rbytes, 0, false});
    return shmRun(hp, ops);
  }
  if (hp->proxy) {
    ProxyOp* ops[2];
    int k = 0;
    if (sbytes > 0) ops[k++] = proxyPost(hp->proxy, true, to, (void*)sbuf, sbytes);
    if (rbytes > 0) ops[k++] = proxyPost(hp->proxy, false, from, rbuf, rbytes);
    return proxyWait(hp->proxy, ops, k);
  }
  // messages larger than INT_MAX are cut in pieces; both sides cut identically
  const size_t piece = 1u << 30;
  size_t so = 0, ro = 0;
  while (so < sbytes || ro < rbytes) {
    int sn = (int)std::min(piece, sbytes - so), rn = (int)std::min(piece, rbytes - ro);
    SockOp ops[2];
    int k = 0;
    if (sn > 0) ops[k++] = SockOp{SOCK_OP_SEND, &hp->peer[to], (char*)sbuf + so, sn, 0};
    if (rn > 0) ops[k++] = SockOp{SOCK_OP_RECV, &hp->peer[from], (char*)rbuf + ro, rn, 0};
    NCCLCHECK(sockMultiOp(ops, k));
    so += sn;
    ro += rn;
  }
  return ncclSuccess;
}

struct Chunks {
  size_t count;
  int n;
  size_t off(int i) const { size_t base = count / n, rem = count % n; return (size_t)i * base + std::min<size_t>(i, rem); }
  size_t len(int i) const { return count / n + ((size_t)i < count % n ? 1 : 0); }
};

struct OpDesc {
  int hop;            // HostOp
  bool premul = false, postscale = false;
  double scale = 1.0;
  int64_t intDiv = 1;
};

static ncclResult_t resolveOp(ncclComm* comm, const Task& t, OpDesc* d) {
  if (t.op == ncclSum || t.op == ncclProd || t.op == ncclMax || t.op == ncclMin) {
    d->hop = t.op == ncclSum ? HOP_SUM : t.op == ncclProd ? HOP_PROD : t.op == ncclMax ? HOP_MAX : HOP_MIN;
    return ncclSuccess;
  }
  if (t.op == ncclAvg) {
    d->hop = HOP_SUM;
    d->postscale = true;
    d->scale = 1.0 / comm->nRanks;
    d->intDiv = comm->nRanks;
    return ncclSuccess;
  }
  int idx = t.op - ncclNumOps;
  if (idx < 0 || idx >= (int)comm->userOps.size() || !comm->userOps[idx].used) {
    WARN("invalid reduction operator %d", t.op);
    return ncclInvalidArgument;
  }
  const UserRedOp& u = comm->userOps[idx];
  uint64_t bits = u.scalarBits;
  if (u.residence == ncclScalarDevice) memcpy(&bits, u.devScalar, typeSize(u.type));  // host plane: plain memory
  d->hop = HOP_SUM;
  d->premul = true;
  switch (u.type) {
    case ncclFloat32: { float f; memcpy(&f, &bits, 4); d->scale = f; } break;
    case ncclFloat64: { double f; memcpy(&f, &bits, 8); d->scale = f; } break;
    case ncclFloat16: d->scale = halfToFloat((uint16_t)bits); break;
    case ncclBfloat16: d->scale = bf16ToFloat((uint16_t)bits); break;
    case ncclFloat8e4m3: d->scale = e4m3ToFloat((uint8_t)bits); break;
    case ncclFloat8e5m2: d->scale = e5m2ToFloat((uint8_t)bits); break;
    default: {
      // integer pre-multiply
      int64_t v = 0;
      memcpy(&v, &bits, typeSize(u.type));
      d->scale = (double)v;
    }
  }
  return ncclSuccess;
}

static ncclRedOp_t hopToRedOp(int hop) { return hop == HOP_SUM ? ncclSum : hop == HOP_PROD ? ncclProd : hop == HOP_MAX ? ncclMax : ncclMin; }

static void premulInto(void* dst, size_t n, ncclDataType_t type, const OpDesc& d) {
  if (!d.premul) return;
  switch (type) {
    case ncclInt8: case ncclUint8: case ncclInt32: case ncclUint32: case ncclInt64: case ncclUint64: {
      int64_t m = (int64_t)d.scale;
      size_t es = typeSize(type);
      for (size_t i = 0; i < n; ++i) {
        int64_t v = 0;
        memcpy(&v, (char*)dst + i * es, es);
        if (type == ncclInt8) v = (int8_t)v; else if (type == ncclInt32) v = (int32_t)v;
        v *= m;
        memcpy((char*)dst + i * es, &v, es);
      }
    } break;
    default: hostScale(dst, n, type, d.scale, 1);
  }
}

static ncclResult_t ringReduceScatterInPlace(ncclComm* comm, char* buf, const Chunks& ch, size_t es, ncclDataType_t type, int hop,
                                             int shift) {
  // After n-1 steps rank r holds the fully reduced chunk (r + shift) mod n.
  HostPlane* hp = comm->hostPlane;
  int n = comm->nRanks, r = comm->rank, next = (r + 1) % n, prev = (r - 1 + n) % n;
  hp->tmp.resize((ch.count / n + 1) * es);
  for (int s = 0; s < n - 1; ++s) {
    int sc = ((r + shift - 1 - s) % n + 2 * n) % n, rc = ((r + shift - 2 - s) % n + 2 * n) % n;
    NCCLCHECK(exchange(hp, next, buf + ch.off(sc) * es, ch.len(sc) * es, prev, hp->tmp.data(), ch.len(rc) * es));
    hostReduceInto(buf + ch.off(rc) * es, hp->tmp.data(), ch.len(rc), type, hop);
  }
  return ncclSuccess;
}

static ncclResult_t ringAllGatherInPlace(ncclComm* comm, char* buf, const Chunks& ch, size_t es, int shift) {
  // Rank r starts owning chunk (r + shift) mod n.
  HostPlane* hp = comm->hostPlane;
  int n = comm->nRanks, r = comm->rank, next = (r + 1) % n, prev = (r - 1 + n) % n;
  for (int s = 0; s < n - 1; ++s) {
    int sc = ((r + shift - s) % n + 2 * n) % n, rc = ((r + shift - 1 - s) % n + 2 * n) % n;
    NCCLCHECK(exchange(hp, next, buf + ch.off(sc) * es, ch.len(sc) * es, prev, buf + ch.off(rc) * es, ch.len(rc) * es));
  }
  return ncclSuccess;
}

// ---- log-step schedules (what the reference calls PAT, parallel aggregated trees: include/collectives.h:411-923).
// ceil(log2 n) exchanges instead of n - 1: step k moves up to 2^k aggregated blocks between ranks 2^k apart.
// `work` holds n blocks of `blk` bytes in rotated order: work[i] belongs to rank (r + i) mod n.
static ncclResult_t logStepAllGather(ncclComm* comm, char* work, size_t blk) {
  HostPlane* hp = comm->hostPlane;
  const int n = comm->nRanks, r = comm->rank;
  for (int dist = 1; dist < n; dist <<= 1) {
    const int cnt = std::min(dist, n - dist);
    const int to = (r - dist + n) % n, from = (r + dist) % n;
    NCCLCHECK(exchange(hp, to, work, (size_t)cnt * blk, from, work + (size_t)dist * blk, (size_t)cnt * blk));
  }
  return ncclSuccess;
}

// The same exchanges backwards: blocks travel towards their owners and are summed on the way; work[0] ends
// as the reduction of this rank's block over all ranks.
static ncclResult_t logStepReduceScatter(ncclComm* comm, char* work, size_t blkElems, size_t es, ncclDataType_t type, int hop) {
  HostPlane* hp = comm->hostPlane;
  const int n = comm->nRanks, r = comm->rank;
  const size_t blk = blkElems * es;
  int top = 1;
  while (top * 2 < n) top <<= 1;
  for (int dist = top; dist >= 1; dist >>= 1) {
    const int cnt = std::min(dist, n - dist);
    const int to = (r + dist) % n, from = (r - dist + n) % n;
    hp->tmp.resize((size_t)cnt * blk);
    NCCLCHECK(exchange(hp, to, work + (size_t)dist * blk, (size_t)cnt * blk, from, hp->tmp.data(), (size_t)cnt * blk));
    hostReduceInto(work, hp->tmp.data(), (size_t)cnt * blkElems, type, hop);
  }
  return ncclSuccess;
}

B200_PARAM(HostLogStepBytes, "B200_HOST_LOGSTEP_BYTES", 65536,
           "host-memory all-gather / reduce-scatter of at most this many bytes per rank use the log-step (PAT) schedule when there are more than two ranks");

static bool useLogStep(ncclComm* comm, size_t bytesPerRank) {
  static const char* e = getEnv("NCCL_ALGO");
  if (comm->nRanks < 3) return false;
  if (e && *e) return !strcasecmp(e, "PAT");
  return bytesPerRank <= (size_t)paramHostLogStepBytes();
}

ncclResult_t hostPlaneRun(ncclComm* comm, const Task& t) {
  HostPlane* hp = comm->hostPlane;
  if (!hp) return ncclInternalError;
  const int n = comm->nRanks, r = comm->rank;
  const size_t es = typeSize(t.type);
  OpDesc od{};
  switch (t.func) {
    case FUNC_ALLREDUCE: {
      NCCLCHECK(resolveOp(comm, t, &od));
      if (hp->collnet && n > 1 && !od.premul && collNetSupports(hp->collnet, t.type, hopToRedOp(od.hop))) {
        NCCLCHECK(collNetAllReduce(comm, hp->collnet, t.send, t.recv, t.count, t.type, hopToRedOp(od.hop)));
        if (od.postscale) hostScale(t.recv, t.count, t.type, od.scale, od.intDiv);
        break;
      }
      if (t.recv != t.send) memcpy(t.recv, t.send, t.count * es);
      premulInto(t.recv, t.count, t.type, od);
      if (n > 1) {
        Chunks ch{t.count, n};
        NCCLCHECK(ringReduceScatterInPlace(comm, (char*)t.recv, ch, es, t.type, od.hop, 1));
        NCCLCHECK(ringAllGatherInPlace(comm, (char*)t.recv, ch, es, 1));
      }
      if (od.postscale) hostScale(t.recv, t.count, t.type, od.scale, od.intDiv);
    } break;
    case FUNC_REDUCESCATTER: {
      NCCLCHECK(resolveOp(comm, t, &od));
      size_t total = t.count * n;
      if (hp->collnet && n > 1 && !od.premul && collNetSupports(hp->collnet, t.type, hopToRedOp(od.hop)) &&
          collNetReduceScatter(comm, hp->collnet, t.send, t.recv, t.count, t.type, hopToRedOp(od.hop)) == ncclSuccess) {
        if (od.postscale) hostScale(t.recv, t.count, t.type, od.scale, od.intDiv);
        break;
      }
      std::vector<char> work(total * es);
      if (useLogStep(comm, t.count * es)) {
        // rotate so that work[i] is the block of rank (r + i) mod n
        const size_t blk = t.count * es;
        for (int i = 0; i < n; ++i) memcpy(work.data() + (size_t)i * blk, (const char*)t.send + (size_t)((r + i) % n) * blk, blk);
        premulInto(work.data(), total, t.type, od);
        NCCLCHECK(logStepReduceScatter(comm, work.data(), t.count, es, t.type, od.hop));
        memcpy(t.recv, work.data(), blk);
        if (od.postscale) hostScale(t.recv, t.count, t.type, od.scale, od.intDiv);
        break;
      }
      memcpy(work.data(), t.send, total * es);
      premulInto(work.data(), total, t.type, od);
      Chunks ch{total, n};  // equal chunks of t.count
      if (n > 1) NCCLCHECK(ringReduceScatterInPlace(comm, work.data(), ch, es, t.type, od.hop, 0));
      memcpy(t.recv, work.data() + (size_t)r * t.count * es, t.count * es);
      if (od.postscale) hostScale(t.recv, t.count, t.type, od.scale, od.intDiv);
    } break;
    case FUNC_ALLGATHER: {
      char* out = (char*)t.recv;
      if (hp->collnet && n > 1 && out + (size_t)r * t.count * es != t.send && collNetAllGather(comm, hp->collnet, t.send, out, t.count * es) == ncclSuccess) break;
      if (useLogStep(comm, t.count * es)) {
        const size_t blk = t.count * es;
        std::vector<char> work((size_t)n * blk);
        memcpy(work.data(), t.send, blk);
        NCCLCHECK(logStepAllGather(comm, work.data(), blk));
        for (int i = 0; i < n; ++i) memcpy(out + (size_t)((r + i) % n) * blk, work.data() + (size_t)i * blk, blk);
        break;
      }
      if (out + (size_t)r * t.count * es != t.send) memcpy(out + (size_t)r * t.count * es, t.send, t.count * es);
      Chunks ch{t.count * n, n};
      if (n > 1) NCCLCHECK(ringAllGatherInPlace(comm, out, ch, es, 0));
    } break;
    case FUNC_BROADCAST: {
      // binomial tree rooted at t.root: in round k every rank that already has the data sends it 2^k positions on
      const size_t bytes = t.count * es;
      const int rel = (r - t.root + n) % n;
      if (r == t.root && t.recv != t.send) memcpy(t.recv, t.send, bytes);
      const void* have = r == t.root ? t.send : t.recv;
      int mask = 1;
      while (mask < n) {                      // receive from the parent: the lowest set bit of rel names it
        if (rel & mask) {
          const int parent = (r - mask + n) % n;
          NCCLCHECK(exchange(hp, parent, nullptr, 0, parent, t.recv, bytes));
          break;
        }
        mask <<= 1;
      }
      for (mask >>= 1; mask > 0; mask >>= 1)   // then serve the children, farthest first
        if (rel + mask < n) {
          const int child = (r + mask) % n;
          NCCLCHECK(exchange(hp, child, have, bytes, child, nullptr, 0));
        }
    } break;
    case FUNC_REDUCE: {
      NCCLCHECK(resolveOp(comm, t, &od));
      // chain root+1 -> root+2 -> ... -> root, each hop adds its own contribution
      std::vector<char> acc(t.count * es);
      memcpy(acc.data(), t.send, t.count * es);
      premulInto(acc.data(), t.count, t.type, od);
      int pos = (r - t.root - 1 + n) % n;  // 0 = first in chain, n-1 = root
      int prev = (r - 1 + n) % n, next = (r + 1) % n;
      if (n > 1 && pos > 0) {
        hp->tmp.resize(t.count * es);
        NCCLCHECK(exchange(hp, prev, nullptr, 0, prev, hp->tmp.data(), t.count * es));
        hostReduceInto(acc.data(), hp->tmp.data(), t.count, t.type, od.hop);
      }
      if (n > 1 && pos < n - 1) NCCLCHECK(exchange(hp, next, acc.data(), t.count * es, next, nullptr, 0));
      if (r == t.root) {
        memcpy(t.recv, acc.data(), t.count * es);
        if (od.postscale) hostScale(t.recv, t.count, t.type, od.scale, od.intDiv);
      }
    } break;
    case FUNC_ALLTOALL: {
      size_t b = t.count * es;
      memcpy((char*)t.recv + (size_t)r * b, (const char*)t.send + (size_t)r * b, b);
      for (int s = 1; s < n; ++s) {
        int to = (r + s) % n, from = (r - s + n) % n;
        NCCLCHECK(exchange(hp, to, (const char*)t.send + (size_t)to * b, b, from, (char*)t.recv + (size_t)from * b, b));
      }
    } break;
    case FUNC_GATHER: {
      size_t b = t.count * es;
      if (r == t.root) {
        memcpy((char*)t.recv + (size_t)r * b, t.send, b);
        for (int p = 0; p < n; ++p) if (p != r) NCCLCHECK(exchange(hp, p, nullptr, 0, p, (char*)t.recv + (size_t)p * b, b));
      } else {
        NCCLCHECK(exchange(hp, t.root, t.send, b, t.root, nullptr, 0));
      }
    } break;
    case FUNC_SCATTER: {
      size_t b = t.count * es;
      if (r == t.root) {
        memcpy(t.recv, (const char*)t.send + (size_t)r * b, b);
        for (int p = 0; p < n; ++p) if (p != r) NCCLCHECK(exchange(hp, p, (const char*)t.send + (size_t)p * b, b, p, nullptr, 0));
      } else {
        NCCLCHECK(exchange(hp, t.root, nullptr, 0, t.root, t.recv, b));
      }
    } break;
    case FUNC_SEND: NCCLCHECK(exchange(hp, t.root, t.send, t.count * es, t.root, nullptr, 0)); break;
    case FUNC_RECV: NCCLCHECK(exchange(hp, t.root, nullptr, 0, t.root, t.recv, t.count * es)); break;
    default:
      WARN("host plane: %s is not available on host-memory communicators", funcName(t.func));
      return ncclInvalidUsage;
  }
  return ncclSuccess;
}

// A group of sends and receives progresses all at once so that any matching order works.
ncclResult_t hostPlaneRunP2pGroup(ncclComm* comm, const std::vector<Task>& tasks) {
  HostPlane* hp = comm->hostPlane;
  if (hp->shm) {
    std::vector<ShmOp> ops;
    std::vector<const Task*> sSelf, rSelf;
    for (auto& t : tasks) {
      size_t bytes = t.count * typeSize(t.type);
      if (t.root == comm->rank) { (t.func == FUNC_SEND ? sSelf : rSelf).push_back(&t); continue; }
      if (t.func == FUNC_SEND) ops.push_back(ShmOp{&hp->shmOut[t.root], (char*)t.send, bytes, 0, true});
      else if (t.func == FUNC_RECV) ops.push_back(ShmOp{&hp->shmIn[t.root], (char*)t.recv, bytes, 0, false});
    }
    if (sSelf.size() != rSelf.size()) { WARN("unmatched send/recv to self"); return ncclInvalidUsage; }
    for (size_t i = 0; i < sSelf.size(); ++i) memcpy(rSelf[i]->recv, sSelf[i]->send, sSelf[i]->count * typeSize(sSelf[i]->type));
    return shmRun(hp, ops);
  }
  if (hp->proxy) {
    std::vector<ProxyOp*> posted;
    std::vector<const Task*> sSelf, rSelf;
    for (auto& t : tasks) {
      size_t bytes = t.count * typeSize(t.type);
      if (t.root == comm->rank) { (t.func == FUNC_SEND ? sSelf : rSelf).push_back(&t); continue; }
      if (t.func == FUNC_SEND) posted.push_back(proxyPost(hp->proxy, true, t.root, (void*)t.send, bytes));
      else if (t.func == FUNC_RECV) posted.push_back(proxyPost(hp->proxy, false, t.root, t.recv, bytes));
    }
    if (sSelf.size() != rSelf.size()) { WARN("unmatched send/recv to self"); return ncclInvalidUsage; }
    for (size_t i = 0; i < sSelf.size(); ++i) memcpy(rSelf[i]->recv, sSelf[i]->send, sSelf[i]->count * typeSize(sSelf[i]->type));
    return proxyWait(hp->proxy, posted.data(), (int)posted.size());
  }
  std::vector<SockOp> ops;
  for (auto& t : tasks) {
    size_t bytes = t.count * typeSize(t.type);
    if (bytes > (size_t)INT32_MAX) { WARN("host plane: grouped p2p larger than 2 GiB"); return ncclInvalidArgument; }
    if (t.root == comm->rank) continue;  // self send/recv pairs are matched below
    if (t.func == FUNC_SEND) ops.push_back(SockOp{SOCK_OP_SEND, &hp->peer[t.root], (void*)t.send, (int)bytes, 0});
    else if (t.func == FUNC_RECV) ops.push_back(SockOp{SOCK_OP_RECV, &hp->peer[t.root], t.recv, (int)bytes, 0});
  }
  std::vector<const Task*> selfSend, selfRecv;
  for (auto& t : tasks) if (t.root == comm->rank) (t.func == FUNC_SEND ? selfSend : selfRecv).push_back(&t);
  if (selfSend.size() != selfRecv.size()) { WARN("unmatched send/recv to self"); return ncclInvalidUsage; }
  for (size_t i = 0; i < selfSend.size(); ++i)
    memcpy(selfRecv[i]->recv, selfSend[i]->send, selfSend[i]->count * typeSize(selfSend[i]->type));
  // Per-socket byte streams keep the order in which the ops were posted; progress them together.
  // sockMultiOp advances every op, but two ops on the same socket+direction must run in order.
  std::vector<SockOp> wave;
  std::vector<char> done(ops.size(), 0);
  size_t left = ops.size();
  while (left) {
    wave.clear();
    std::vector<size_t> idx;
    for (size_t i = 0; i < ops.size(); ++i) {
      if (done[i]) continue;
      bool clash = false;
      for (auto& w : wave) if (w.sock == ops[i].sock && w.kind == ops[i].kind) clash = true;
      if (clash) continue;
      wave.push_back(ops[i]);
      idx.push_back(i);
    }
    NCCLCHECK(sockMultiOp(wave.data(), (int)wave.size()));
    for (size_t i : idx) done[i] = 1;
    left -= idx.size();
  }
  return ncclSuccess;
}

}  // namespace b200
