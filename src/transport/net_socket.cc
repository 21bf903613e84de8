// Built-in network backend "Socket": the ncclNet_t table over TCP.
// A send / receive pair has one TCP connection, or several (NCCL_SOCKET_NTHREADS x NCCL_NSOCKS_PERTHREAD): a message travels as
// an 8-byte length on the first connection followed by the payload, cut into equal parts over the connections when it is
// larger than 64 KiB. isend / irecv only record the request and test() moves whatever the kernel accepts without blocking, so one
// proxy thread keeps many transfers and all connections in flight (no helper threads are created). Connections of several
// dialling comms may reach a listener interleaved; each announces its comm with a token in its first bytes.
// Reference parity: src/transport/net_socket.cc (devices/properties :50-346, listen/connect/accept :408-540, test :608-720,
// isend/irecv :757; multi-socket striping with its two variables).
#include <string.h>

#include <atomic>
#include <deque>
#include <map>
#include <unistd.h>

#include "../core/socket.h"
#include "net.h"

namespace b200 {

B200_PARAM(SocketNthreads, "SOCKET_NTHREADS", 1, "With NCCL_NSOCKS_PERTHREAD: their product is the number of TCP connections per send / receive pair of the socket backend (1 to 16); no extra threads are created, the proxy thread moves all of them")
B200_PARAM(NsocksPerThread, "NSOCKS_PERTHREAD", 1, "See NCCL_SOCKET_NTHREADS")

namespace {

constexpr int kMaxIfs = 16;
constexpr uint64_t kNetSocketMagic = 0x4e45545342323030ull;   // "NETSB200"

struct Devices {
  int n = -1;
  char names[kMaxIfs][64];
  SockAddr addrs[kMaxIfs];
};
Devices gDevs;
std::mutex gDevLock;

void loadDevices() {
  std::lock_guard<std::mutex> g(gDevLock);
  if (gDevs.n >= 0) return;
  gDevs.n = findInterfaces(gDevs.names, gDevs.addrs, kMaxIfs);
  if (gDevs.n < 0) gDevs.n = 0;
}

struct Handle {            // what listen() hands to the sender; fits NCCL_NET_HANDLE_MAXSIZE
  SockAddr addr;
  uint64_t magic;
};
static_assert(sizeof(Handle) <= NCCL_NET_HANDLE_MAXSIZE, "handle too large");

struct Request;
struct Comm {
  Socket sock;                  // first connection: carries the 8-byte length of every message and the first part of its payload
  std::vector<Socket> extra;    // further connections of the same comm (NCCL_SOCKET_NTHREADS x NCCL_NSOCKS_PERTHREAD in all)
  bool isSend;
  std::deque<Request*> queue;   // requests share the byte streams: only the oldest may move bytes
  int nSocks() const { return 1 + (int)extra.size(); }
  Socket* socket(int i) { return i == 0 ? &sock : &extra[i - 1]; }
};
struct Hello { uint64_t token; int32_t index, total; };   // first bytes on every connection: which comm it belongs to
struct Partial { Comm* comm; int have; };
struct ListenComm {
  Socket sock;
  std::map<uint64_t, Partial> partial;   // comms whose connections have not all arrived yet
};
constexpr int kMaxSocks = 16;
constexpr uint64_t kMinPart = 64 << 10;   // smaller messages travel on the first connection only
struct Request {
  Comm* comm;
  bool isSend;
  char* data;
  uint64_t size;        // send: bytes to send; recv: capacity, then bytes received
  uint64_t header;
  int headerOff = 0;
  uint64_t off[kMaxSocks] = {};   // bytes moved per connection
  bool headerDone = false;
  void* prof = nullptr;                       // event of this request at the profiler (through the callback given at init)
  ncclProfilerNetSockDescr_v1_t profDescr;
};

ncclProfilerCallback_t gProf = nullptr;
void profRequest(Request* r, void* phandle) {
  if (!gProf || !phandle) return;
  r->profDescr.type = ncclProfileSocket;
  r->profDescr.sock.fd = r->comm->sock.fd;
  r->profDescr.sock.op = r->isSend ? 0 : 1;
  r->profDescr.sock.length = r->size;
  gProf(&r->prof, ncclProfilerNetEventStart, phandle, NCCL_PROFILER_NET_TYPE_SOCK | NCCL_PROFILER_NET_SOCKET_VER, &r->profDescr);
}

ncclResult_t sInit(void** ctx, uint64_t, ncclNetCommConfig_t*, ncclDebugLogger_t, ncclProfilerCallback_t prof) {
  if (prof) gProf = prof;
  loadDevices();
  if (ctx) *ctx = nullptr;
  return ncclSuccess;
}
ncclResult_t sDevices(int* ndev) { loadDevices(); *ndev = gDevs.n; return ncclSuccess; }

ncclResult_t sGetProperties(int dev, ncclNetProperties_t* p) {
  loadDevices();
  if (dev < 0 || dev >= gDevs.n) return ncclInvalidArgument;
  memset(p, 0, sizeof(*p));
  p->name = gDevs.names[dev];
  p->pciPath = nullptr;
  p->guid = dev;
  p->ptrSupport = NCCL_PTR_HOST;
  p->regIsGlobal = 0;
  p->speed = strcmp(gDevs.names[dev], "lo") == 0 ? 100000 : 10000;
  p->port = 0;
  p->latency = 0;
  p->maxComms = 65536;
  p->maxRecvs = 1;
  p->netDeviceType = NCCL_NET_DEVICE_HOST;
  p->netDeviceVersion = 0;
  p->vProps.ndevs = 1;
  p->vProps.devs[0] = dev;
  p->maxP2pBytes = (size_t)1 << 40;
  p->maxCollBytes = (size_t)1 << 30;
  p->maxMultiRequestSize = 1;
  p->railId = -1;
  p->planeId = -1;
  return ncclSuccess;
}

ncclResult_t sListen(void*, int dev, void* handle, void** listenComm) {
  loadDevices();
  if (dev < 0 || dev >= gDevs.n) return ncclInvalidArgument;
  ListenComm* l = new ListenComm;
  NCCLCHECK(sockInit(&l->sock, &gDevs.addrs[dev], kNetSocketMagic, SOCK_NET));
  ncclResult_t r = sockListen(&l->sock);
  if (r != ncclSuccess) { delete l; return r; }
  Handle h;
  memset(&h, 0, sizeof(h));
  h.addr = l->sock.addr;
  h.magic = kNetSocketMagic;
  memset(handle, 0, NCCL_NET_HANDLE_MAXSIZE);
  memcpy(handle, &h, sizeof(h));
  *listenComm = l;
  return ncclSuccess;
}

// How a message of `size` bytes is cut over `n` connections: equal parts of at least kMinPart, rounded up to 4 KiB; both
// ends compute the same cut from the size in the header.
inline uint64_t partBytes(uint64_t size, int n) {
  if (n <= 1 || size <= kMinPart) return size;
  uint64_t per = std::max<uint64_t>((size + n - 1) / n, kMinPart);
  return (per + 4095) & ~(uint64_t)4095;
}

ncclResult_t sConnect(void*, int, void* handle, void** sendComm, ncclNetDeviceHandle_t** devComm) {
  Handle h;
  memcpy(&h, handle, sizeof(h));
  Comm* c = new Comm;
  c->isSend = true;
  const int total = (int)std::min<int64_t>(std::max<int64_t>(paramSocketNthreads() * paramNsocksPerThread(), 1), kMaxSocks);
  static std::atomic<uint64_t> counter{0};
  const uint64_t token = ((uint64_t)getpid() << 40) ^ ((uint64_t)(uintptr_t)c << 8) ^ ++counter;
  c->extra.resize(total - 1);
  ncclResult_t r = ncclSuccess;
  for (int i = 0; i < total && r == ncclSuccess; ++i) {
    Socket* sk = c->socket(i);
    r = sockInit(sk, &h.addr, h.magic, SOCK_NET);
    if (r == ncclSuccess) r = sockConnect(sk);
    Hello hello = {token, i, total};
    if (r == ncclSuccess) r = sockSend(sk, &hello, sizeof(hello));
  }
  if (r != ncclSuccess) { for (int i = 0; i < total; ++i) sockClose(c->socket(i)); delete c; return r; }
  *sendComm = c;
  if (devComm) *devComm = nullptr;
  return ncclSuccess;
}

ncclResult_t sAccept(void* listenComm, void** recvComm, ncclNetDeviceHandle_t** devComm) {
  ListenComm* l = (ListenComm*)listenComm;
  if (devComm) *devComm = nullptr;
  // connections of several dialling comms may arrive interleaved: they are sorted by the token in their first bytes until one
  // comm has all of its connections
  for (;;) {
    Socket sk;
    NCCLCHECK(sockAccept(&sk, &l->sock));
    Hello hello;
    ncclResult_t r = sockRecv(&sk, &hello, sizeof(hello));
    if (r != ncclSuccess || hello.total < 1 || hello.total > kMaxSocks || hello.index < 0 || hello.index >= hello.total) { sockClose(&sk); if (r != ncclSuccess) return r; continue; }
    Partial& pa = l->partial[hello.token];
    if (!pa.comm) {
      pa.comm = new Comm;
      pa.comm->isSend = false;
      pa.comm->extra.resize(hello.total - 1);
      pa.have = 0;
    }
    if (pa.comm->nSocks() != hello.total) { sockClose(&sk); continue; }
    *pa.comm->socket(hello.index) = sk;
    if (++pa.have == hello.total) {
      *recvComm = pa.comm;
      l->partial.erase(hello.token);
      return ncclSuccess;
    }
  }
}

ncclResult_t sRegMr(void*, void*, size_t, int type, void** mhandle) {
  if (type != NCCL_PTR_HOST) return ncclInvalidArgument;   // TCP reads and writes host memory only
  *mhandle = nullptr;
  return ncclSuccess;
}
ncclResult_t sRegMrDmaBuf(void*, void*, size_t, int, uint64_t, int, void**) { return ncclInvalidUsage; }
ncclResult_t sDeregMr(void*, void*) { return ncclSuccess; }

ncclResult_t sIsend(void* sendComm, void* data, size_t size, int, void*, void* phandle, void** request) {
  Request* r = new Request;
  r->comm = (Comm*)sendComm;
  r->isSend = true;
  r->data = (char*)data;
  r->size = size;
  r->header = size;
  r->comm->queue.push_back(r);
  profRequest(r, phandle);
  *request = r;
  return ncclSuccess;
}

ncclResult_t sIrecv(void* recvComm, int n, void** data, size_t* sizes, int*, void**, void** phandles, void** request) {
  if (n != 1) return ncclInvalidArgument;
  Request* r = new Request;
  r->comm = (Comm*)recvComm;
  r->isSend = false;
  r->data = (char*)data[0];
  r->size = sizes[0];
  r->header = 0;
  r->comm->queue.push_back(r);
  profRequest(r, phandles ? phandles[0] : nullptr);
  *request = r;
  return ncclSuccess;
}

ncclResult_t sIflush(void*, int, void**, int*, void**, void** request) { *request = nullptr; return ncclSuccess; }

ncclResult_t sTest(void* request, int* done, int* sizes) {
  Request* r = (Request*)request;
  *done = 0;
  if (!r) { *done = 1; return ncclSuccess; }
  if (r->comm->queue.front() != r) return ncclSuccess;
  const SockOpKind kind = r->isSend ? SOCK_OP_SEND : SOCK_OP_RECV;
  if (!r->headerDone) {
    NCCLCHECK(sockProgress(kind, &r->comm->sock, &r->header, 8, &r->headerOff));
    if (r->headerOff < 8) return ncclSuccess;
    r->headerDone = true;
    if (!r->isSend) {
      if (r->header > r->size) { WARN("net socket: message of %llu bytes does not fit the posted %llu", (unsigned long long)r->header, (unsigned long long)r->size); return ncclInternalError; }
      r->size = r->header;
    }
  }
  const int n = r->comm->nSocks();
  const uint64_t per = partBytes(r->size, n);
  bool all = true;
  for (int i = 0; i < n; ++i) {
    const uint64_t lo = std::min<uint64_t>(r->size, (uint64_t)i * per), len = std::min<uint64_t>(per, r->size - lo);
    while (r->off[i] < len) {
      int chunk = (int)std::min<uint64_t>(len - r->off[i], 1u << 30), moved = 0;
      NCCLCHECK(sockProgress(kind, r->comm->socket(i), r->data + lo + r->off[i], chunk, &moved));
      r->off[i] += moved;
      if (moved < chunk) { all = false; break; }
    }
  }
  if (!all) return ncclSuccess;
  *done = 1;
  if (sizes) sizes[0] = (int)std::min<uint64_t>(r->size, 0x7fffffff);
  r->comm->queue.pop_front();
  if (r->prof && gProf) gProf(&r->prof, ncclProfilerNetEventStop, nullptr, 0, nullptr);
  delete r;
  return ncclSuccess;
}

ncclResult_t sCloseComm(void* comm) {
  Comm* c = (Comm*)comm;
  if (c) {
    for (Request* r : c->queue) { if (r->prof && gProf) gProf(&r->prof, ncclProfilerNetEventStop, nullptr, 0, nullptr); delete r; }
    for (int i = 0; i < c->nSocks(); ++i) sockClose(c->socket(i));
    delete c;
  }
  return ncclSuccess;
}
ncclResult_t sCloseListen(void* listenComm) {
  ListenComm* l = (ListenComm*)listenComm;
  if (l) {
    for (auto& kv : l->partial) { for (int i = 0; i < kv.second.comm->nSocks(); ++i) sockClose(kv.second.comm->socket(i)); delete kv.second.comm; }
    sockClose(&l->sock);
    delete l;
  }
  return ncclSuccess;
}
ncclResult_t sGetDeviceMr(void*, void*, void**) { return ncclInvalidUsage; }
ncclResult_t sIrecvConsumed(void*, int, void*) { return ncclSuccess; }
ncclResult_t sMakeVDevice(int*, ncclNetVDeviceProps_t*) { return ncclInvalidUsage; }
ncclResult_t sFinalize(void*) { return ncclSuccess; }
ncclResult_t sSetNetAttr(void*, ncclNetAttr_t*) { return ncclSuccess; }

}  // namespace

ncclNet_t netSocketBackend = {"Socket", sInit, sDevices, sGetProperties, sListen, sConnect, sAccept, sRegMr, sRegMrDmaBuf, sDeregMr, sIsend, sIrecv,
                              sIflush, sTest, sCloseComm, sCloseComm, sCloseListen, sGetDeviceMr, sIrecvConsumed, sMakeVDevice, sFinalize, sSetNetAttr};

}  // namespace b200
