// Example network plugin: ncclNet_v12 over UNIX-domain stream sockets (abstract namespace), for
// ranks of one host. It shows the contract a backend must meet: listen() fills an opaque handle,
// connect()/accept() may return a NULL comm ("call again"), isend()/irecv() only queue work and
// test() makes progress without blocking. Messages are an 8-byte length plus payload.
// Reference parity: plugins/net/example/plugin.c (table layout and call contract).
#include <errno.h>
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <deque>

#include "plugin/nccl_net.h"

namespace {

std::atomic<int> gSeq{0};
ncclDebugLogger_t gLog = nullptr;

struct Handle { char name[64]; };
struct Listen { int fd; };
struct Req;
struct Comm { int fd; std::deque<Req*> q; };
struct Req {
  Comm* c;
  bool send;
  char* data;
  uint64_t size, header, off = 0;
  int hoff = 0;
};

void nonblock(int fd) { fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK); }

socklen_t fill(sockaddr_un* sa, const char* name) {
  memset(sa, 0, sizeof(*sa));
  sa->sun_family = AF_UNIX;
  size_t n = strlen(name);
  memcpy(sa->sun_path + 1, name, n);   // leading NUL: abstract namespace, nothing to unlink
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

ncclResult_t nInit(void** ctx, uint64_t, ncclNetCommConfig_t*, ncclDebugLogger_t log, ncclProfilerCallback_t) {
  gLog = log;
  if (ctx) *ctx = nullptr;
  return ncclSuccess;
}
ncclResult_t nDevices(int* n) { *n = 1; return ncclSuccess; }
ncclResult_t nProps(int dev, ncclNetProperties_t* p) {
  if (dev != 0) return ncclInvalidArgument;
  memset(p, 0, sizeof(*p));
  static char name[] = "unix0";
  p->name = name;
  p->ptrSupport = NCCL_PTR_HOST;
  p->speed = 100000;
  p->maxComms = 65536;
  p->maxRecvs = 1;
  p->netDeviceType = NCCL_NET_DEVICE_HOST;
  p->vProps.ndevs = 1;
  p->maxP2pBytes = (size_t)1 << 40;
  p->maxCollBytes = (size_t)1 << 30;
  p->maxMultiRequestSize = 1;
  p->railId = p->planeId = -1;
  return ncclSuccess;
}
ncclResult_t nListen(void*, int, void* handle, void** lc) {
  Handle h;
  memset(&h, 0, sizeof(h));
  snprintf(h.name, sizeof(h.name), "nccl-unix-net-%d-%d", (int)getpid(), gSeq++);
  int fd = socket(AF_UNIX, SOCK_STREAM, 0);
  if (fd < 0) return ncclSystemError;
  sockaddr_un sa;
  socklen_t len = fill(&sa, h.name);
  if (bind(fd, (sockaddr*)&sa, len) != 0 || listen(fd, 1024) != 0) { close(fd); return ncclSystemError; }
  nonblock(fd);
  memset(handle, 0, NCCL_NET_HANDLE_MAXSIZE);
  memcpy(handle, &h, sizeof(h));
  *lc = new Listen{fd};
  return ncclSuccess;
}
ncclResult_t nConnect(void*, int, void* handle, void** sc, ncclNetDeviceHandle_t** dh) {
  Handle h;
  memcpy(&h, handle, sizeof(h));
  *sc = nullptr;
  if (dh) *dh = nullptr;
  int fd = socket(AF_UNIX, SOCK_STREAM, 0);
  if (fd < 0) return ncclSystemError;
  sockaddr_un sa;
  socklen_t len = fill(&sa, h.name);
  if (connect(fd, (sockaddr*)&sa, len) != 0) {
    int e = errno;
    close(fd);
    return (e == ECONNREFUSED || e == EAGAIN || e == ENOENT) ? ncclSuccess : ncclSystemError;   // not yet: the caller retries
  }
  nonblock(fd);
  *sc = new Comm{fd, {}};
  return ncclSuccess;
}
ncclResult_t nAccept(void* lc, void** rc, ncclNetDeviceHandle_t** dh) {
  *rc = nullptr;
  if (dh) *dh = nullptr;
  int fd = accept(((Listen*)lc)->fd, nullptr, nullptr);
  if (fd < 0) return (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) ? ncclSuccess : ncclSystemError;
  nonblock(fd);
  *rc = new Comm{fd, {}};
  return ncclSuccess;
}
ncclResult_t nRegMr(void*, void*, size_t, int type, void** mh) { *mh = nullptr; return type == NCCL_PTR_HOST ? ncclSuccess : ncclInvalidArgument; }
ncclResult_t nRegMrDmaBuf(void*, void*, size_t, int, uint64_t, int, void**) { return ncclInvalidUsage; }
ncclResult_t nDeregMr(void*, void*) { return ncclSuccess; }
ncclResult_t nIsend(void* sc, void* data, size_t size, int, void*, void*, void** req) {
  Req* r = new Req{(Comm*)sc, true, (char*)data, size, size};
  r->c->q.push_back(r);
  *req = r;
  return ncclSuccess;
}
ncclResult_t nIrecv(void* rc, int n, void** data, size_t* sizes, int*, void**, void**, void** req) {
  if (n != 1) return ncclInvalidArgument;
  Req* r = new Req{(Comm*)rc, false, (char*)data[0], sizes[0], 0};
  r->c->q.push_back(r);
  *req = r;
  return ncclSuccess;
}
ncclResult_t nIflush(void*, int, void**, int*, void**, void** req) { *req = nullptr; return ncclSuccess; }

// moves bytes without blocking; returns false on a broken connection
bool move(Req* r, char* p, uint64_t want, uint64_t* off) {
  while (*off < want) {
    ssize_t k = r->send ? send(r->c->fd, p + *off, want - *off, MSG_NOSIGNAL | MSG_DONTWAIT) : recv(r->c->fd, p + *off, want - *off, MSG_DONTWAIT);
    if (k > 0) { *off += (uint64_t)k; continue; }
    if (k < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) return true;
    return false;
  }
  return true;
}
ncclResult_t nTest(void* req, int* done, int* sizes) {
  *done = 0;
  Req* r = (Req*)req;
  if (!r) { *done = 1; return ncclSuccess; }
  if (r->c->q.front() != r) return ncclSuccess;
  if (r->hoff < 8) {
    uint64_t ho = (uint64_t)r->hoff;
    if (!move(r, (char*)&r->header, 8, &ho)) return ncclRemoteError;
    r->hoff = (int)ho;
    if (r->hoff < 8) return ncclSuccess;
    if (!r->send) {
      if (r->header > r->size) return ncclInternalError;
      r->size = r->header;
    }
  }
  if (!move(r, r->data, r->size, &r->off)) return ncclRemoteError;
  if (r->off < r->size) return ncclSuccess;
  *done = 1;
  if (sizes) sizes[0] = (int)r->size;
  r->c->q.pop_front();
  delete r;
  return ncclSuccess;
}
ncclResult_t nCloseComm(void* c) {
  Comm* k = (Comm*)c;
  if (k) {
    for (Req* r : k->q) delete r;
    close(k->fd);
    delete k;
  }
  return ncclSuccess;
}
ncclResult_t nCloseListen(void* l) {
  if (l) { close(((Listen*)l)->fd); delete (Listen*)l; }
  return ncclSuccess;
}
ncclResult_t nGetDeviceMr(void*, void*, void**) { return ncclInvalidUsage; }
ncclResult_t nIrecvConsumed(void*, int, void*) { return ncclSuccess; }
ncclResult_t nMakeVDevice(int*, ncclNetVDeviceProps_t*) { return ncclInvalidUsage; }
ncclResult_t nFinalize(void*) { return ncclSuccess; }
ncclResult_t nSetNetAttr(void*, ncclNetAttr_t*) { return ncclSuccess; }

}  // namespace

// -DUNIX_NET_ABI=8|9|10|11 builds the same backend behind an earlier interface instead (one table per
// library), which is how the library's adapters for deployed older plugins are tested.
#ifndef UNIX_NET_ABI
#define UNIX_NET_ABI 12
#endif
#define EXPORT extern "C" __attribute__((visibility("default")))

#if UNIX_NET_ABI == 12
EXPORT const ncclNet_v12_t ncclNetPlugin_v12 = {
    "UnixExample", nInit, nDevices, nProps, nListen, nConnect, nAccept, nRegMr, nRegMrDmaBuf, nDeregMr, nIsend, nIrecv, nIflush, nTest,
    nCloseComm, nCloseComm, nCloseListen, nGetDeviceMr, nIrecvConsumed, nMakeVDevice, nFinalize, nSetNetAttr};
#else
#include "plugin/nccl_net_compat.h"
namespace {
template <typename P> ncclResult_t oldProps(int dev, P* p) {
  ncclNetProperties_t full;
  ncclResult_t r = nProps(dev, &full);
  if (r != ncclSuccess) return r;
  memset(p, 0, sizeof(*p));
  p->name = full.name; p->pciPath = full.pciPath; p->guid = full.guid; p->ptrSupport = full.ptrSupport; p->regIsGlobal = full.regIsGlobal;
  p->speed = full.speed; p->port = full.port; p->latency = full.latency; p->maxComms = full.maxComms; p->maxRecvs = full.maxRecvs;
  p->netDeviceType = full.netDeviceType; p->netDeviceVersion = full.netDeviceVersion;
  return ncclSuccess;
}
template <typename P> ncclResult_t oldProps9(int dev, P* p) {
  ncclResult_t r = oldProps(dev, p);
  if (r == ncclSuccess) { p->vProps.ndevs = 1; p->vProps.devs[0] = dev; p->maxP2pBytes = (size_t)1 << 40; p->maxCollBytes = (size_t)1 << 40; }
  return r;
}
ncclResult_t oInitLog(ncclDebugLogger_t log) { return nInit(nullptr, 0, nullptr, log, nullptr); }
ncclResult_t oInitLogProf(ncclDebugLogger_t log, ncclProfilerCallback_t prof) { return nInit(nullptr, 0, nullptr, log, prof); }
ncclResult_t oListen(int dev, void* h, void** lc) { return nListen(nullptr, dev, h, lc); }
ncclResult_t oConnect(int dev, void* h, void** sc, ncclNetDeviceHandle_t** dh) { return nConnect(nullptr, dev, h, sc, dh); }
ncclResult_t oConnectCfg(int dev, ncclNetCommConfig_t*, void* h, void** sc, ncclNetDeviceHandle_t** dh) { return nConnect(nullptr, dev, h, sc, dh); }
ncclResult_t oIsend9(void* sc, void* d, size_t n, int tag, void* mh, void** req) { return nIsend(sc, d, n, tag, mh, nullptr, req); }
ncclResult_t oIrecv9(void* rc, int n, void** d, size_t* sz, int* tags, void** mhs, void** req) { return nIrecv(rc, n, d, sz, tags, mhs, nullptr, req); }
ncclResult_t oIsend8(void* sc, void* d, int n, int tag, void* mh, void** req) { return nIsend(sc, d, (size_t)n, tag, mh, nullptr, req); }
ncclResult_t oIrecv8(void* rc, int n, void** d, int* sz, int* tags, void** mhs, void** req) {
  size_t wide[NCCL_NET_MAX_REQUESTS];
  for (int i = 0; i < n; ++i) wide[i] = (size_t)sz[i];
  return nIrecv(rc, n, d, wide, tags, mhs, nullptr, req);
}
}  // namespace
#if UNIX_NET_ABI == 11
EXPORT const ncclNet_v11_t ncclNetPlugin_v11 = {
    "UnixExample", nInit, nDevices, oldProps9<ncclNetProperties_v11_t>, nListen, nConnect, nAccept, nRegMr, nRegMrDmaBuf, nDeregMr, nIsend, nIrecv,
    nIflush, nTest, nCloseComm, nCloseComm, nCloseListen, nGetDeviceMr, nIrecvConsumed, nMakeVDevice, nFinalize, nSetNetAttr};
#elif UNIX_NET_ABI == 10
EXPORT const ncclNet_v10_t ncclNetPlugin_v10 = {
    "UnixExample", oInitLogProf, nDevices, oldProps9<ncclNetProperties_v10_t>, oListen, oConnectCfg, nAccept, nRegMr, nRegMrDmaBuf, nDeregMr, nIsend,
    nIrecv, nIflush, nTest, nCloseComm, nCloseComm, nCloseListen, nGetDeviceMr, nIrecvConsumed, nMakeVDevice};
#elif UNIX_NET_ABI == 9
EXPORT const ncclNet_v9_t ncclNetPlugin_v9 = {
    "UnixExample", oInitLog, nDevices, oldProps9<ncclNetProperties_v9_t>, oListen, oConnect, nAccept, nRegMr, nRegMrDmaBuf, nDeregMr, oIsend9, oIrecv9,
    nIflush, nTest, nCloseComm, nCloseComm, nCloseListen, nGetDeviceMr, nIrecvConsumed, nMakeVDevice};
#elif UNIX_NET_ABI == 8
EXPORT const ncclNet_v8_t ncclNetPlugin_v8 = {
    "UnixExample", oInitLog, nDevices, oldProps<ncclNetProperties_v8_t>, oListen, oConnect, nAccept, nRegMr, nRegMrDmaBuf, nDeregMr, oIsend8, oIrecv8,
    nIflush, nTest, nCloseComm, nCloseComm, nCloseListen, nGetDeviceMr, nIrecvConsumed};
#else
#error "UNIX_NET_ABI must be 8, 9, 10, 11 or 12"
#endif
#endif

#ifdef UNIX_NET_GIN
// With -DUNIX_NET_GIN the library also exports a table for GPU-initiated networking: enough of it for a loader to learn
// what the plugin offers (one device, plain signals); the data entry points report that nothing is connected.
#include "plugin/nccl_gin.h"
static ncclResult_t gInit(void** ctx, uint64_t, ncclDebugLogger_t) { *ctx = (void*)1; return ncclSuccess; }
static ncclResult_t gDevices(int* n) { *n = 1; return ncclSuccess; }
static ncclResult_t gProps(ncclGinProperties_v14_t* p) { p->supportsStrongSignals = true; p->supportsVASignals = false; return ncclSuccess; }
static ncclResult_t gNetProps(int dev, ncclNetProperties_t* p) { return nProps(dev, p); }
static ncclResult_t gListen(void*, int, void*, void**) { return ncclInternalError; }
static ncclResult_t gConnect(void*, void*[], int, int, void*, void**) { return ncclInternalError; }
static ncclResult_t gCreate(void*, ncclGinConfig_v14_t*, void**, void**) { return ncclInternalError; }
static ncclResult_t gReg(void*, void*, size_t, int, uint64_t, void**, void**) { return ncclInternalError; }
static ncclResult_t gRegDma(void*, void*, size_t, int, uint64_t, int, uint64_t, void**, void**) { return ncclInternalError; }
static ncclResult_t gClose(void*) { return ncclSuccess; }
static ncclResult_t gDeReg(void*, void*) { return ncclSuccess; }
static ncclResult_t gErr(void*, bool* e) { *e = false; return ncclSuccess; }
EXPORT const ncclGin_v14_t ncclGinPlugin_v14 = {"UnixExampleGin", gInit, gDevices, gProps, gNetProps, gListen, gConnect, gCreate, gReg, gRegDma, gDeReg,
                                                gClose, gClose, gClose, gClose, gErr, gClose};
#endif
