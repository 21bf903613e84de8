// Adapters that present a network plugin of an earlier interface (v8 ... v11) as the newest table.
// One plugin library is loaded per process, so each adapter keeps the old table in a static and the
// adapter functions are plain C functions that forward with the arguments the old version takes:
//   v11  properties are widened (rail / plane ids unknown: -1)
//   v10  no per-communicator context: the adapter's context remembers the traffic class for connect()
//   v9   no profiler callback and no profiler handles
//   v8   sizes are ints (messages are cut at 2 GiB - 1 by maxP2pBytes), no virtual devices
// Reference parity: src/plugin/net/net_v8.cc ... net_v11.cc.
#include <limits.h>

#include "plugin/nccl_net_compat.h"
#include "plugin.h"

namespace b200 {

static ncclNet_v11_t* g11;
static ncclNet_v10_t* g10;
static ncclNet_v9_t* g9;
static ncclNet_v8_t* g8;
static ncclNet_t gShim;
static char gShimName[64];

struct OldCtx { ncclNetCommConfig_t cfg; };   // what init() received, for interfaces that want it later

template <typename P> static void widenCommon(const P& o, ncclNetProperties_t* p) {
  memset(p, 0, sizeof(*p));
  p->name = o.name; p->pciPath = o.pciPath; p->guid = o.guid; p->ptrSupport = o.ptrSupport; p->regIsGlobal = o.regIsGlobal;
  p->speed = o.speed; p->port = o.port; p->latency = o.latency; p->maxComms = o.maxComms; p->maxRecvs = o.maxRecvs;
  p->netDeviceType = o.netDeviceType; p->netDeviceVersion = o.netDeviceVersion;
  p->vProps.ndevs = 1;
  p->maxP2pBytes = INT_MAX; p->maxCollBytes = INT_MAX; p->maxMultiRequestSize = 1;
  p->railId = -1; p->planeId = -1;
}
template <typename P> static void widenV9(const P& o, ncclNetProperties_t* p) {
  widenCommon(o, p);
  p->forceFlush = o.forceFlush; p->vProps = o.vProps; p->maxP2pBytes = o.maxP2pBytes; p->maxCollBytes = o.maxCollBytes;
}

// ------------------------------------------------------------------ v11
static ncclResult_t v11Props(int dev, ncclNetProperties_t* p) {
  ncclNetProperties_v11_t o;
  memset(&o, 0, sizeof(o));
  ncclResult_t r = g11->getProperties(dev, &o);
  if (r != ncclSuccess) return r;
  widenV9(o, p);
  p->maxMultiRequestSize = o.maxMultiRequestSize;
  return ncclSuccess;
}

// ------------------------------------------------------------------ v10 / v9 / v8 share the context-free shape
static ncclResult_t oldInit(void** ctx, uint64_t, ncclNetCommConfig_t* cfg, ncclDebugLogger_t log, ncclProfilerCallback_t prof) {
  OldCtx* c = new OldCtx;
  c->cfg.trafficClass = cfg ? cfg->trafficClass : NCCL_NET_TRAFFIC_CLASS_UNDEF;
  *ctx = c;
  if (g10) return g10->init(log, prof);
  if (g9) return g9->init(log);
  return g8->init(log);
}
static ncclResult_t oldFinalize(void* ctx) { delete (OldCtx*)ctx; return ncclSuccess; }
static ncclResult_t oldDevices(int* n) { return g10 ? g10->devices(n) : g9 ? g9->devices(n) : g8->devices(n); }
static ncclResult_t oldProps(int dev, ncclNetProperties_t* p) {
  if (g8) {
    ncclNetProperties_v8_t o;
    memset(&o, 0, sizeof(o));
    ncclResult_t r = g8->getProperties(dev, &o);
    if (r == ncclSuccess) { widenCommon(o, p); p->vProps.devs[0] = dev; }
    return r;
  }
  ncclNetProperties_v9_t o;
  memset(&o, 0, sizeof(o));
  ncclResult_t r = g10 ? g10->getProperties(dev, &o) : g9->getProperties(dev, &o);
  if (r == ncclSuccess) widenV9(o, p);
  return r;
}
static ncclResult_t oldListen(void*, int dev, void* handle, void** lc) {
  return g10 ? g10->listen(dev, handle, lc) : g9 ? g9->listen(dev, handle, lc) : g8->listen(dev, handle, lc);
}
static ncclResult_t oldConnect(void* ctx, int dev, void* handle, void** sc, ncclNetDeviceHandle_t** dh) {
  if (g10) return g10->connect(dev, ctx ? &((OldCtx*)ctx)->cfg : nullptr, handle, sc, dh);
  return g9 ? g9->connect(dev, handle, sc, dh) : g8->connect(dev, handle, sc, dh);
}
static ncclResult_t oldAccept(void* lc, void** rc, ncclNetDeviceHandle_t** dh) {
  return g10 ? g10->accept(lc, rc, dh) : g9 ? g9->accept(lc, rc, dh) : g8->accept(lc, rc, dh);
}
static ncclResult_t oldRegMr(void* c, void* d, size_t s, int t, void** m) {
  return g10 ? g10->regMr(c, d, s, t, m) : g9 ? g9->regMr(c, d, s, t, m) : g8->regMr(c, d, s, t, m);
}
static ncclResult_t oldRegMrDmaBuf(void* c, void* d, size_t s, int t, uint64_t off, int fd, void** m) {
  return g10 ? g10->regMrDmaBuf(c, d, s, t, off, fd, m) : g9 ? g9->regMrDmaBuf(c, d, s, t, off, fd, m) : g8->regMrDmaBuf(c, d, s, t, off, fd, m);
}
static ncclResult_t oldDeregMr(void* c, void* m) { return g10 ? g10->deregMr(c, m) : g9 ? g9->deregMr(c, m) : g8->deregMr(c, m); }
static ncclResult_t oldIsend(void* sc, void* data, size_t size, int tag, void* mh, void* ph, void** req) {
  if (g10) return g10->isend(sc, data, size, tag, mh, ph, req);
  if (g9) return g9->isend(sc, data, size, tag, mh, req);
  if (size > (size_t)INT_MAX) return ncclInternalError;   // maxP2pBytes told the caller to cut messages
  return g8->isend(sc, data, (int)size, tag, mh, req);
}
static ncclResult_t oldIrecv(void* rc, int n, void** data, size_t* sizes, int* tags, void** mhs, void** phs, void** req) {
  if (g10) return g10->irecv(rc, n, data, sizes, tags, mhs, phs, req);
  if (g9) return g9->irecv(rc, n, data, sizes, tags, mhs, req);
  int isz[NCCL_NET_MAX_REQUESTS];
  if (n > NCCL_NET_MAX_REQUESTS) return ncclInternalError;
  for (int i = 0; i < n; ++i) {
    if (sizes[i] > (size_t)INT_MAX) return ncclInternalError;
    isz[i] = (int)sizes[i];
  }
  return g8->irecv(rc, n, data, isz, tags, mhs, req);
}
static ncclResult_t oldIflush(void* rc, int n, void** data, int* sizes, void** mhs, void** req) {
  return g10 ? g10->iflush(rc, n, data, sizes, mhs, req) : g9 ? g9->iflush(rc, n, data, sizes, mhs, req) : g8->iflush(rc, n, data, sizes, mhs, req);
}
static ncclResult_t oldTest(void* req, int* done, int* sizes) { return g10 ? g10->test(req, done, sizes) : g9 ? g9->test(req, done, sizes) : g8->test(req, done, sizes); }
static ncclResult_t oldCloseSend(void* c) { return g10 ? g10->closeSend(c) : g9 ? g9->closeSend(c) : g8->closeSend(c); }
static ncclResult_t oldCloseRecv(void* c) { return g10 ? g10->closeRecv(c) : g9 ? g9->closeRecv(c) : g8->closeRecv(c); }
static ncclResult_t oldCloseListen(void* c) { return g10 ? g10->closeListen(c) : g9 ? g9->closeListen(c) : g8->closeListen(c); }
static ncclResult_t oldGetDeviceMr(void* c, void* m, void** d) {
  auto fn = g10 ? g10->getDeviceMr : g9 ? g9->getDeviceMr : g8->getDeviceMr;
  return fn ? fn(c, m, d) : ncclInternalError;
}
static ncclResult_t oldIrecvConsumed(void* c, int n, void* req) {
  auto fn = g10 ? g10->irecvConsumed : g9 ? g9->irecvConsumed : g8->irecvConsumed;
  return fn ? fn(c, n, req) : ncclSuccess;
}
static ncclResult_t oldMakeVDevice(int* d, ncclNetVDeviceProps_t* props) {
  auto fn = g10 ? g10->makeVDevice : g9 ? g9->makeVDevice : nullptr;
  return fn ? fn(d, props) : ncclInvalidUsage;
}
static ncclResult_t noNetAttr(void*, ncclNetAttr_t*) { return ncclSuccess; }

// Looks for the newest older table in `lib`; returns an adapter with the current signature, or null.
ncclNet_t* netCompatWrap(void* lib, int* version) {
  memset(&gShim, 0, sizeof(gShim));
  if ((g11 = (ncclNet_v11_t*)pluginSymbol(lib, "ncclNetPlugin_v11"))) {
    *version = 11;
    snprintf(gShimName, sizeof(gShimName), "%s", g11->name ? g11->name : "?");
    gShim.name = gShimName;
    gShim.init = g11->init; gShim.devices = g11->devices; gShim.getProperties = v11Props; gShim.listen = g11->listen; gShim.connect = g11->connect;
    gShim.accept = g11->accept; gShim.regMr = g11->regMr; gShim.regMrDmaBuf = g11->regMrDmaBuf; gShim.deregMr = g11->deregMr; gShim.isend = g11->isend;
    gShim.irecv = g11->irecv; gShim.iflush = g11->iflush; gShim.test = g11->test; gShim.closeSend = g11->closeSend; gShim.closeRecv = g11->closeRecv;
    gShim.closeListen = g11->closeListen; gShim.getDeviceMr = g11->getDeviceMr; gShim.irecvConsumed = g11->irecvConsumed;
    gShim.makeVDevice = g11->makeVDevice; gShim.finalize = g11->finalize; gShim.setNetAttr = g11->setNetAttr;
    return &gShim;
  }
  const char* name = nullptr;
  if ((g10 = (ncclNet_v10_t*)pluginSymbol(lib, "ncclNetPlugin_v10"))) { *version = 10; name = g10->name; }
  else if ((g9 = (ncclNet_v9_t*)pluginSymbol(lib, "ncclNetPlugin_v9"))) { *version = 9; name = g9->name; }
  else if ((g8 = (ncclNet_v8_t*)pluginSymbol(lib, "ncclNetPlugin_v8"))) { *version = 8; name = g8->name; }
  else return nullptr;
  snprintf(gShimName, sizeof(gShimName), "%s", name ? name : "?");
  gShim.name = gShimName;
  gShim.init = oldInit; gShim.devices = oldDevices; gShim.getProperties = oldProps; gShim.listen = oldListen; gShim.connect = oldConnect;
  gShim.accept = oldAccept; gShim.regMr = oldRegMr; gShim.regMrDmaBuf = oldRegMrDmaBuf; gShim.deregMr = oldDeregMr; gShim.isend = oldIsend;
  gShim.irecv = oldIrecv; gShim.iflush = oldIflush; gShim.test = oldTest; gShim.closeSend = oldCloseSend; gShim.closeRecv = oldCloseRecv;
  gShim.closeListen = oldCloseListen; gShim.getDeviceMr = oldGetDeviceMr; gShim.irecvConsumed = oldIrecvConsumed;
  gShim.makeVDevice = oldMakeVDevice; gShim.finalize = oldFinalize; gShim.setNetAttr = noNetAttr;
  return &gShim;
}

}  // namespace b200
