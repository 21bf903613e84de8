// Example profiler plugin: records every event it is offered and writes them at finalize as a
// Chrome trace (chrome://tracing, Perfetto) to $NCCL_PROFILE_DUMP_FILE-<commId>-<rank>.json
// (default ./nccl_trace). NCCL_PROFILE_EVENT_MASK selects event kinds (default: everything).
// Reference parity: plugins/profiler/example (plugin.cc event pools, print_event.cc trace output).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include <mutex>
#include <string>
#include <vector>

#include "plugin/nccl_profiler.h"
#include "plugin/nccl_profiler_net.h"

namespace {

double nowUs() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec * 1e6 + ts.tv_nsec / 1e3;
}

struct Ctx;
struct Event {
  Ctx* ctx;
  uint64_t type;
  std::string name, args;
  double t0, t1 = 0;
  int sleeps = 0, appended = 0;   // ProxyCtrl: states seen
};
struct Ctx {
  uint64_t commId;
  int rank;
  std::mutex lock;
  std::vector<Event*> done;
};

const char* kindName(uint64_t t) {
  switch (t) {
    case ncclProfileGroup: return "Group";
    case ncclProfileColl: return "Coll";
    case ncclProfileP2p: return "P2p";
    case ncclProfileProxyOp: return "ProxyOp";
    case ncclProfileProxyStep: return "ProxyStep";
    case ncclProfileProxyCtrl: return "ProxyCtrl";
    case ncclProfileKernelCh: return "KernelCh";
    case ncclProfileNetPlugin: return "NetPlugin";
    case ncclProfileGroupApi: return "GroupApi";
    case ncclProfileCollApi: return "CollApi";
    case ncclProfileP2pApi: return "P2pApi";
    case ncclProfileKernelLaunch: return "KernelLaunch";
    case ncclProfileCeColl: return "CeColl";
    case ncclProfileCeSync: return "CeSync";
    case ncclProfileCeBatch: return "CeBatch";
    default: return "Event";
  }
}

ncclResult_t pInit(void** context, uint64_t commId, int* mask, const char*, int, int, int rank, ncclDebugLogger_t) {
  Ctx* c = new Ctx;
  c->commId = commId;
  c->rank = rank;
  if (*mask == 0) *mask = 0x7fff;
  *context = c;
  return ncclSuccess;
}

ncclResult_t pStart(void* context, void** handle, ncclProfilerEventDescr_t* d) {
  Event* e = new Event;
  e->ctx = (Ctx*)context;
  e->type = d->type;
  e->t0 = nowUs();
  char buf[256] = "";
  if (d->type == ncclProfileColl) {
    e->name = d->coll.func ? d->coll.func : "coll";
    snprintf(buf, sizeof(buf), "\"count\":%zu,\"algo\":\"%s\",\"proto\":\"%s\",\"channels\":%d,\"seq\":%llu", d->coll.count, d->coll.algo ? d->coll.algo : "",
             d->coll.proto ? d->coll.proto : "", d->coll.nChannels, (unsigned long long)d->coll.seqNumber);
  } else if (d->type == ncclProfileCollApi) {
    e->name = std::string(d->collApi.func ? d->collApi.func : "coll") + " (API)";
    snprintf(buf, sizeof(buf), "\"count\":%zu,\"datatype\":\"%s\"", d->collApi.count, d->collApi.datatype ? d->collApi.datatype : "");
  } else if (d->type == ncclProfileP2p) {
    e->name = d->p2p.func ? d->p2p.func : "p2p";
    snprintf(buf, sizeof(buf), "\"count\":%zu,\"peer\":%d", d->p2p.count, d->p2p.peer);
  } else if (d->type == ncclProfileP2pApi) {
    e->name = std::string(d->p2pApi.func ? d->p2pApi.func : "p2p") + " (API)";
  } else if (d->type == ncclProfileProxyOp) {
    e->name = d->proxyOp.isSend ? "ProxySend" : "ProxyRecv";
    snprintf(buf, sizeof(buf), "\"peer\":%d,\"steps\":%d,\"chunk\":%d", d->proxyOp.peer, d->proxyOp.nSteps, d->proxyOp.chunkSize);
  } else if (d->type == ncclProfileKernelCh) {
    e->name = kindName(d->type);
    snprintf(buf, sizeof(buf), "\"channel\":%d,\"gpu_start_ns\":%llu", d->kernelCh.channelId, (unsigned long long)d->kernelCh.pTimer);
  } else if (d->type == ncclProfileNetPlugin) {
    // the backend's own record: which backend and which version of its record is in the plugin id
    const unsigned id = (unsigned)d->netPlugin.id, ver = id & NCCL_PROFILER_NET_VER_MASK;
    if ((id & NCCL_PROFILER_NET_TYPE_MASK) == NCCL_PROFILER_NET_TYPE_IB && ver == NCCL_PROFILER_NET_IB_VER && d->netPlugin.data) {
      const ncclProfilerNetIbDescr_v1_t* n = (const ncclProfilerNetIbDescr_v1_t*)d->netPlugin.data;
      e->name = "NetIb Qp";
      snprintf(buf, sizeof(buf), "\"device\":%d,\"qp\":%d,\"opcode\":%d,\"wr_id\":%llu,\"bytes\":%zu", n->qp.device, n->qp.qpNum, n->qp.opcode,
               (unsigned long long)n->qp.wr_id, n->qp.length);
    } else if ((id & NCCL_PROFILER_NET_TYPE_MASK) == NCCL_PROFILER_NET_TYPE_SOCK && ver == NCCL_PROFILER_NET_SOCKET_VER && d->netPlugin.data) {
      const ncclProfilerNetSockDescr_v1_t* n = (const ncclProfilerNetSockDescr_v1_t*)d->netPlugin.data;
      e->name = n->sock.op ? "NetSock Recv" : "NetSock Send";
      snprintf(buf, sizeof(buf), "\"fd\":%d,\"bytes\":%zu", n->sock.fd, n->sock.length);
    } else {
      e->name = kindName(d->type);
      snprintf(buf, sizeof(buf), "\"plugin_id\":%u", id);
    }
  } else {
    e->name = kindName(d->type);
  }
  e->args = buf;
  *handle = e;
  return ncclSuccess;
}

ncclResult_t pStop(void* handle) {
  Event* e = (Event*)handle;
  if (!e) return ncclSuccess;
  e->t1 = nowUs();
  if (e->type == ncclProfileProxyCtrl) {
    char buf[64];
    snprintf(buf, sizeof(buf), "\"sleeps\":%d,\"operations\":%d", e->sleeps, e->appended);
    e->args = buf;
  }
  std::lock_guard<std::mutex> g(e->ctx->lock);
  e->ctx->done.push_back(e);
  return ncclSuccess;
}

ncclResult_t pState(void* handle, ncclProfilerEventState_t st, ncclProfilerEventStateArgs_t* a) {
  Event* e = (Event*)handle;
  char buf[64];
  if (e && a && e->type == ncclProfileKernelCh && st == ncclProfilerKernelChStop) {
    snprintf(buf, sizeof(buf), ",\"gpu_stop_ns\":%llu", (unsigned long long)a->kernelCh.pTimer);
    e->args += buf;
  } else if (e && a && e->type == ncclProfileProxyStep && (st == ncclProfilerProxyStepSendWait || st == ncclProfilerProxyStepRecvWait)) {
    snprintf(buf, sizeof(buf), "%s\"bytes\":%zu", e->args.empty() ? "" : ",", a->proxyStep.transSize);
    e->args += buf;
  } else if (e && e->type == ncclProfileProxyCtrl) {
    // how often the proxy thread went to sleep and how many operations it was handed
    if (st == ncclProfilerProxyCtrlSleep) e->sleeps++;
    if (st == ncclProfilerProxyCtrlActive && a) e->appended += a->proxyCtrl.appendedProxyOps;
  }
  return ncclSuccess;
}

ncclResult_t pFinalize(void* context) {
  Ctx* c = (Ctx*)context;
  const char* base = getenv("NCCL_PROFILE_DUMP_FILE");
  char path[512];
  snprintf(path, sizeof(path), "%s-%llx-%d.json", base && *base ? base : "nccl_trace", (unsigned long long)c->commId, c->rank);
  FILE* f = fopen(path, "w");
  if (f) {
    fprintf(f, "[\n");
    bool first = true;
    for (Event* e : c->done) {
      fprintf(f, "%s{\"name\":\"%s\",\"cat\":\"%s\",\"ph\":\"X\",\"ts\":%.3f,\"dur\":%.3f,\"pid\":%d,\"tid\":\"%s\",\"args\":{%s}}", first ? "" : ",\n", e->name.c_str(),
              kindName(e->type), e->t0, e->t1 - e->t0, c->rank, kindName(e->type), e->args.c_str());
      first = false;
    }
    fprintf(f, "\n]\n");
    fclose(f);
  }
  for (Event* e : c->done) delete e;
  delete c;
  return ncclSuccess;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) const ncclProfiler_v6_t ncclProfiler_v6 = {"trace", pInit, pStart, pStop, pState, pFinalize};
