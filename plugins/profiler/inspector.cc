// Inspector: an always-on profiler plugin that turns collective / point-to-point task events
// into per-operation latency and bandwidth records.
//   - one JSON line per completed operation, written by a background thread to
//     $NCCL_INSPECTOR_DUMP_DIR/<host>-pid<pid>-rank<rank>.jsonl every
//     NCCL_INSPECTOR_DUMP_THREAD_INTERVAL_MICROSECONDS (default 1 s)
//   - with NCCL_INSPECTOR_PROM_DUMP=1, a Prometheus text file next to it (node-exporter textfile
//     collector format) with gauges nccl_bus_bandwidth_gbs, nccl_algorithm_bandwidth_gbs,
//     nccl_collective_exec_time_microseconds and counters nccl_collective_count, nccl_p2p_count,
//     nccl_p2p_bytes_total, labelled by communicator, rank and collective.
// Execution time is the device window reported by the kernel-channel event when there is one,
// the host-side span otherwise. busBW follows the usual convention (all-reduce 2(n-1)/n; all-gather,
// reduce-scatter, all-to-all (n-1)/n; others 1).
// Reference parity: plugins/profiler/inspector (inspector.cc, inspector_plugin.cc,
// inspector_json.cc, inspector_prom.cc); metric names from its README.md:164-166.
#include <algorithm>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#include <condition_variable>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "plugin/nccl_profiler.h"

namespace {

uint64_t nowNs() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + ts.tv_nsec;
}

size_t typeBytes(const char* t) {
  if (!t) return 1;
  if (strstr(t, "64")) return 8;
  if (strstr(t, "32")) return 4;
  if (strstr(t, "16")) return 2;
  return 1;
}

struct Stats { uint64_t count = 0; double lastUs = 0, lastAlg = 0, lastBus = 0, sumUs = 0; uint64_t bytes = 0; };

struct Ctx {
  uint64_t commId;
  std::string commName;
  int nranks, rank;
  std::mutex lock;
  std::vector<std::string> lines;
  std::map<std::string, Stats> stats;
  Stats p2p;
  std::string base;
  bool prom = false;
  bool stop = false;
  std::thread dumper;
  std::condition_variable cv;
  long intervalUs = 1000000;
};

struct Event {
  Ctx* ctx;
  uint64_t type;
  Event* parent = nullptr;
  std::string func, algo, proto, dtype;
  size_t count = 0;
  int nChannels = 0, peer = -1;
  uint64_t seq = 0;
  uint64_t hostStart = 0;
  uint64_t devStart = 0, devStop = 0;
  bool haveDev = false;
};

double busFactor(const std::string& f, int n) {
  if (n <= 1) return 1.0;
  if (f == "AllReduce") return 2.0 * (n - 1) / n;
  if (f == "AllGather" || f == "ReduceScatter" || f == "AlltoAll") return (double)(n - 1) / n;
  return 1.0;
}

void flush(Ctx* c) {
  std::vector<std::string> lines;
  std::map<std::string, Stats> stats;
  Stats p2p;
  {
    std::lock_guard<std::mutex> g(c->lock);
    lines.swap(c->lines);
    stats = c->stats;
    p2p = c->p2p;
  }
  if (!lines.empty()) {
    FILE* f = fopen((c->base + ".jsonl").c_str(), "a");
    if (f) {
      for (auto& l : lines) fputs(l.c_str(), f);
      fclose(f);
    }
  }
  if (c->prom) {
    std::string tmp = c->base + ".prom.tmp", fin = c->base + ".prom";
    FILE* f = fopen(tmp.c_str(), "w");
    if (!f) return;
    fprintf(f, "# TYPE nccl_bus_bandwidth_gbs gauge\n# TYPE nccl_algorithm_bandwidth_gbs gauge\n# TYPE nccl_collective_exec_time_microseconds gauge\n# TYPE nccl_collective_count counter\n");
    for (auto& kv : stats) {
      char lab[256];
      snprintf(lab, sizeof(lab), "{comm=\"0x%llx\",rank=\"%d\",nranks=\"%d\",collective=\"%s\"}", (unsigned long long)c->commId, c->rank, c->nranks, kv.first.c_str());
      fprintf(f, "nccl_bus_bandwidth_gbs%s %.3f\n", lab, kv.second.lastBus);
      fprintf(f, "nccl_algorithm_bandwidth_gbs%s %.3f\n", lab, kv.second.lastAlg);
      fprintf(f, "nccl_collective_exec_time_microseconds%s %.3f\n", lab, kv.second.lastUs);
      fprintf(f, "nccl_collective_count%s %llu\n", lab, (unsigned long long)kv.second.count);
    }
    fprintf(f, "# TYPE nccl_p2p_count counter\n# TYPE nccl_p2p_bytes_total counter\n");
    fprintf(f, "nccl_p2p_count{comm=\"0x%llx\",rank=\"%d\"} %llu\n", (unsigned long long)c->commId, c->rank, (unsigned long long)p2p.count);
    fprintf(f, "nccl_p2p_bytes_total{comm=\"0x%llx\",rank=\"%d\"} %llu\n", (unsigned long long)c->commId, c->rank, (unsigned long long)p2p.bytes);
    fclose(f);
    rename(tmp.c_str(), fin.c_str());   // readers never see a half-written file
  }
}

void dumperMain(Ctx* c) {
  std::unique_lock<std::mutex> lk(c->lock);
  while (!c->stop) {
    c->cv.wait_for(lk, std::chrono::microseconds(c->intervalUs));
    lk.unlock();
    flush(c);
    lk.lock();
  }
}

ncclResult_t pInit(void** context, uint64_t commId, int* mask, const char* commName, int, int nranks, int rank, ncclDebugLogger_t log) {
  Ctx* c = new Ctx;
  c->commId = commId;
  c->commName = commName ? commName : "";
  c->nranks = nranks;
  c->rank = rank;
  const char* dir = getenv("NCCL_INSPECTOR_DUMP_DIR");
  char host[128] = "host";
  gethostname(host, sizeof(host) - 1);
  char base[512];
  snprintf(base, sizeof(base), "%s/%s-pid%d-rank%d", dir && *dir ? dir : ".", host, (int)getpid(), rank);
  c->base = base;
  const char* p = getenv("NCCL_INSPECTOR_PROM_DUMP");
  c->prom = p && atoi(p) != 0;
  const char* iv = getenv("NCCL_INSPECTOR_DUMP_THREAD_INTERVAL_MICROSECONDS");
  if (iv && atol(iv) > 0) c->intervalUs = atol(iv);
  *mask = ncclProfileColl | ncclProfileP2p | ncclProfileKernelCh;
  c->dumper = std::thread(dumperMain, c);
  if (log) log(NCCL_LOG_INFO, NCCL_PROFILE, __FILE__, __LINE__, "inspector: records go to %s.jsonl%s", base, c->prom ? " and .prom" : "");
  *context = c;
  return ncclSuccess;
}

ncclResult_t pStart(void* context, void** handle, ncclProfilerEventDescr_t* d) {
  Ctx* c = (Ctx*)context;
  Event* e = new Event;
  e->ctx = c;
  e->type = d->type;
  e->hostStart = nowNs();
  if (d->type == ncclProfileColl) {
    e->func = d->coll.func ? d->coll.func : "";
    e->algo = d->coll.algo ? d->coll.algo : "";
    e->proto = d->coll.proto ? d->coll.proto : "";
    e->dtype = d->coll.datatype ? d->coll.datatype : "";
    e->count = d->coll.count;
    e->nChannels = d->coll.nChannels;
    e->seq = d->coll.seqNumber;
  } else if (d->type == ncclProfileP2p) {
    e->func = d->p2p.func ? d->p2p.func : "";
    e->dtype = d->p2p.datatype ? d->p2p.datatype : "";
    e->count = d->p2p.count;
    e->peer = d->p2p.peer;
    e->nChannels = d->p2p.nChannels;
  } else if (d->type == ncclProfileKernelCh) {
    e->parent = (Event*)d->parentObj;
    e->devStart = d->kernelCh.pTimer;
  }
  *handle = e;
  return ncclSuccess;
}

ncclResult_t pState(void* handle, ncclProfilerEventState_t st, ncclProfilerEventStateArgs_t* a) {
  Event* e = (Event*)handle;
  if (e && e->type == ncclProfileKernelCh && st == ncclProfilerKernelChStop && a) {
    e->devStop = a->kernelCh.pTimer;
    if (e->parent) {   // the operation spans its CTAs: earliest start, latest stop
      e->parent->devStart = e->parent->haveDev ? std::min(e->parent->devStart, e->devStart) : e->devStart;
      e->parent->devStop = e->parent->haveDev ? std::max(e->parent->devStop, e->devStop) : e->devStop;
      e->parent->haveDev = true;
    }
  }
  return ncclSuccess;
}

ncclResult_t pStop(void* handle) {
  Event* e = (Event*)handle;
  if (!e) return ncclSuccess;
  Ctx* c = e->ctx;
  if (e->type == ncclProfileColl || e->type == ncclProfileP2p) {
    const double us = e->haveDev ? (e->devStop - e->devStart) / 1e3 : (nowNs() - e->hostStart) / 1e3;
    size_t bytes = e->count * typeBytes(e->dtype.c_str());
    if (e->func == "AllGather" || e->func == "AlltoAll") bytes *= (size_t)c->nranks;   // count is per rank for these
    const double alg = us > 0 ? bytes / us / 1e3 : 0;
    const double bus = alg * busFactor(e->func, c->nranks);
    char line[768];
    snprintf(line, sizeof(line),
             "{\"comm\":\"0x%llx\",\"comm_name\":\"%s\",\"rank\":%d,\"nranks\":%d,\"kind\":\"%s\",\"func\":\"%s\",\"seq\":%llu,\"count\":%zu,"
             "\"datatype\":\"%s\",\"bytes\":%zu,\"algo\":\"%s\",\"proto\":\"%s\",\"channels\":%d,\"peer\":%d,\"timing\":\"%s\",\"exec_time_us\":%.3f,"
             "\"alg_bw_gbs\":%.3f,\"bus_bw_gbs\":%.3f}\n",
             (unsigned long long)c->commId, c->commName.c_str(), c->rank, c->nranks, e->type == ncclProfileColl ? "coll" : "p2p", e->func.c_str(),
             (unsigned long long)e->seq, e->count, e->dtype.c_str(), bytes, e->algo.c_str(), e->proto.c_str(), e->nChannels, e->peer,
             e->haveDev ? "device" : "host", us, alg, bus);
    std::lock_guard<std::mutex> g(c->lock);
    c->lines.push_back(line);
    Stats& s = e->type == ncclProfileColl ? c->stats[e->func] : c->p2p;
    s.count++;
    s.lastUs = us;
    s.lastAlg = alg;
    s.lastBus = bus;
    s.sumUs += us;
    s.bytes += bytes;
  }
  delete e;
  return ncclSuccess;
}

ncclResult_t pFinalize(void* context) {
  Ctx* c = (Ctx*)context;
  {
    std::lock_guard<std::mutex> g(c->lock);
    c->stop = true;
  }
  c->cv.notify_all();
  if (c->dumper.joinable()) c->dumper.join();
  flush(c);
  delete c;
  return ncclSuccess;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) const ncclProfiler_v6_t ncclProfiler_v6 = {"inspector", pInit, pStart, pStop, pState, pFinalize};
