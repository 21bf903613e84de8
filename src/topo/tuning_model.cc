// Analytic latency / bandwidth model per (collective, algorithm, protocol), after the reference's
// cost model: time = latency + bytes / algorithm bandwidth, with base and per-hop latencies and
// per-protocol bandwidth efficiencies. It feeds ncclGroupSimulateEnd and tuner plugins; kernel
// selection itself uses the measured table (sched/tuning.cc).
// Reference parity: src/graph/tuning.cc (constants :139-212, ncclTopoTuneModel :243-618,
// ncclTopoGetAlgoTime :630-655).
#include <math.h>

#include "topo.h"

namespace b200 {

// microseconds
static const float kBaseLat[MODEL_ALGOS][MODEL_PROTOS] = {
    /* tree */ {6.8f, 14.0f, 8.4f}, /* ring */ {6.6f, 14.0f, 8.4f}, /* collnet direct */ {0, 0, 0}, /* collnet chain */ {0, 0, 0},
    /* nvls */ {0, 0, 0}, /* nvls tree */ {0, 0, 0}, /* pat */ {8.0f, 8.0f, 8.0f}};
static const float kNvlinkLat[MODEL_ALGOS][MODEL_PROTOS] = {
    {0.6f, 1.25f, 4.0f}, {0.6f, 1.9f, 3.4f}, {0, 0, 3.7f}, {0, 0, 2.8f}, {0, 0, 25.0f}, {0, 0, 25.0f}, {0.6f, 1.9f, 3.4f}};
static const float kPciLat[MODEL_PROTOS] = {1.0f, 1.9f, 4.0f};
static const float kNetLat[MODEL_PROTOS] = {5.0f, 8.5f, 14.0f};

void topoTuneModel(const TopoSystem* sys, const TopoGraph* ring, const TopoGraph* tree, const TopoGraph* nvls, int nRanks, int nNodes,
                   int compCap, TuneModel* m) {
  (void)sys;
  *m = TuneModel();
  m->nRanks = nRanks;
  m->nNodes = nNodes;
  if (nRanks <= 1) return;
  const bool blackwell = compCap >= 100;
  const float nvlsEff = blackwell ? 0.74f : 0.85f;
  const float llMaxBw = blackwell ? 2 * 141.0f : 2 * 39.0f;   // whole-GPU cap of the 8-byte-flag protocol
  const int ppn = nRanks / std::max(nNodes, 1);
  for (int func = 0; func < FUNC_COUNT; ++func) {
    const int nsteps = func == FUNC_ALLREDUCE ? 2 * (nRanks - 1) : (func == FUNC_REDUCESCATTER || func == FUNC_ALLGATHER) ? nRanks - 1 : nRanks;
    for (int a = 0; a < MODEL_ALGOS; ++a) {
      const TopoGraph* g = a == MODEL_RING || a == MODEL_PAT ? ring : (a == MODEL_NVLS || a == MODEL_NVLS_TREE) ? nvls : tree;
      if (a == MODEL_COLLNET_DIRECT || a == MODEL_COLLNET_CHAIN) continue;             // no in-network reduction backend
      if ((a == MODEL_NVLS || a == MODEL_NVLS_TREE) && (g->nChannels == 0 || nNodes > 1)) continue;
      if (a == MODEL_TREE && func != FUNC_ALLREDUCE) continue;
      if (a == MODEL_PAT && !(func == FUNC_ALLGATHER || func == FUNC_REDUCESCATTER)) continue;
      if ((a == MODEL_NVLS || a == MODEL_NVLS_TREE) && !(func == FUNC_ALLREDUCE || func == FUNC_ALLGATHER || func == FUNC_REDUCESCATTER)) continue;
      for (int p = 0; p < MODEL_PROTOS; ++p) {
        if ((a == MODEL_NVLS || a == MODEL_NVLS_TREE) && p != MODEL_SIMPLE) continue;
        float bw = nNodes <= 2 ? g->bwIntra : g->bwInter;
        float busBw = g->nChannels * bw;
        if (a == MODEL_RING && p == MODEL_LL) busBw = std::min(llMaxBw, busBw * 0.5f);
        if (a == MODEL_RING && p == MODEL_LL128) busBw = busBw * 0.92f;
        if (a == MODEL_TREE) busBw = std::min(busBw * 0.92f, g->nChannels * (blackwell ? 70.0f : 39.0f));
        if (a == MODEL_TREE && p == MODEL_LL) busBw = std::min(busBw / 3.8f, llMaxBw);
        if (a == MODEL_TREE && p == MODEL_LL128) busBw = std::min(busBw * 0.7f, g->nChannels * (blackwell ? 55.6f : 31.67f));
        if (a == MODEL_NVLS || a == MODEL_NVLS_TREE) busBw = std::min(busBw, blackwell ? 720.0f : 360.0f) * nvlsEff;
        if (a == MODEL_PAT) busBw *= 0.75f;
        // bus bandwidth -> algorithm bandwidth
        float ratio = 1.0f;
        if (a == MODEL_RING || a == MODEL_PAT) ratio = (float)nRanks / nsteps;
        else if (a == MODEL_NVLS || a == MODEL_NVLS_TREE) ratio = func == FUNC_ALLREDUCE ? 5.0f / 6.0f : 1.0f;
        else ratio = 0.5f;
        m->bandwidths[func][a][p] = busBw * ratio;
        // latency
        float lat = kBaseLat[a][p];
        const float intraLat = kNvlinkLat[a][p];
        const float interLat = kNetLat[p];
        if (a == MODEL_RING) {
          const int netSteps = nNodes > 1 ? (func == FUNC_ALLREDUCE ? 2 * (nNodes - 1) : nNodes - 1) : 0;
          lat += (nsteps - netSteps) * intraLat + netSteps * interLat;
        } else if (a == MODEL_TREE) {
          lat += 2 * ((ppn - 1) * intraLat + log2f((float)std::max(nNodes, 1)) * interLat);
          if (nNodes == 1) lat += 2 * log2f((float)nRanks) * intraLat * 0.5f;
        } else if (a == MODEL_NVLS || a == MODEL_NVLS_TREE) {
          lat += intraLat + (nNodes > 1 ? interLat : 0);
        } else if (a == MODEL_PAT) {
          lat += log2f((float)nRanks) * (nNodes > 1 ? interLat : intraLat) + kPciLat[p] * 0;
        }
        m->latencies[func][a][p] = lat;
      }
    }
  }
}

float topoAlgoTime(const TuneModel* m, int func, int algo, int proto, size_t bytes) {
  if (func < 0 || func >= FUNC_COUNT || algo < 0 || algo >= MODEL_ALGOS || proto < 0 || proto >= MODEL_PROTOS) return -1.0f;
  float bw = m->bandwidths[func][algo][proto];
  if (bw <= 0) return -1.0f;
  float lat = m->latencies[func][algo][proto];
  // trees lose efficiency on mid-size messages (pipeline fill), as the reference's correction table models
  if (algo == MODEL_TREE && func == FUNC_ALLREDUCE) {
    int logSize = bytes > 0 ? (int)log2f((float)(bytes >> 6)) : 0;
    static const float corr[MODEL_PROTOS][23] = {
        {1.0f, 1.0f, 1.0f, 1.0f, .9f, .8f, .7f, .7f, .7f, .7f, .6f, .5f, .4f, .4f, .5f, .6f, .7f, .8f, .9f, 1.0f, 1.0f, 1.0f, 1.0f},
        {1.0f, 1.0f, 1.0f, 1.0f, 1.0f, .9f, .8f, .8f, .8f, .7f, .6f, .6f, .6f, .6f, .6f, .6f, .8f, .9f, .9f, .9f, .9f, 1.0f, 1.0f},
        {.9f, .9f, .9f, .9f, .9f, .9f, .9f, .8f, .7f, .6f, .6f, .5f, .5f, .5f, .5f, .6f, .7f, .8f, .7f, .7f, .8f, .9f, .9f}};
    if (logSize >= 0 && logSize < 23) bw *= corr[proto][logSize];
  }
  return lat + (float)bytes / (1000.0f * bw);
}

}  // namespace b200
