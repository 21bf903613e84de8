// Tuner plugin glue. For every collective the analytic model fills a cost table
// [algorithm][protocol] (microseconds, -1 = unavailable); the plugin edits it and may set the
// channel count; the cheapest remaining entry is mapped onto this data plane's kernels:
//   LL / LL128 protocol -> flagged-line one-shot kernels      ring + simple -> ring kernel
//   tree + simple       -> double-binary-tree kernel          NVLS / NVLS tree -> multimem kernels
//   PAT                 -> direct peer (two-shot) kernels     channel count -> CTA count
// Reference parity: src/plugin/tuner.cc:20-118, tuner/tuner_v5.cc, tuner_v6.cc; cost table built
// the way src/enqueue.cc (getAlgoInfo, updateCollCostTable) does before calling getCollInfo.
#include "../mem/symmetric.h"
#include "../topo/topo.h"
#include "plugin.h"

namespace b200 {

ncclResult_t tunerLoad(ncclComm* comm) {
  const char* want = getEnv("NCCL_TUNER_PLUGIN");
  std::string resolved;
  void* lib = pluginOpen(PLUGIN_TUNER, &resolved);
  if (!lib) { (void)want; return ncclSuccess; }
  TunerState* ts = new TunerState;
  ts->lib = lib;
  // newest interface the library exports, down to v2
  if ((ts->v6 = (ncclTuner_v6_t*)pluginSymbol(lib, "ncclTunerPlugin_v6"))) ts->version = 6;
  else if ((ts->v5 = (ncclTuner_v5_t*)pluginSymbol(lib, "ncclTunerPlugin_v5"))) ts->version = 5;
  else if ((ts->v4 = (ncclTuner_v4_t*)pluginSymbol(lib, "ncclTunerPlugin_v4"))) ts->version = 4;
  else if ((ts->v3 = (ncclTuner_v3_t*)pluginSymbol(lib, "ncclTunerPlugin_v3"))) ts->version = 3;
  else if ((ts->v2 = (ncclTuner_v2_t*)pluginSymbol(lib, "ncclTunerPlugin_v2"))) ts->version = 2;
  if (!ts->version) {
    WARN("tuner plugin %s exports none of ncclTunerPlugin_v6 ... ncclTunerPlugin_v2", resolved.c_str());
    delete ts;
    return ncclSuccess;
  }
  ts->name = ts->v6 ? ts->v6->name : ts->v5 ? ts->v5->name : ts->v4 ? ts->v4->name : ts->v3 ? ts->v3->name : ts->v2->name;
  ncclNvlDomainInfo_t dom = {comm->nNodes, comm->nRanks / std::max(comm->nNodes, 1), (comm->nRanks + comm->nNodes - 1) / std::max(comm->nNodes, 1)};
  ncclTunerConstants_t k;
  memset(&k, 0, sizeof(k));
  // the constants of the analytic model that a plugin may want to see (microseconds, GB/s)
  static const double base[NCCL_NUM_ALGORITHMS][NCCL_NUM_PROTOCOLS] = {{6.8, 14.0, 8.4}, {6.6, 14.0, 8.4}, {0, 0, 0}, {0, 0, 0}, {0, 0, 0}, {0, 0, 0}, {8.0, 8.0, 8.0}};
  memcpy(k.baseLatencies, base, sizeof(base));
  for (int s = 0; s < NCCL_NUM_TUNING_SCALES; ++s) {
    k.llMaxBws[NCCL_BLACKWELL_COMPCAP_IDX][s] = s == 0 ? 141.0 : s == 1 ? 45.0 : 40.0;
    k.perChMaxRingLL128Bws[NCCL_BLACKWELL_COMPCAP_IDX][s] = 40.0;
    k.perChMaxTreeLL128Bws[NCCL_BLACKWELL_COMPCAP_IDX][s] = 55.6;
    k.perChMaxTreeBws[NCCL_BLACKWELL_COMPCAP_IDX][s] = 70.0;
    k.perChMaxNVLSTreeBws[NCCL_BLACKWELL_COMPCAP_IDX][s] = s == 1 ? 96.0 : 80.0;
  }
  ncclResult_t r;
  switch (ts->version) {
    case 6: r = ts->v6->init(&ts->ctx, comm->commHash, comm->nRanks, comm->nNodes, pluginLogger, &dom, &k); break;
    case 5: r = ts->v5->init(&ts->ctx, comm->commHash, comm->nRanks, comm->nNodes, pluginLogger, &dom, &k); break;
    case 4: r = ts->v4->init(comm->nRanks, comm->nNodes, pluginLogger, &ts->ctx); break;
    case 3: r = ts->v3->init(comm->nRanks, comm->nNodes, pluginLogger, &ts->ctx); break;
    default: r = ts->v2->init(comm->nRanks, comm->nNodes, pluginLogger, &ts->ctx); break;
  }
  if (r != ncclSuccess) {
    WARN("tuner plugin %s failed to initialise (%d); built-in selection stays in charge", ts->name.c_str(), (int)r);
    delete ts;
    return ncclSuccess;
  }
  comm->tuner = ts;
  INFO(SUB_TUNING, "tuner plugin %s (%s, interface v%d) attached to communicator %llx", ts->name.c_str(), resolved.c_str(), ts->version, (unsigned long long)comm->commHash);
  return ncclSuccess;
}

void tunerUnload(ncclComm* comm) {
  TunerState* ts = comm->tuner;
  if (!ts) return;
  if (ts->v6 && ts->v6->finalize) ts->v6->finalize(ts->ctx);
  else if (ts->v5 && ts->v5->finalize) ts->v5->finalize(ts->ctx);
  else if (ts->v4 && ts->v4->destroy) ts->v4->destroy(ts->ctx);
  else if (ts->v3 && ts->v3->destroy) ts->v3->destroy(ts->ctx);
  else if (ts->v2 && ts->v2->destroy) ts->v2->destroy(ts->ctx);
  delete ts;   // the library stays mapped: other communicators may use it
  comm->tuner = nullptr;
}

bool tunerPick(ncclComm* comm, int func, size_t bytes, int numPipeOps, bool registered, int* algo, int* ctas) {
  TunerState* ts = comm->tuner;
  if (!ts || func < 0 || func >= NCCL_NUM_FUNCTIONS) return false;   // plugins tune the five classic collectives
  float table[NCCL_NUM_ALGORITHMS][NCCL_NUM_PROTOCOLS];
  float* rows[NCCL_NUM_ALGORITHMS];
  for (int a = 0; a < NCCL_NUM_ALGORITHMS; ++a) {
    rows[a] = table[a];
    for (int p = 0; p < NCCL_NUM_PROTOCOLS; ++p) {
      float t = comm->topo ? topoAlgoTime(&comm->topo->model, func, a, p, bytes) : -1.0f;
      table[a][p] = t < 0 ? (float)NCCL_ALGO_PROTO_IGNORE : t;
    }
  }
  int nChannels = 0;
  int bestA = -1, bestP = -1;
  float best = 0;
  ncclResult_t rc;
  switch (ts->version) {
    case 6: rc = ts->v6->getCollInfo(ts->ctx, (ncclFunc_t)func, bytes, numPipeOps, rows, NCCL_NUM_ALGORITHMS, NCCL_NUM_PROTOCOLS, registered ? 1 : 0, &nChannels); break;
    case 5: rc = ts->v5->getCollInfo(ts->ctx, (ncclFunc_t)func, bytes, numPipeOps, rows, NCCL_NUM_ALGORITHMS, NCCL_NUM_PROTOCOLS, registered ? 1 : 0, &nChannels); break;
    case 4: rc = ts->v4->getCollInfo(ts->ctx, (ncclFunc_t)func, bytes, numPipeOps, rows, NCCL_NUM_ALGORITHMS, NCCL_NUM_PROTOCOLS, registered ? 1 : 0, &nChannels); break;
    case 3: rc = ts->v3->getCollInfo(ts->ctx, (ncclFunc_t)func, bytes, numPipeOps, rows, NCCL_NUM_ALGORITHMS, NCCL_NUM_PROTOCOLS, &nChannels); break;
    default: {
      // v2 answers with one (algorithm, protocol) pair; undefined values leave the choice to the library
      int a2 = NCCL_ALGO_UNDEF, p2 = NCCL_PROTO_UNDEF;
      const bool nvls = comm->sym && comm->sym->mcUsable;
      rc = ts->v2->getCollInfo(ts->ctx, (ncclFunc_t)func, bytes, 0, nvls ? 1 : 0, numPipeOps, &a2, &p2, &nChannels);
      if (rc == ncclSuccess && (a2 < 0 || a2 >= NCCL_NUM_ALGORITHMS || p2 < 0 || p2 >= NCCL_NUM_PROTOCOLS)) return false;
      if (rc == ncclSuccess) {
        for (int a = 0; a < NCCL_NUM_ALGORITHMS; ++a)
          for (int p = 0; p < NCCL_NUM_PROTOCOLS; ++p) table[a][p] = (a == a2 && p == p2) ? 0.0f : (float)NCCL_ALGO_PROTO_IGNORE;
      }
      break;
    }
  }
  if (rc != ncclSuccess) return false;
  for (int a = 0; a < NCCL_NUM_ALGORITHMS; ++a)
    for (int p = 0; p < NCCL_NUM_PROTOCOLS; ++p) {
      if (table[a][p] < 0) continue;
      if (bestA < 0 || table[a][p] < best) { best = table[a][p]; bestA = a; bestP = p; }
    }
  if (bestA < 0) return false;
  int pick;
  if (bestA == NCCL_ALGO_COLLNET_DIRECT || bestA == NCCL_ALGO_COLLNET_CHAIN) return false;   // no in-network reduction backend
  if (bestP == NCCL_PROTO_LL || bestP == NCCL_PROTO_LL128) pick = ALGO_LL_ONESHOT;
  else if (bestA == NCCL_ALGO_RING) pick = ALGO_RING;
  else if (bestA == NCCL_ALGO_TREE) pick = func == FUNC_ALLREDUCE ? ALGO_TREE : ALGO_RING;
  else if (bestA == NCCL_ALGO_NVLS || bestA == NCCL_ALGO_NVLS_TREE) pick = ALGO_NVLS;
  else pick = ALGO_P2P;
  *algo = pick;
  *ctas = nChannels > 0 ? nChannels : 0;
  TRACE(SUB_TUNING, "tuner plugin: %s %zu bytes -> algorithm %d protocol %d (%.1f us), %d channels", funcName(func), bytes, bestA, bestP, best, nChannels);
  return true;
}

}  // namespace b200
