// Example tuner plugin driven by a CSV file (NCCL_TUNER_CONFIG_FILE, default
// ./nccl_tuner.conf). Each line:
//   collective,minBytes,maxBytes,algorithm,protocol,channels[,nNodes[,nRanks[,numPipeOps[,regBuff]]]]
// with collective in {broadcast,reduce,allgather,reducescatter,allreduce}, algorithm in
// {tree,ring,collnet_direct,collnet_chain,nvls,nvls_tree,pat}, protocol in {ll,ll128,simple};
// -1 for channels / nNodes / nRanks / numPipeOps / regBuff means "any". The first matching line
// wins: its (algorithm, protocol) entry of the cost table is set to 0 so that the core picks it.
// Reference parity: plugins/tuner/example/plugin.c (CSV format and matching rules).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>

#include <string>
#include <vector>

#include "plugin/nccl_tuner.h"

namespace {

struct Rule {
  int coll;
  size_t lo, hi;
  int algo, proto, channels, nNodes, nRanks, pipeOps, regBuff;
};
struct Ctx {
  std::vector<Rule> rules;
  size_t nRanks, nNodes;
  ncclDebugLogger_t log;
};

int lookup(const char* s, const char* const* names, int n) {
  for (int i = 0; i < n; ++i) if (!strcasecmp(s, names[i])) return i;
  return -1;
}
const char* const kColls[] = {"broadcast", "reduce", "allgather", "reducescatter", "allreduce"};
const char* const kAlgos[] = {"tree", "ring", "collnet_direct", "collnet_chain", "nvls", "nvls_tree", "pat"};
const char* const kProtos[] = {"ll", "ll128", "simple"};

ncclResult_t tInit(void** ctx, uint64_t, size_t nRanks, size_t nNodes, ncclDebugLogger_t log, ncclNvlDomainInfo_t*, ncclTunerConstants_t*) {
  Ctx* c = new Ctx;
  c->nRanks = nRanks;
  c->nNodes = nNodes;
  c->log = log;
  const char* path = getenv("NCCL_TUNER_CONFIG_FILE");
  if (!path) path = "nccl_tuner.conf";
  FILE* f = fopen(path, "r");
  if (f) {
    char line[512];
    while (fgets(line, sizeof(line), f)) {
      if (line[0] == '#' || line[0] == '\n') continue;
      std::vector<std::string> tok;
      for (char* p = strtok(line, ",\n\r"); p; p = strtok(nullptr, ",\n\r")) {
        while (*p == ' ') ++p;
        tok.push_back(p);
      }
      if (tok.size() < 6) continue;
      Rule r;
      r.coll = lookup(tok[0].c_str(), kColls, 5);
      r.lo = strtoull(tok[1].c_str(), nullptr, 0);
      r.hi = strtoull(tok[2].c_str(), nullptr, 0);
      r.algo = lookup(tok[3].c_str(), kAlgos, 7);
      r.proto = lookup(tok[4].c_str(), kProtos, 3);
      r.channels = atoi(tok[5].c_str());
      r.nNodes = tok.size() > 6 ? atoi(tok[6].c_str()) : -1;
      r.nRanks = tok.size() > 7 ? atoi(tok[7].c_str()) : -1;
      r.pipeOps = tok.size() > 8 ? atoi(tok[8].c_str()) : -1;
      r.regBuff = tok.size() > 9 ? atoi(tok[9].c_str()) : -1;
      if (r.coll < 0 || r.algo < 0 || r.proto < 0) continue;
      c->rules.push_back(r);
    }
    fclose(f);
  }
  if (log) log(NCCL_LOG_INFO, NCCL_TUNING, __FILE__, __LINE__, "csv tuner: %zu rule(s) from %s", c->rules.size(), path);
  *ctx = c;
  return ncclSuccess;
}

ncclResult_t tGetCollInfo(void* ctx, ncclFunc_t coll, size_t nBytes, int numPipeOps, float** table, int numAlgo, int numProto, int regBuff, int* nChannels) {
  Ctx* c = (Ctx*)ctx;
  for (const Rule& r : c->rules) {
    if (r.coll != (int)coll || nBytes < r.lo || nBytes > r.hi) continue;
    if (r.nNodes >= 0 && (size_t)r.nNodes != c->nNodes) continue;
    if (r.nRanks >= 0 && (size_t)r.nRanks != c->nRanks) continue;
    if (r.pipeOps >= 0 && r.pipeOps != numPipeOps) continue;
    if (r.regBuff >= 0 && r.regBuff != regBuff) continue;
    if (r.algo >= numAlgo || r.proto >= numProto) continue;
    if (table[r.algo][r.proto] == (float)NCCL_ALGO_PROTO_IGNORE) continue;   // the core cannot run this combination
    table[r.algo][r.proto] = 0.0f;
    if (r.channels > 0) *nChannels = r.channels;
    return ncclSuccess;
  }
  return ncclSuccess;
}

ncclResult_t tFinalize(void* ctx) { delete (Ctx*)ctx; return ncclSuccess; }

}  // namespace

extern "C" __attribute__((visibility("default"))) const ncclTuner_v6_t ncclTunerPlugin_v6 = {"csv", tInit, tGetCollInfo, tFinalize, nullptr};
