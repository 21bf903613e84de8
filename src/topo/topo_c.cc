// C hooks over the topology code for tests and tools (no communicator needed).
#include <stdio.h>

#include "topo.h"

using namespace b200;

extern "C" {

// Parses a topology XML, builds the system, computes paths and searches ring channels.
// Writes a one-line JSON summary into out. Returns 0 on success.
int b200TopoAnalyze(const char* xmlText, char* out, int outLen) {
  std::string err;
  XmlNode* x = xmlParse(xmlText, &err);
  if (!x) { snprintf(out, outLen, "{\"error\": \"%s\"}", err.c_str()); return 1; }
  TopoSystem* s = topoFromXml(x, &err);
  if (!s) { snprintf(out, outLen, "{\"error\": \"%s\"}", err.c_str()); delete x; return 2; }
  topoComputePaths(s);
  TopoGraph g;
  topoSearch(s, &g, 1, 32);
  std::string ring = "[";
  if (!g.order.empty()) for (size_t i = 0; i < g.order[0].size(); ++i) ring += (i ? "," : "") + std::to_string(g.order[0][i]);
  ring += "]";
  int worst = PATH_LOC, best = PATH_DIS;
  int n = (int)s->byType[TOPO_GPU].size();
  for (int a = 0; a < n; ++a)
    for (int b = 0; b < n; ++b) {
      if (a == b) continue;
      int t = s->nodes[s->byType[TOPO_GPU][a]].paths[s->byType[TOPO_GPU][b]].type;
      worst = std::max(worst, t);
      best = std::min(best, t);
    }
  TuneModel m;
  TopoGraph nv = g;
  nv.nChannels = s->byType[TOPO_NVS].empty() ? 0 : 32;
  int cc = n ? s->nodes[s->byType[TOPO_GPU][0]].cudaCompCap : 0;
  topoTuneModel(s, &g, &g, &nv, n, 1, cc, &m);
  snprintf(out, outLen,
           "{\"gpus\": %d, \"nvswitch\": %d, \"nets\": %d, \"channels\": %d, \"speed\": %.1f, \"type\": \"%s\", \"best_path\": \"%s\", "
           "\"worst_path\": \"%s\", \"ring0\": %s, \"max_bw\": %.1f, \"t_ring_simple_1M\": %.2f, \"t_nvls_1M\": %.2f, \"t_tree_ll_1K\": %.2f}",
           n, (int)s->byType[TOPO_NVS].size(), (int)s->byType[TOPO_NET].size(), g.nChannels, g.bwIntra, topoPathName(g.typeIntra),
           topoPathName(n > 1 ? best : PATH_LOC), topoPathName(n > 1 ? worst : PATH_LOC), ring.c_str(), s->maxBw,
           topoAlgoTime(&m, FUNC_ALLREDUCE, MODEL_RING, MODEL_SIMPLE, 1 << 20), topoAlgoTime(&m, FUNC_ALLREDUCE, MODEL_NVLS, MODEL_SIMPLE, 1 << 20),
           topoAlgoTime(&m, FUNC_ALLREDUCE, MODEL_TREE, MODEL_LL, 1 << 10));
  delete s;
  delete x;
  return 0;
}

// Searches the ring, tree and NVLS graphs of a topology (interNode: the job spans nodes, so channels attach to NICs)
// and writes them as graph XML into out. Returns 0 on success.
int b200TopoGraphs(const char* xmlText, int interNode, int crossNic, char* out, int outLen) {
  std::string err;
  XmlNode* x = xmlParse(xmlText, &err);
  if (!x) return 1;
  TopoSystem* s = topoFromXml(x, &err);
  if (!s) { delete x; return 2; }
  topoComputePaths(s);
  TopoGraph ring, tree, nvls;
  ring.pattern = PATTERN_RING;
  tree.pattern = PATTERN_BALANCED_TREE;
  nvls.pattern = PATTERN_NVLS;
  ring.inter = tree.inter = nvls.inter = interNode != 0;
  ring.crossNic = tree.crossNic = crossNic;
  topoSearch(s, &ring, 1, 32);
  topoSearch(s, &tree, 1, std::max(1, ring.nChannels));
  topoSearch(s, &nvls, 1, 32);
  XmlNode* gx = graphToXml({ring, tree, nvls});
  std::string t = xmlDump(gx);
  snprintf(out, outLen, "%s", t.c_str());
  delete gx;
  delete s;
  delete x;
  return (int)t.size() < outLen ? 0 : 3;
}

// Reads graphs 0..2 of a graph XML for ranks 0..nRanks-1 and writes them out again (the dump of what was understood).
// Returns 0, or 10 + the id of the first graph that was refused (message in out).
int b200TopoGraphReload(const char* graphXml, int nRanks, char* out, int outLen) {
  std::string err;
  XmlNode* gx = xmlParse(graphXml, &err);
  if (!gx) { snprintf(out, outLen, "%s", err.c_str()); return 1; }
  std::vector<int> ranks;
  for (int r = 0; r < nRanks; ++r) ranks.push_back(r);
  std::vector<TopoGraph> gs(3);
  for (int i = 0; i < 3; ++i) {
    if (graphFromXml(gx, i, ranks, &gs[i], &err) != ncclSuccess) { snprintf(out, outLen, "%s", err.c_str()); delete gx; return 10 + i; }
  }
  XmlNode* back = graphToXml(gs);
  std::string t = xmlDump(back);
  snprintf(out, outLen, "%s", t.c_str());
  delete back;
  delete gx;
  return 0;
}

// Probes this machine and writes its topology XML into out (truncated to outLen).
int b200TopoProbe(char* out, int outLen) {
  XmlNode* x = xmlFromSystem();
  std::string t = xmlDump(x);
  snprintf(out, outLen, "%s", t.c_str());
  delete x;
  return 0;
}

void b200Btree(int n, int rank, int* up, int* d0, int* d1) {
  int pct;
  getBtree(n, rank, up, d0, d1, &pct);
}
void b200Dtree(int n, int rank, int* out6) {
  int p0, p1;
  getDtree(n, rank, &out6[0], &out6[1], &out6[2], &p0, &out6[3], &out6[4], &out6[5], &p1);
}

}  // extern "C"
