// System graph from the topology XML, all-pairs paths, and the communicator-level entry points.
// Reference parity: src/graph/topo.cc (ncclTopoGetSystemFromXml :958, link helpers :92-197,
// NVLink targets :811), src/graph/paths.cc (ncclTopoSetPaths :38, ncclTopoCheckP2p :298,
// ncclTopoComputePaths :721).
#include "topo.h"

#include <stdio.h>

#include <algorithm>
#include <deque>
#include <fstream>

namespace b200 {

const char* topoPathName(int t) {
  static const char* n[] = {"LOC", "NVL", "NVB", "C2C", "PIX", "PXB", "PXN", "PHB", "SYS", "NET", "DIS"};
  return t >= 0 && t <= PATH_DIS ? n[t] : "?";
}

int TopoSystem::find(int type, int64_t id) const {
  for (int i : byType[type]) if (nodes[i].id == id) return i;
  return -1;
}

static int addNode(TopoSystem* s, int type, int64_t id, const std::string& name) {
  int i = s->find(type, id);
  if (i >= 0) return i;
  TopoNode n;
  n.type = type;
  n.id = id;
  n.name = name;
  s->nodes.push_back(n);
  s->byType[type].push_back((int)s->nodes.size() - 1);
  return (int)s->nodes.size() - 1;
}

static void addLink(TopoSystem* s, int a, int b, int type, float bw) {
  for (auto& l : s->nodes[a].links) if (l.remNode == b && l.type == type) { l.bw += bw; goto back; }
  s->nodes[a].links.push_back(TopoLink{type, bw, b});
back:
  for (auto& l : s->nodes[b].links) if (l.remNode == a && l.type == type) { l.bw += bw; return; }
  s->nodes[b].links.push_back(TopoLink{type, bw, a});
}

// "32.0 GT/s PCIe" x16 -> GB/s relative to the Gen3 x16 reference value
static float pciBw(const XmlNode* pci) {
  const char* sp = pci->attr("link_speed");
  float gts = sp ? (float)atof(sp) : 8.0f;
  if (gts <= 0) gts = 8.0f;
  int width = pci->attrInt("link_width", 16);
  if (width <= 0) width = 16;
  return kPciBw * (gts / 8.0f) * (width / 16.0f);
}

struct NvlinkTodo { int gpu; int64_t target; int count; bool toSwitch; };

static void walkPci(TopoSystem* s, const XmlNode* x, int parent, float bwToParent, std::vector<NvlinkTodo>* nvl) {
  for (auto* c : x->subs) {
    if (c->name == "pci") {
      const char* bus = c->attr("busid");
      int64_t id = bus ? busIdToInt64(bus) : 0;
      bool leaf = c->findSub("gpu") || c->findSub("nic");
      float bw = pciBw(c);
      if (leaf) {
        // the device hangs directly on `parent`; no separate node for its own function
        const XmlNode* cc = c;
        for (auto* d : cc->subs) {
          if (d->name == "gpu") {
            int g = addNode(s, TOPO_GPU, id, bus ? bus : "gpu");
            s->nodes[g].dev = d->attrInt("dev", -1);
            s->nodes[g].rank = d->attrInt("rank", s->nodes[g].dev);
            s->nodes[g].cudaCompCap = d->attrInt("sm", 0);
            addLink(s, g, parent, LINK_PCI, bw);
            for (auto* l : d->subs) {
              if (l->name != "nvlink") continue;
              const char* tgt = l->attr("target");
              const char* tclass = l->attr("tclass");
              bool sw = !tclass || strtol(tclass, nullptr, 0) == 0x068000;
              nvl->push_back(NvlinkTodo{g, tgt ? busIdToInt64(tgt) : 0, l->attrInt("count", 1), sw});
            }
          } else if (d->name == "nic") {
            int nic = addNode(s, TOPO_NIC, id, bus ? bus : "nic");
            addLink(s, nic, parent, LINK_PCI, bw);
            for (auto* nn : d->subs) {
              if (nn->name != "net") continue;
              int net = addNode(s, TOPO_NET, nn->attrInt("dev", 0), nn->attr("name") ? nn->attr("name") : "net");
              float nbw = (float)nn->attrFloat("speed", 10000) / 8000.0f;   // Mb/s -> GB/s
              s->nodes[net].netBw = nbw;
              addLink(s, net, nic, LINK_NET, nbw);
            }
          }
        }
      } else {
        int sw = addNode(s, TOPO_PCI, id, bus ? bus : "pci");
        addLink(s, sw, parent, LINK_PCI, bw);
        walkPci(s, c, sw, bw, nvl);
      }
    }
  }
}

TopoSystem* topoFromXml(const XmlNode* root, std::string* err) {
  if (!root || root->name != "system") { if (err) *err = "top element must be <system>"; return nullptr; }
  TopoSystem* s = new TopoSystem;
  std::vector<NvlinkTodo> nvl;
  for (auto* c : root->subs) {
    if (c->name != "cpu") continue;
    int cpu = addNode(s, TOPO_CPU, c->attrInt("numaid", 0), std::string("cpu") + (c->attr("numaid") ? c->attr("numaid") : "0"));
    walkPci(s, c, cpu, 0, &nvl);
  }
  // CPUs of one machine talk over the socket interconnect
  for (size_t i = 0; i < s->byType[TOPO_CPU].size(); ++i)
    for (size_t j = i + 1; j < s->byType[TOPO_CPU].size(); ++j) addLink(s, s->byType[TOPO_CPU][i], s->byType[TOPO_CPU][j], LINK_SYS, 16.0f);
  // NVLinks: GPU to GPU, or GPU to the (single) switch fabric
  int nvs = -1;
  for (auto& t : nvl) {
    float per = s->nodes[t.gpu].cudaCompCap >= 100 ? kNvlinkBwSm100 : kNvlinkBwSm90;
    if (t.toSwitch) {
      if (nvs < 0) nvs = addNode(s, TOPO_NVS, 0, "nvswitch");
      bool have = false;
      for (auto& l : s->nodes[t.gpu].links) if (l.remNode == nvs) have = true;
      if (!have) addLink(s, t.gpu, nvs, LINK_NVL, per * t.count);
    } else {
      int peer = s->find(TOPO_GPU, t.target);
      if (peer < 0 || peer == t.gpu) continue;
      bool have = false;
      for (auto& l : s->nodes[t.gpu].links) if (l.remNode == peer && l.type == LINK_NVL) have = true;
      if (!have) addLink(s, t.gpu, peer, LINK_NVL, per * t.count);
    }
  }
  if (s->byType[TOPO_GPU].empty() && s->byType[TOPO_NET].empty() && s->byType[TOPO_CPU].empty()) {
    if (err) *err = "topology has no devices";
    delete s;
    return nullptr;
  }
  return s;
}

// Class of a path from the sequence of link types / intermediate nodes it crosses.
static int classify(const TopoSystem* s, int from, const std::vector<int>& via, const std::vector<int>& linkTypes) {
  if (via.empty()) return PATH_LOC;
  bool allNvl = true;
  int cpus = 0, pciSwitches = 0, gpusBetween = 0;
  bool net = false, sys = false;
  for (size_t i = 0; i < via.size(); ++i) {
    int lt = linkTypes[i];
    if (lt != LINK_NVL) allNvl = false;
    // the hop between a NIC and its network port says nothing about distance inside the machine: a path that starts
    // or ends at a NET node is classed by its PCI / NVLink part; only traffic that crosses the network is PATH_NET
    if (lt == LINK_NET && i != 0 && i + 1 != via.size()) net = true;
    if (lt == LINK_NET) continue;
    if (lt == LINK_SYS) sys = true;
    if (i + 1 < via.size()) {
      const TopoNode& mid = s->nodes[via[i]];
      if (mid.type == TOPO_CPU) ++cpus;
      if (mid.type == TOPO_PCI) ++pciSwitches;
      if (mid.type == TOPO_GPU) ++gpusBetween;
    }
  }
  if (net) return PATH_NET;
  if (allNvl) return gpusBetween ? PATH_NVB : PATH_NVL;
  if (gpusBetween) return PATH_PXN;   // NVLink to a peer GPU, then that GPU's PCI links (how a GPU reaches a NIC it is not close to)
  if (sys || cpus > 1) return PATH_SYS;
  if (cpus == 1) return PATH_PHB;
  if (pciSwitches > 1) return PATH_PXB;
  return PATH_PIX;
}

void topoComputePaths(TopoSystem* s) {
  const int N = (int)s->nodes.size();
  s->maxBw = 0;
  for (int src = 0; src < N; ++src) {
    auto& paths = s->nodes[src].paths;
    paths.assign(N, TopoPath{});
    // breadth-first search, widest path among the shortest; NVLink hops are preferred over PCI by
    // exploring them first
    std::vector<int> prev(N, -1), prevLink(N, -1), hops(N, 1 << 20);
    std::vector<float> bw(N, 0);
    std::deque<int> q;
    hops[src] = 0;
    bw[src] = kLocBw;
    q.push_back(src);
    while (!q.empty()) {
      int u = q.front();
      q.pop_front();
      // a GPU may only forward NVLink traffic (relay through a GPU), never PCI traffic
      std::vector<TopoLink> links = s->nodes[u].links;
      std::stable_sort(links.begin(), links.end(), [](const TopoLink& a, const TopoLink& b) { return a.type < b.type; });
      for (auto& l : links) {
        int v = l.remNode;
        if (u != src && s->nodes[u].type == TOPO_GPU && l.type != LINK_NVL) continue;
        if (u != src && s->nodes[u].type == TOPO_NET) continue;
        float nb = std::min(bw[u], l.bw);
        if (hops[u] + 1 < hops[v] || (hops[u] + 1 == hops[v] && nb > bw[v] && prevLink[v] >= l.type)) {
          bool first = hops[v] == (1 << 20);
          hops[v] = hops[u] + 1;
          bw[v] = nb;
          prev[v] = u;
          prevLink[v] = l.type;
          if (first) q.push_back(v);
        }
      }
    }
    for (int dst = 0; dst < N; ++dst) {
      TopoPath& p = paths[dst];
      if (dst == src) { p.type = PATH_LOC; p.bw = kLocBw; p.hops = 0; continue; }
      if (prev[dst] < 0) continue;
      std::vector<int> via, lts;
      for (int v = dst; v != src; v = prev[v]) { via.push_back(v); lts.push_back(prevLink[v]); }
      std::reverse(via.begin(), via.end());
      std::reverse(lts.begin(), lts.end());
      p.via = via;
      p.hops = (int)via.size();
      p.bw = bw[dst];
      p.type = classify(s, src, via, lts);
      if (s->nodes[src].type == TOPO_GPU && s->nodes[dst].type == TOPO_GPU) s->maxBw = std::max(s->maxBw, p.bw);
    }
  }
  s->totalBw = 0;
  for (int g : s->byType[TOPO_GPU]) {
    float t = 0;
    for (auto& l : s->nodes[g].links) if (l.type == LINK_NVL) t += l.bw;
    s->totalBw = std::max(s->totalBw, t > 0 ? t : kPciBw);
  }
}

static int gpuByRank(const TopoSystem* s, int rank) {
  for (int g : s->byType[TOPO_GPU]) if (s->nodes[g].rank == rank) return g;
  return -1;
}

int topoGpuPathType(const TopoSystem* s, int a, int b, float* bw) {
  int ga = gpuByRank(s, a), gb = gpuByRank(s, b);
  if (ga < 0 || gb < 0 || s->nodes[ga].paths.empty()) return PATH_DIS;
  if (bw) *bw = s->nodes[ga].paths[gb].bw;
  return s->nodes[ga].paths[gb].type;
}

bool topoCheckP2p(const TopoSystem* s, int a, int b, int* pathType) {
  int t = topoGpuPathType(s, a, b);
  if (pathType) *pathType = t;
  // peer access is used up to "same CPU root complex" (PHB) by default; NCCL_P2P_LEVEL narrows it
  int level = PATH_PHB;
  const char* e = getEnv("NCCL_P2P_LEVEL");
  if (e) {
    for (int i = 0; i <= PATH_SYS; ++i) if (!strcasecmp(e, topoPathName(i))) level = i;
  }
  return t <= level;
}

std::string topoDescribe(const TopoSystem* s) {
  std::string out;
  char line[256];
  static const char* tn[] = {"GPU", "PCI", "NVS", "CPU", "NIC", "NET"};
  static const char* ln[] = {"LOC", "NVL", "C2C", "PCI", "SYS", "NET"};
  for (auto& n : s->nodes) {
    snprintf(line, sizeof(line), "%s/%llx (%s)", tn[n.type], (unsigned long long)n.id, n.name.c_str());
    out += line;
    for (auto& l : n.links) {
      snprintf(line, sizeof(line), "  +%s[%.1f]-%s/%llx", ln[l.type], l.bw, tn[s->nodes[l.remNode].type], (unsigned long long)s->nodes[l.remNode].id);
      out += line;
    }
    out += "\n";
  }
  return out;
}

// ---------------------------------------------------------------- communicator entry points
ncclResult_t topoInit(ncclComm* comm) {
  TopoState* st = new TopoState;
  comm->topo = st;
  std::string err;
  const char* file = getEnv("NCCL_TOPO_FILE");
  if (file && *file) {
    st->xml = xmlLoadFile(file, &err);
    if (!st->xml) { WARN("NCCL_TOPO_FILE %s: %s", file, err.c_str()); return ncclInvalidUsage; }
    INFO(SUB_GRAPH, "Loaded topology from %s", file);
  } else {
    st->xml = xmlFromSystem();
    // tag my GPU with my rank; peers on this host contribute theirs through the bootstrap
    struct Tag { int64_t busId; int rank; int dev; };
    std::vector<Tag> tags(comm->nRanks);
    tags[comm->rank] = Tag{comm->peers[comm->rank].busId, comm->rank, comm->cudaDev};
    for (int r = 0; r < comm->nRanks; ++r) tags[r] = Tag{comm->peers[r].busId, r, comm->peers[r].cudaDev};
    std::vector<XmlNode*> stack{st->xml};
    while (!stack.empty()) {
      XmlNode* n = stack.back();
      stack.pop_back();
      if (n->name == "pci" && n->findSub("gpu")) {
        int64_t id = busIdToInt64(n->attr("busid") ? n->attr("busid") : "");
        for (auto& t : tags)
          if (t.busId == id && comm->peers[t.rank].hostHash == comm->peers[comm->rank].hostHash) n->findSub("gpu")->setAttr("rank", std::to_string(t.rank));
      }
      for (auto* c : n->subs) stack.push_back(c);
    }
  }
  const char* dump = getEnv("NCCL_TOPO_DUMP_FILE");
  const char* dumpRank = getEnv("NCCL_TOPO_DUMP_FILE_RANK");
  if (dump && *dump && (dumpRank && *dumpRank ? comm->rank == atoi(dumpRank) : comm->localRank == 0)) {
    std::ofstream f(dump);
    f << xmlDump(st->xml);
  }
  st->sys = topoFromXml(st->xml, &err);
  if (!st->sys) { WARN("topology: %s", err.c_str()); return ncclInternalError; }
  topoComputePaths(st->sys);
  if (debugLevel() >= LOG_INFO) INFO(SUB_GRAPH, "=== System ===\n%s", topoDescribe(st->sys).c_str());
  // channel graphs for the three patterns and the analytic model on top of them; NCCL_GRAPH_FILE replaces the search
  const bool inter = comm->nNodes > 1;
  st->ring.pattern = PATTERN_RING;
  st->tree.pattern = PATTERN_BALANCED_TREE;
  st->nvls.pattern = PATTERN_NVLS;
  st->ring.inter = st->tree.inter = st->nvls.inter = inter;
  std::vector<int> localRanks;
  for (int gi : st->sys->byType[TOPO_GPU]) localRanks.push_back(st->sys->nodes[gi].rank);
  bool loaded = false;
  const char* gfile = getEnv("NCCL_GRAPH_FILE");
  if (gfile && *gfile) {
    XmlNode* gx = xmlLoadFile(gfile, &err);
    TopoGraph* gs[3] = {&st->ring, &st->tree, &st->nvls};
    loaded = gx != nullptr;
    for (int i = 0; loaded && i < 3; ++i) {
      ncclResult_t r = graphFromXml(gx, i, localRanks, gs[i], &err);
      if (r == ncclInvalidArgument && i == 2) { st->nvls.nChannels = 0; continue; }   // a file without an NVLS graph switches it off
      if (r != ncclSuccess) loaded = false;
    }
    if (!loaded) WARN("NCCL_GRAPH_FILE %s: %s; searching instead", gfile, err.c_str());
    else INFO(SUB_GRAPH, "Loaded channel graphs from %s", gfile);
    delete gx;
  }
  if (!loaded) {
    topoSearch(st->sys, &st->ring, 1, 32);
    // trees share the ring's channel count where the links allow it, so that both serve the same launches
    topoSearch(st->sys, &st->tree, 1, std::max(1, st->ring.nChannels));
    st->tree.sameChannels = st->tree.nChannels == st->ring.nChannels;
    if (!st->sys->byType[TOPO_NVS].empty() && comm->compCap >= 90) topoSearch(st->sys, &st->nvls, 1, 32);
    else st->nvls.nChannels = 0;
  }
  topoTuneModel(st->sys, &st->ring, &st->tree, &st->nvls, comm->nRanks, comm->nNodes, comm->compCap, &st->model);
  const char* gdump = getEnv("NCCL_GRAPH_DUMP_FILE");
  const char* gdumpRank = getEnv("NCCL_GRAPH_DUMP_FILE_RANK");
  if (gdump && *gdump && comm->rank == (gdumpRank && *gdumpRank ? atoi(gdumpRank) : 0)) {
    XmlNode* gx = graphToXml({st->ring, st->tree, st->nvls});
    std::ofstream f(gdump);
    f << xmlDump(gx);
    delete gx;
  }
  INFO(SUB_GRAPH, "ring graph: %d channels at %.1f GB/s (%s); tree graph: %d at %.1f; NVLS heads %d at %.1f", st->ring.nChannels, st->ring.bwIntra,
       topoPathName(st->ring.typeIntra), st->tree.nChannels, st->tree.bwIntra, st->nvls.nChannels, st->nvls.bwIntra);
  return ncclSuccess;
}

void topoDestroy(ncclComm* comm) {
  TopoState* st = comm->topo;
  if (!st) return;
  delete st->xml;
  delete st->sys;
  delete st;
  comm->topo = nullptr;
}

}  // namespace b200
