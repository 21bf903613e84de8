// Channel-graph search, ring / tree construction.
// A channel is a walk through every local GPU that consumes its bandwidth on every link it crosses:
//   ring           closed walk (inside one node), or NET -> GPUs -> NET when the job spans nodes;
//   tree patterns  open chain whose links carry traffic in both directions; the network attaches at the
//                  first GPU (PATTERN_TREE) or is spread over the first two (balanced / split tree);
//   NVLS           one head GPU per channel; every GPU exchanges the channel's share with the switch.
// For each per-channel speed of the architecture's ladder (highest first) a depth-first search packs as many
// channels as the links carry; the graph with the largest total bandwidth wins. On a switch fabric every GPU
// pair is equivalent and the search collapses to "link bandwidth / speed" channels in rank order; on hybrid or
// PCI machines the search picks orders that avoid slow hops, and NICs are taken closest-first per channel.
// Graphs can be written to and read from XML (NCCL_GRAPH_DUMP_FILE / NCCL_GRAPH_FILE).
// Reference parity: src/graph/search.cc (speed ladders :1051-1067, ncclTopoCompute :1074-1313, NIC choice
// :437-520, graph XML :900-1040), src/graph/rings.cc (ncclBuildRings), src/graph/trees.cc (ncclGetBtree / ncclGetDtree).
#include <algorithm>
#include <functional>

#include <strings.h>

#include "topo.h"

namespace b200 {

static const float kSpeedsSm100[] = {90, 80, 70, 60, 50, 45, 40, 30, 24, 20, 19, 18};
static const float kSpeedsSm90[] = {60, 50, 40, 30, 24, 20, 15, 12, 11, 6, 3};
static const float kSpeedsOld[] = {40, 30, 20, 18, 15, 12, 10, 9, 7, 6, 5, 4, 3};

struct Residual {
  std::vector<std::vector<float>> bw;   // per node, per link
};

static int linkIndex(const TopoSystem* s, int from, int to, bool preferNvl) {
  int best = -1;
  for (size_t i = 0; i < s->nodes[from].links.size(); ++i) {
    const TopoLink& l = s->nodes[from].links[i];
    if (l.remNode != to) continue;
    if (best < 0 || (preferNvl && l.type == LINK_NVL)) best = (int)i;
  }
  return best;
}

// Consumes (sign=-1) or restores (sign=+1) `speed` along the path from a to b; false when a link is short.
static bool followPath(const TopoSystem* s, Residual* r, int a, int b, float speed, int sign) {
  if (a == b) return true;
  const TopoPath& p = s->nodes[a].paths[b];
  if (p.type == PATH_DIS || p.via.empty()) return false;
  int cur = a;
  std::vector<std::pair<int, int>> touched;
  for (int nxt : p.via) {
    int li = linkIndex(s, cur, nxt, p.type <= PATH_NVB);
    if (li < 0 || (sign < 0 && r->bw[cur][li] + 1e-3f < speed)) {
      for (auto& t : touched) r->bw[t.first][t.second] -= sign * speed;
      return false;
    }
    r->bw[cur][li] += sign * speed;
    touched.push_back({cur, li});
    cur = nxt;
  }
  return true;
}

// Both directions of a hop (tree links carry the reduction up and the broadcast down).
static bool followBoth(const TopoSystem* s, Residual* r, int a, int b, float speed, int sign) {
  if (!followPath(s, r, a, b, speed, sign)) return false;
  if (!followPath(s, r, b, a, speed, sign)) { followPath(s, r, a, b, speed, -sign); return false; }
  return true;
}

// NET nodes ordered for a GPU: best path class first, then widest, then rotated by channel so that
// equally close NICs share the channels. Reference parity: ncclTopoSelectNets (src/graph/search.cc:437-520).
static std::vector<int> netsFor(const TopoSystem* s, int gpuNode, int channel) {
  const std::vector<int>& nets = s->byType[TOPO_NET];
  std::vector<int> out;
  const int m = (int)nets.size();
  for (int k = 0; k < m; ++k) out.push_back(nets[(k + channel) % m]);
  std::stable_sort(out.begin(), out.end(), [&](int a, int b) {
    const TopoPath& pa = s->nodes[gpuNode].paths[a];
    const TopoPath& pb = s->nodes[gpuNode].paths[b];
    if (pa.type != pb.type) return pa.type < pb.type;
    return pa.bw > pb.bw;
  });
  return out;
}

struct ChannelPlan {
  std::vector<int> gpus;   // indices into byType[TOPO_GPU], in walk order
  int netIn = -1, netOut = -1;   // node indices of the NET nodes (-1 inside one node)
};

// One channel of `pattern` at the given speeds on the residual bandwidths; true when it fits (bandwidth consumed).
static bool placeChannel(const TopoSystem* s, Residual* res, int pattern, bool inter, int crossNic, float bwIntra, float bwInter, int ch, long* budget,
                         ChannelPlan* plan, int* worstIntra, int* worstInter) {
  const std::vector<int>& gpus = s->byType[TOPO_GPU];
  const int n = (int)gpus.size();
  const bool tree = pattern == PATTERN_TREE || pattern == PATTERN_BALANCED_TREE || pattern == PATTERN_SPLIT_TREE;
  auto hop = [&](int a, int b, float speed, int sign) { return tree ? followBoth(s, res, a, b, speed, sign) : followPath(s, res, a, b, speed, sign); };

  // candidate starts: inside one node the walk starts at GPU `ch % n` (rotation spreads link use); across nodes
  // every (NIC, closest GPU) pair is a candidate, NICs rotated by channel
  struct Start { int g; int net; };
  std::vector<Start> starts;
  if (!inter) {
    for (int k = 0; k < n; ++k) starts.push_back({(ch + k) % n, -1});
  } else {
    const std::vector<int>& nets = s->byType[TOPO_NET];
    const int m = (int)nets.size();
    for (int k = 0; k < m; ++k) {
      int net = nets[(ch + k) % m];
      std::vector<int> order(n);
      for (int i = 0; i < n; ++i) order[i] = i;
      std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
        const TopoPath& pa = s->nodes[net].paths[gpus[a]];
        const TopoPath& pb = s->nodes[net].paths[gpus[b]];
        if (pa.type != pb.type) return pa.type < pb.type;
        return pa.bw > pb.bw;
      });
      // only the GPUs of the best class for this NIC: a farther GPU would be served better by another NIC
      int bestType = s->nodes[net].paths[gpus[order[0]]].type;
      for (int g : order) if (s->nodes[net].paths[gpus[g]].type == bestType) starts.push_back({g, net});
    }
  }

  for (const Start& st : starts) {
    if (--*budget < 0) return false;
    std::vector<int> walk{st.g};
    std::vector<char> used(n, 0);
    used[st.g] = 1;
    int netOut = -1;
    // network entry
    if (st.net >= 0 && !followPath(s, res, st.net, gpus[st.g], bwInter, -1)) continue;
    std::function<bool()> dfs = [&]() -> bool {
      if (--*budget < 0) return false;
      const int cur = walk.back();
      if ((int)walk.size() == n) {
        if (!inter) return tree ? true : hop(gpus[cur], gpus[walk[0]], bwIntra, -1);
        // network exit: ring leaves from the last GPU; tree patterns talk to the network at the head of the chain
        int exitGpu = pattern == PATTERN_RING ? cur : (pattern == PATTERN_TREE || n < 2) ? walk[0] : walk[1];
        // rings leave through the NIC they entered by unless crossing is allowed; the tree patterns take the NIC closest
        // to the GPU that talks to the network (which spreads a chain's traffic over two NICs for balanced / split trees)
        std::vector<int> cand = (crossNic || pattern != PATTERN_RING) ? netsFor(s, gpus[exitGpu], ch) : std::vector<int>{st.net};
        if (pattern == PATTERN_RING && crossNic) {   // still the same NIC first
          auto it = std::find(cand.begin(), cand.end(), st.net);
          if (it != cand.end()) std::rotate(cand.begin(), it, it + 1);
        }
        for (int net : cand) {
          if (s->nodes[gpus[exitGpu]].paths[net].type == PATH_DIS) continue;
          if (followPath(s, res, gpus[exitGpu], net, bwInter, -1)) { netOut = net; return true; }
        }
        return false;
      }
      // closest unused GPUs first (best path class, then index order rotated by channel)
      std::vector<int> cand;
      for (int k = 1; k <= n; ++k) {
        int v = (cur + k + ch) % n;
        if (!used[v]) cand.push_back(v);
      }
      std::stable_sort(cand.begin(), cand.end(), [&](int a, int b) { return s->nodes[gpus[cur]].paths[gpus[a]].type < s->nodes[gpus[cur]].paths[gpus[b]].type; });
      for (int v : cand) {
        if (!hop(gpus[cur], gpus[v], bwIntra, -1)) continue;
        used[v] = 1;
        walk.push_back(v);
        if (dfs()) return true;
        walk.pop_back();
        used[v] = 0;
        hop(gpus[cur], gpus[v], bwIntra, +1);
      }
      return false;
    };
    if (dfs()) {
      plan->gpus = walk;
      plan->netIn = st.net;
      plan->netOut = netOut;
      for (int i = 0; i + 1 < n; ++i) *worstIntra = std::max(*worstIntra, s->nodes[gpus[walk[i]]].paths[gpus[walk[i + 1]]].type);
      if (!inter && !tree && n > 1) *worstIntra = std::max(*worstIntra, s->nodes[gpus[walk[n - 1]]].paths[gpus[walk[0]]].type);
      if (st.net >= 0) *worstInter = std::max(*worstInter, s->nodes[st.net].paths[gpus[st.g]].type);
      return true;
    }
    if (st.net >= 0) followPath(s, res, st.net, gpus[st.g], bwInter, +1);
  }
  return false;
}

// NVLS channel with head `h`: the switch reads the channel's share from every GPU and the head writes the result
// back through the switch to every GPU, so every GPU's link to the switch carries `speed` in both directions.
static bool placeNvlsChannel(const TopoSystem* s, Residual* res, int h, float speed) {
  const std::vector<int>& gpus = s->byType[TOPO_GPU];
  if (s->byType[TOPO_NVS].empty()) return false;
  const int nvs = s->byType[TOPO_NVS][0];
  std::vector<int> done;
  for (int g : gpus) {
    if (s->nodes[g].paths[nvs].type != PATH_NVL || !followBoth(s, res, g, nvs, speed, -1)) {
      for (int d : done) followBoth(s, res, d, nvs, speed, +1);
      return false;
    }
    done.push_back(g);
  }
  (void)h;
  return true;
}

ncclResult_t topoSearch(const TopoSystem* s, TopoGraph* g, int minChannels, int maxChannels) {
  const std::vector<int>& gpus = s->byType[TOPO_GPU];
  const int n = (int)gpus.size();
  const int pattern = g->pattern;
  const bool inter = g->inter && !s->byType[TOPO_NET].empty();
  g->nChannels = 0;
  g->order.clear();
  g->nets.clear();
  g->heads.clear();
  g->bwIntra = g->bwInter = 0;
  g->typeIntra = PATH_LOC;
  g->typeInter = inter ? PATH_NET : PATH_LOC;
  if (n == 0) return ncclSuccess;
  if (g->crossNic < 0) g->crossNic = 0;
  int crossNic = g->crossNic;
  if (const char* e = getEnv("NCCL_CROSS_NIC")) { if (*e) crossNic = atoi(e) != 0; }   // 2 ("let the search decide") counts as allowed
  if (n == 1 && !inter) {
    if (pattern == PATTERN_NVLS) return ncclSuccess;   // nothing to reduce in a switch
    g->nChannels = std::max(1, minChannels);
    g->order.assign(g->nChannels, std::vector<int>{s->nodes[gpus[0]].rank});
    g->nets.assign(g->nChannels, {-1, -1});
    g->bwIntra = kLocBw;
    return ncclSuccess;
  }
  int cc = s->nodes[gpus[0]].cudaCompCap;
  const float* ladder = cc >= 100 ? kSpeedsSm100 : cc >= 90 ? kSpeedsSm90 : kSpeedsOld;
  int nl = cc >= 100 ? 12 : cc >= 90 ? 11 : 13;
  float bestTotal = 0;
  for (int si = 0; si < nl; ++si) {
    const float speed = ladder[si];
    Residual res;
    res.bw.resize(s->nodes.size());
    for (size_t i = 0; i < s->nodes.size(); ++i) for (auto& l : s->nodes[i].links) res.bw[i].push_back(l.bw);
    std::vector<std::vector<int>> orders;
    std::vector<std::array<int, 2>> nets;
    std::vector<int> heads;
    int worstIntra = PATH_LOC, worstInter = inter ? PATH_LOC : PATH_LOC;
    long budget = 200000;   // search steps for this speed
    if (pattern == PATTERN_NVLS) {
      // one head per GPU, in rank order; all heads or none (a partial set would unbalance the shares)
      const int want = std::min(n, maxChannels);
      for (int h = 0; h < want; ++h) {
        if (!placeNvlsChannel(s, &res, h, speed)) break;
        heads.push_back(s->nodes[gpus[h]].rank);
      }
      if ((int)heads.size() != want) heads.clear();
      for (size_t h = 0; h < heads.size(); ++h) {
        std::vector<int> ranks;
        for (int i = 0; i < n; ++i) ranks.push_back(s->nodes[gpus[(h + i) % n]].rank);
        orders.push_back(ranks);
        nets.push_back({-1, -1});
      }
      worstIntra = PATH_NVL;
    } else {
      for (int ch = 0; ch < maxChannels; ++ch) {
        ChannelPlan plan;
        if (!placeChannel(s, &res, pattern, inter, crossNic, speed, speed, ch, &budget, &plan, &worstIntra, &worstInter)) break;
        std::vector<int> ranks;
        for (int gi : plan.gpus) ranks.push_back(s->nodes[gpus[gi]].rank);
        orders.push_back(ranks);
        nets.push_back({plan.netIn >= 0 ? (int)s->nodes[plan.netIn].id : -1, plan.netOut >= 0 ? (int)s->nodes[plan.netOut].id : -1});
      }
    }
    const float total = speed * orders.size();
    if ((int)orders.size() >= minChannels && !orders.empty() && total > bestTotal * 1.01f) {
      bestTotal = total;
      g->nChannels = (int)orders.size();
      g->order = orders;
      g->nets = nets;
      g->heads = heads;
      g->bwIntra = speed;
      g->bwInter = speed;
      g->typeIntra = worstIntra;
      g->typeInter = inter ? worstInter : PATH_LOC;
    }
  }
  if (g->nChannels == 0 && pattern != PATTERN_NVLS) {
    // nothing fits even the lowest speed: one channel in rank order
    std::vector<int> ranks;
    for (int gi : gpus) ranks.push_back(s->nodes[gi].rank);
    g->nChannels = 1;
    g->order.assign(1, ranks);
    int net = inter ? (int)s->nodes[s->byType[TOPO_NET][0]].id : -1;
    g->nets.assign(1, {net, net});
    g->bwIntra = g->bwInter = ladder[nl - 1];
    g->typeIntra = PATH_SYS;
  }
  return ncclSuccess;
}

static int pathTypeByName(const char* name) {
  for (int t = 0; t <= PATH_DIS; ++t) if (name && !strcasecmp(name, topoPathName(t))) return t;
  return PATH_DIS;
}

XmlNode* graphToXml(const std::vector<TopoGraph>& graphs) {
  XmlNode* root = new XmlNode;
  root->name = "graphs";
  root->setAttr("version", "1");
  int id = 0;
  for (auto& g : graphs) {
    XmlNode* x = root->addSub("graph");
    x->setAttr("id", std::to_string(id++));
    x->setAttr("pattern", std::to_string(g.pattern));
    x->setAttr("crossnic", std::to_string(g.crossNic));
    x->setAttr("nchannels", std::to_string(g.nChannels));
    x->setAttr("speedintra", std::to_string(g.bwIntra));
    x->setAttr("speedinter", std::to_string(g.bwInter));
    x->setAttr("latencyinter", std::to_string(g.latencyInter));
    x->setAttr("typeintra", topoPathName(g.typeIntra));
    x->setAttr("typeinter", topoPathName(g.typeInter));
    x->setAttr("samechannels", std::to_string(g.sameChannels));
    for (size_t c = 0; c < g.order.size(); ++c) {
      XmlNode* ch = x->addSub("channel");
      const bool hasNet = c < g.nets.size() && g.nets[c][0] >= 0;
      if (hasNet) ch->addSub("net")->setAttr("dev", std::to_string(g.nets[c][0]));
      for (int r : g.order[c]) ch->addSub("gpu")->setAttr("dev", std::to_string(r));
      if (hasNet) ch->addSub("net")->setAttr("dev", std::to_string(g.nets[c][1] >= 0 ? g.nets[c][1] : g.nets[c][0]));
    }
  }
  return root;
}

// Reads the graph with the given id back. The channels must each visit every rank in `ranks` exactly once.
ncclResult_t graphFromXml(const XmlNode* root, int id, const std::vector<int>& ranks, TopoGraph* g, std::string* err) {
  if (!root || root->name != "graphs") { if (err) *err = "no <graphs> element"; return ncclInvalidUsage; }
  for (const XmlNode* x : root->subs) {
    if (x->name != "graph" || x->attrInt("id", -1) != id) continue;
    TopoGraph out = *g;
    out.pattern = x->attrInt("pattern", g->pattern);
    out.crossNic = x->attrInt("crossnic", 0);
    out.bwIntra = (float)x->attrFloat("speedintra", 0);
    out.bwInter = (float)x->attrFloat("speedinter", 0);
    out.latencyInter = (float)x->attrFloat("latencyinter", 0);
    out.typeIntra = pathTypeByName(x->attr("typeintra"));
    out.typeInter = pathTypeByName(x->attr("typeinter"));
    out.sameChannels = x->attrInt("samechannels", 1);
    out.order.clear();
    out.nets.clear();
    out.heads.clear();
    for (const XmlNode* ch : x->subs) {
      if (ch->name != "channel") continue;
      std::vector<int> order;
      std::array<int, 2> nets{-1, -1};
      for (const XmlNode* e : ch->subs) {
        if (e->name == "gpu") order.push_back(e->attrInt("dev", -1));
        else if (e->name == "net") nets[order.empty() ? 0 : 1] = e->attrInt("dev", -1);
      }
      std::vector<int> a = order, b = ranks;
      std::sort(a.begin(), a.end());
      std::sort(b.begin(), b.end());
      if (a != b) { if (err) *err = "channel " + std::to_string(out.order.size()) + " of graph " + std::to_string(id) + " does not visit every local rank exactly once"; return ncclInvalidUsage; }
      out.order.push_back(order);
      out.nets.push_back(nets);
      if (out.pattern == PATTERN_NVLS) out.heads.push_back(order[0]);
    }
    out.nChannels = (int)out.order.size();
    if (x->attrInt("nchannels", out.nChannels) != out.nChannels) { if (err) *err = "nchannels does not match the number of <channel> elements"; return ncclInvalidUsage; }
    *g = out;
    return ncclSuccess;
  }
  if (err) *err = "graph " + std::to_string(id) + " not found";
  return ncclInvalidArgument;
}

// ---------------------------------------------------------------- rings and trees
ncclResult_t buildRing(int nRanks, const std::vector<int>& order, std::vector<int>* prev, std::vector<int>* next) {
  if ((int)order.size() != nRanks) return ncclInternalError;
  prev->assign(nRanks, -1);
  next->assign(nRanks, -1);
  std::vector<char> seen(nRanks, 0);
  for (int i = 0; i < nRanks; ++i) {
    int r = order[i];
    if (r < 0 || r >= nRanks || seen[r]) { WARN("ring order is not a permutation of the ranks"); return ncclInternalError; }
    seen[r] = 1;
    (*next)[r] = order[(i + 1) % nRanks];
    (*prev)[r] = order[(i + nRanks - 1) % nRanks];
  }
  return ncclSuccess;
}

// In-order binary tree: the lowest set bit of a rank decides its level (odd ranks are leaves, ranks
// with lowest bit 2 sit one level up, and so on). Rank 0 is the root and has a single child, the
// largest power of two below nRanks; a rank whose computed parent or child falls outside
// [0, nRanks) is re-attached to the nearest existing rank on the same side.
void getBtree(int nRanks, int rank, int* u, int* d0, int* d1, int* parentChildType) {
  int up, down0, down1;
  int bit;
  for (bit = 1; bit < nRanks; bit <<= 1) if (bit & rank) break;
  if (rank == 0) {
    *u = -1;
    *d0 = -1;
    // the child of the root is the largest power of two below nRanks
    *d1 = nRanks > 1 ? bit >> 1 : -1;
    *parentChildType = 0;
    return;
  }
  up = (rank ^ bit) | (bit << 1);
  if (up >= nRanks) up = rank ^ bit;   // the natural parent does not exist: climb the other way
  *parentChildType = rank < up ? 0 : 1;
  *u = up;
  int lowbit = bit >> 1;
  down0 = lowbit == 0 ? -1 : rank - lowbit;
  down1 = lowbit == 0 ? -1 : rank + lowbit;
  while (down1 >= nRanks) {   // shrink the right subtree until it fits
    down1 = lowbit == 0 ? -1 : rank + lowbit;
    lowbit >>= 1;
  }
  *d0 = down0;
  *d1 = down1;
}

void getDtree(int nRanks, int rank, int* s0, int* d0_0, int* d0_1, int* pct0, int* s1, int* d1_0, int* d1_1, int* pct1) {
  getBtree(nRanks, rank, s0, d0_0, d0_1, pct0);
  if (nRanks % 2 == 1) {
    // odd: second tree is the first one shifted by one rank
    int shifted = (rank - 1 + nRanks) % nRanks;
    int u, a, b;
    getBtree(nRanks, shifted, &u, &a, &b, pct1);
    *s1 = u == -1 ? -1 : (u + 1) % nRanks;
    *d1_0 = a == -1 ? -1 : (a + 1) % nRanks;
    *d1_1 = b == -1 ? -1 : (b + 1) % nRanks;
  } else {
    // even: second tree is the mirror image
    int u, a, b;
    getBtree(nRanks, nRanks - 1 - rank, &u, &a, &b, pct1);
    *s1 = u == -1 ? -1 : nRanks - 1 - u;
    *d1_0 = a == -1 ? -1 : nRanks - 1 - a;
    *d1_1 = b == -1 ? -1 : nRanks - 1 - b;
  }
}

}  // namespace b200
