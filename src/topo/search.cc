// Channel-graph search, ring / tree construction.
// A channel is a ring through every local GPU; each channel consumes its bandwidth on every link
// of the paths it follows. For each per-channel speed of the architecture's ladder (highest
// first) a depth-first search packs as many rings as the links carry; the graph with the largest
// total bandwidth wins. On a switch fabric every GPU pair is equivalent and the search collapses
// to "link bandwidth / speed" channels in rank order; on hybrid or PCI machines the search picks
// orders that avoid slow hops.
// Reference parity: src/graph/search.cc (speed ladders :1051-1067, ncclTopoCompute :1074-1313),
// src/graph/rings.cc (ncclBuildRings), src/graph/trees.cc (ncclGetBtree / ncclGetDtree).
#include <algorithm>
#include <functional>

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
  const TopoPath& p = s->nodes[a].paths[b];
  if (p.type == PATH_DIS || p.via.empty()) return false;
  int cur = a;
  std::vector<std::pair<int, int>> touched;
  for (int nxt : p.via) {
    int li = linkIndex(s, cur, nxt, p.type <= PATH_NVB);
    if (li < 0) return false;
    if (sign < 0 && r->bw[cur][li] + 1e-3f < speed) {
      for (auto& t : touched) r->bw[t.first][t.second] += speed;
      return false;
    }
    r->bw[cur][li] += sign * speed;
    touched.push_back({cur, li});
    cur = nxt;
  }
  return true;
}

ncclResult_t topoSearch(const TopoSystem* s, TopoGraph* g, int minChannels, int maxChannels) {
  const std::vector<int>& gpus = s->byType[TOPO_GPU];
  const int n = (int)gpus.size();
  g->nChannels = 0;
  g->order.clear();
  g->bwIntra = g->bwInter = 0;
  g->typeIntra = PATH_LOC;
  if (n == 0) return ncclSuccess;
  if (n == 1) {
    g->nChannels = std::max(1, minChannels);
    g->order.assign(g->nChannels, std::vector<int>{s->nodes[gpus[0]].rank});
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
    std::vector<std::vector<int>> rings;
    int worstType = PATH_LOC;
    long budget = 200000;   // search steps for this speed
    for (int ch = 0; ch < maxChannels; ++ch) {
      std::vector<int> ring{0};
      std::vector<char> used(n, 0);
      used[0] = 1;
      bool found = false;
      std::function<bool()> dfs = [&]() -> bool {
        if (--budget < 0) return false;
        int cur = ring.back();
        if ((int)ring.size() == n) {
          if (!followPath(s, &res, gpus[cur], gpus[0], speed, -1)) return false;
          return true;
        }
        // try the closest unused GPUs first (best path class, then index order rotated by channel)
        std::vector<int> cand;
        for (int k = 1; k <= n; ++k) {
          int v = (cur + k + ch) % n;
          if (!used[v]) cand.push_back(v);
        }
        std::stable_sort(cand.begin(), cand.end(), [&](int a, int b) { return s->nodes[gpus[cur]].paths[gpus[a]].type < s->nodes[gpus[cur]].paths[gpus[b]].type; });
        for (int v : cand) {
          if (!followPath(s, &res, gpus[cur], gpus[v], speed, -1)) continue;
          used[v] = 1;
          ring.push_back(v);
          if (dfs()) return true;
          ring.pop_back();
          used[v] = 0;
          followPath(s, &res, gpus[cur], gpus[v], speed, +1);
        }
        return false;
      };
      found = dfs();
      if (!found) break;
      std::vector<int> ranks;
      for (int i = 0; i < n; ++i) {
        ranks.push_back(s->nodes[gpus[ring[i]]].rank);
        worstType = std::max(worstType, s->nodes[gpus[ring[i]]].paths[gpus[ring[(i + 1) % n]]].type);
      }
      rings.push_back(ranks);
    }
    const float total = speed * rings.size();
    if ((int)rings.size() >= minChannels && total > bestTotal * 1.01f) {
      bestTotal = total;
      g->nChannels = (int)rings.size();
      g->order = rings;
      g->bwIntra = speed;
      g->bwInter = speed;
      g->typeIntra = worstType;
    }
  }
  if (g->nChannels == 0) {
    // nothing fits even the lowest speed: one channel in rank order
    std::vector<int> ranks;
    for (int gi : gpus) ranks.push_back(s->nodes[gi].rank);
    g->nChannels = 1;
    g->order.assign(1, ranks);
    g->bwIntra = ladder[nl - 1];
    g->typeIntra = PATH_SYS;
  }
  return ncclSuccess;
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
    x->setAttr("nchannels", std::to_string(g.nChannels));
    x->setAttr("speedintra", std::to_string(g.bwIntra));
    x->setAttr("speedinter", std::to_string(g.bwInter));
    x->setAttr("typeintra", topoPathName(g.typeIntra));
    for (auto& ch : g.order) {
      XmlNode* c = x->addSub("channel");
      for (int r : ch) c->addSub("gpu")->setAttr("dev", std::to_string(r));
    }
  }
  return root;
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
