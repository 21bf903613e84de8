// Topology detection, path computation, channel-graph search and the analytic tuning model.
// The measured data plane of a single NVSwitch domain needs none of this on its hot path (every
// peer is one hop away at full bandwidth); the machinery exists for detection, for the dumps and
// injection files that users of the reference rely on (NCCL_TOPO_FILE, NCCL_TOPO_DUMP_FILE,
// NCCL_GRAPH_DUMP_FILE), for ring / tree orders on machines that are not fully connected, and to
// predict collective times (ncclGroupSimulateEnd, tuner plugins).
// Reference parity: src/graph/{xml,topo,paths,search,connect,rings,trees,tuning}.cc.
#pragma once
#include <array>
#include <map>
#include <string>
#include <vector>

#include "../comm/comm.h"

namespace b200 {

// ---------------------------------------------------------------- XML (xml.cc)
struct XmlNode {
  std::string name;
  std::vector<std::pair<std::string, std::string>> attrs;
  std::vector<XmlNode*> subs;
  XmlNode* parent = nullptr;
  ~XmlNode() { for (auto* s : subs) delete s; }
  const char* attr(const char* key) const;
  void setAttr(const std::string& key, const std::string& value);
  int attrInt(const char* key, int deflt = 0) const;
  double attrFloat(const char* key, double deflt = 0) const;
  XmlNode* addSub(const std::string& name);
  XmlNode* findSub(const char* name, const char* attrKey = nullptr, const char* attrValue = nullptr);
};
XmlNode* xmlParse(const std::string& text, std::string* err);
XmlNode* xmlLoadFile(const char* path, std::string* err);
std::string xmlDump(const XmlNode* root, int indent = 0);
// Probes this machine: CPUs (NUMA nodes), the PCI hierarchy above every visible GPU, NVLinks
// (through NVML when available, else from the peer-access matrix), NICs from sysfs.
XmlNode* xmlFromSystem();
// Merges the <system> trees of several processes of one host (ranks see different GPUs).
void xmlFuse(XmlNode* dst, const XmlNode* src);

// ---------------------------------------------------------------- system graph (topo.cc)
enum TopoNodeType { TOPO_GPU = 0, TOPO_PCI = 1, TOPO_NVS = 2, TOPO_CPU = 3, TOPO_NIC = 4, TOPO_NET = 5, TOPO_NODE_TYPES = 6 };
enum TopoLinkType { LINK_LOC = 0, LINK_NVL = 1, LINK_C2C = 2, LINK_PCI = 3, LINK_SYS = 4, LINK_NET = 5 };
// Path classes, best to worst (same meaning as the reference's PATH_* values).
enum TopoPathType { PATH_LOC = 0, PATH_NVL = 1, PATH_NVB = 2, PATH_C2C = 3, PATH_PIX = 4, PATH_PXB = 5, PATH_PXN = 6, PATH_PHB = 7, PATH_SYS = 8, PATH_NET = 9, PATH_DIS = 10 };
const char* topoPathName(int type);

constexpr float kNvlinkBwSm100 = 40.1f;   // GB/s per NVLink-5 link as modelled by the reference (src/graph/topo.h:24)
constexpr float kNvlinkBwSm90 = 20.6f;
constexpr float kPciBw = 12.0f;           // PCIe Gen3 x16 reference value; scaled by link speed / width
constexpr float kLocBw = 5000.0f;

struct TopoLink {
  int type;
  float bw;
  int remNode;   // index into TopoSystem::nodes
};
struct TopoPath {
  int type = PATH_DIS;
  float bw = 0;
  int hops = 0;
  std::vector<int> via;   // node indices after the source, ending at the destination
};
struct TopoNode {
  int type;
  int64_t id;             // GPU: bus id; CPU: NUMA id; NIC/NET: device id; PCI: bus id
  int rank = -1, dev = -1, cudaCompCap = 0;   // GPU
  float netBw = 0;        // NET
  std::string name;
  std::vector<TopoLink> links;
  std::vector<TopoPath> paths;   // to every node (filled by topoComputePaths)
};
struct TopoSystem {
  std::vector<TopoNode> nodes;
  std::vector<int> byType[TOPO_NODE_TYPES];
  float maxBw = 0, totalBw = 0;
  int find(int type, int64_t id) const;
};

TopoSystem* topoFromXml(const XmlNode* root, std::string* err);
void topoComputePaths(TopoSystem* sys);
// Path class between two GPUs (by rank); PATH_DIS when unknown.
int topoGpuPathType(const TopoSystem* sys, int rankA, int rankB, float* bw = nullptr);
bool topoCheckP2p(const TopoSystem* sys, int rankA, int rankB, int* pathType = nullptr);
std::string topoDescribe(const TopoSystem* sys);

// ---------------------------------------------------------------- channel graphs (search.cc)
enum TopoPattern { PATTERN_RING = 4, PATTERN_BALANCED_TREE = 1, PATTERN_SPLIT_TREE = 2, PATTERN_TREE = 3, PATTERN_NVLS = 5 };
struct TopoGraph {
  // inputs of the search
  int pattern = PATTERN_RING;
  bool inter = false;     // the job spans nodes: channels enter and leave through NET nodes
  int crossNic = 0;       // a ring may leave through another NIC than it entered (NCCL_CROSS_NIC overrides)
  // results
  int nChannels = 0;
  float bwIntra = 0, bwInter = 0, latencyInter = 0;
  int typeIntra = PATH_DIS, typeInter = PATH_DIS;
  int sameChannels = 1;
  std::vector<std::vector<int>> order;      // per channel: ranks in walk order (local GPUs of this node)
  std::vector<std::array<int, 2>> nets;     // per channel: NET device entered from / left through (-1 inside one node)
  std::vector<int> heads;                   // NVLS: head rank of every channel
};
// Finds the largest set of channels of graph->pattern (see search.cc) at the highest per-channel bandwidth of the
// architecture's speed ladder that the links can carry, within a step budget.
ncclResult_t topoSearch(const TopoSystem* sys, TopoGraph* graph, int minChannels, int maxChannels);
// Graph files: ids 0 ring, 1 tree, 2 NVLS in the order topoInit writes them.
XmlNode* graphToXml(const std::vector<TopoGraph>& graphs);
ncclResult_t graphFromXml(const XmlNode* root, int id, const std::vector<int>& ranks, TopoGraph* graph, std::string* err);

// rings / trees (rings.cc)
// Global ring over all ranks from per-node local orders: prev/next of every rank.
ncclResult_t buildRing(int nRanks, const std::vector<int>& order, std::vector<int>* prev, std::vector<int>* next);
// Binary tree in in-order numbering: parent and up to two children of `rank` among `nRanks`.
void getBtree(int nRanks, int rank, int* up, int* down0, int* down1, int* parentChildType);
// Second tree of the double binary tree: shifted (odd counts) or mirrored (even counts) so that
// every rank is a leaf in one tree and an interior node in the other.
void getDtree(int nRanks, int rank, int* s0, int* d0_0, int* d0_1, int* parentChildType0, int* s1, int* d1_0, int* d1_1, int* parentChildType1);

// ---------------------------------------------------------------- analytic model (tuning_model.cc)
enum ModelAlgo { MODEL_TREE = 0, MODEL_RING = 1, MODEL_COLLNET_DIRECT = 2, MODEL_COLLNET_CHAIN = 3, MODEL_NVLS = 4, MODEL_NVLS_TREE = 5, MODEL_PAT = 6, MODEL_ALGOS = 7 };
enum ModelProto { MODEL_LL = 0, MODEL_LL128 = 1, MODEL_SIMPLE = 2, MODEL_PROTOS = 3 };
struct TuneModel {
  float latencies[FUNC_COUNT][MODEL_ALGOS][MODEL_PROTOS];
  float bandwidths[FUNC_COUNT][MODEL_ALGOS][MODEL_PROTOS];
  int nRanks = 1, nNodes = 1;
};
void topoTuneModel(const TopoSystem* sys, const TopoGraph* ring, const TopoGraph* tree, const TopoGraph* nvls, int nRanks, int nNodes,
                   int compCap, TuneModel* model);
// Predicted time in microseconds; negative when the combination is not available.
float topoAlgoTime(const TuneModel* model, int func, int algo, int proto, size_t bytes);

struct TopoState {
  XmlNode* xml = nullptr;
  TopoSystem* sys = nullptr;
  TopoGraph ring, tree, nvls;
  TuneModel model;
};

ncclResult_t topoInit(ncclComm* comm);
void topoDestroy(ncclComm* comm);

}  // namespace b200
