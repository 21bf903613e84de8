// Built-in network backend "IB": the ncclNet_t table over InfiniBand / RoCE verbs (reliable-connected queue pairs).
//
// libibverbs is opened at run time (NCCL_B200_IBV_LIB, default libibverbs.so.1); without it, or without an active
// port, the backend reports no device and the socket backend serves the job.
//
// One connection = one queue pair on each side, set up over a TCP side channel (address in the listen handle):
// the dialling side sends its queue-pair number, port address and the location of its credit table; the listening
// side answers with the same, and a last byte from the dialling side says that its queue pair can receive.
// Messages of one connection are matched in order: the k-th isend meets the k-th irecv.
//   * small messages (up to the receiver's eager size) travel as SEND with the sequence number as immediate into
//     receive buffers that the receiver posted when the connection was made, so a send completes without a matching
//     irecv; the irecv copies the payload out and re-posts the buffer.
//   * larger messages are receiver-driven: irecv writes {address, key, capacity} into the sender's credit table with
//     an RDMA write; isend returns "not yet" until the entry of its sequence number is there, then moves the payload
//     with one RDMA write with immediate (the byte count) straight into the user buffer.
// Buffers passed without a registration handle are registered on the fly through a reference-counted cache of
// page-aligned regions per device.
// With NCCL_IB_QPS_PER_CONNECTION > 1 a connection has several queue pairs: eager messages and credits stay on the first, a
// message that travels by RDMA write is cut into one part per queue pair (each with its own write with immediate), and the
// receiver completes it when every queue pair has delivered its part.
// Reference parity: src/transport/net_ib/{init,connect,p2p,reg}.cc, src/misc/ibvwrap.cc. Left out: grouped receives (maxRecvs is
// 1), NIC fusion, the GPUDirect flush (device memory is offered only when a peer-memory kernel module or dma-buf registration is
// present), resiliency / port fail-over.
#include <arpa/inet.h>
#include <dlfcn.h>
#include <errno.h>
#include <limits.h>
#include <poll.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <deque>
#include <string>

#include "../core/socket.h"
#include "ibv_abi.h"
#include "net.h"

namespace b200 {

B200_PARAM(IbDisable, "IB_DISABLE", 0, "1: do not use the InfiniBand / RoCE backend even when verbs devices are present")
B200_PARAM(IbGidIndex, "IB_GID_INDEX", -1, "GID table entry used for RoCE and routed InfiniBand (-1: first RoCE v2 entry of NCCL_IB_ADDR_FAMILY, else the first entry in use)")
B200_PARAM(IbRoceVersion, "IB_ROCE_VERSION_NUM", 2, "RoCE version looked for when the GID index is chosen automatically")
B200_PARAM(IbTimeout, "IB_TIMEOUT", 20, "Queue-pair acknowledgement time-out exponent (4.096 us * 2^n)")
B200_PARAM(IbRetryCnt, "IB_RETRY_CNT", 7, "Queue-pair transport retry count")
B200_PARAM(IbSl, "IB_SL", 0, "InfiniBand service level")
B200_PARAM(IbTc, "IB_TC", 0, "Traffic class of the global route (RoCE)")
B200_PARAM(IbPkey, "IB_PKEY", 0, "Partition key index")
B200_PARAM(IbUseInline, "IB_USE_INLINE", 1, "Send messages and credit entries that fit as inline data of the work request")
B200_PARAM(IbRelaxedOrdering, "IB_PCI_RELAXED_ORDERING", 0, "1: memory regions are registered with relaxed PCIe ordering (falls back to strict ordering where the adapter refuses it)")
B200_PARAM(IbQps, "IB_QPS_PER_CONNECTION", 1, "Queue pairs per connection (1 to 8; both ends use the smaller of their settings): messages that travel by RDMA write are split evenly over them")
B200_PARAM(IbEagerBytes, "B200_IB_EAGER_BYTES", 8192, "Largest message that travels eagerly (SEND into pre-posted buffers) instead of by receiver-driven RDMA write")

namespace {

constexpr int kSlots = 32;                 // messages in flight per connection and direction
constexpr int kMaxReqs = 2 * kSlots;
constexpr int kMaxIbDevs = 32;
constexpr int kMaxQps = 8;                // queue pairs of one connection
constexpr uint64_t kIbMagic = 0x4942564242323030ull;   // "IBVBB200"
constexpr uint64_t kCreditWrId = ~0ull;    // work-request id of credit-table writes (no request behind them)
constexpr size_t kPage = 4096;

IbvApi ibv;
ncclDebugLogger_t gLog = nullptr;
ncclProfilerCallback_t gProf = nullptr;

struct MrEntry { uintptr_t start; size_t bytes; ibv_mr* mr; int refs; };

struct IbDev {
  std::string name;
  ibv_context* ctx = nullptr;
  int port = 1;
  ibv_port_attr attr;
  int gidIndex = 0;
  ibv_gid gid;
  uint64_t guid = 0;
  int maxQp = 0;
  int speedMbps = 0;
  char pciPath[PATH_MAX] = "";
  ibv_pd* pd = nullptr;
  std::mutex lock;
  std::vector<MrEntry> mrs;
  bool dmaBuf = false;
};
IbDev gDevs[kMaxIbDevs];
int gNDevs = -1;
std::mutex gInitLock;
bool gPeerMem = false;

bool loadVerbs() {
  const char* path = getEnv("NCCL_B200_IBV_LIB");
  if (!path || !*path) path = getEnv("NCCL_IBVERBS_LIB");   // the reference's name of the same setting
  void* h = dlopen(path && *path ? path : "libibverbs.so.1", RTLD_NOW | RTLD_LOCAL);
  if (!h) return false;
  bool ok = true;
  auto need = [&](void** fn, const char* name) { *fn = dlsym(h, name); if (!*fn) ok = false; };
  need((void**)&ibv.get_device_list, "ibv_get_device_list");
  need((void**)&ibv.free_device_list, "ibv_free_device_list");
  need((void**)&ibv.get_device_name, "ibv_get_device_name");
  need((void**)&ibv.open_device, "ibv_open_device");
  need((void**)&ibv.close_device, "ibv_close_device");
  need((void**)&ibv.query_device, "ibv_query_device");
  need((void**)&ibv.query_port, "ibv_query_port");
  need((void**)&ibv.query_gid, "ibv_query_gid");
  need((void**)&ibv.alloc_pd, "ibv_alloc_pd");
  need((void**)&ibv.dealloc_pd, "ibv_dealloc_pd");
  need((void**)&ibv.reg_mr, "ibv_reg_mr");
  need((void**)&ibv.dereg_mr, "ibv_dereg_mr");
  need((void**)&ibv.create_cq, "ibv_create_cq");
  need((void**)&ibv.destroy_cq, "ibv_destroy_cq");
  need((void**)&ibv.create_qp, "ibv_create_qp");
  need((void**)&ibv.modify_qp, "ibv_modify_qp");
  need((void**)&ibv.destroy_qp, "ibv_destroy_qp");
  ibv.reg_dmabuf_mr = (decltype(ibv.reg_dmabuf_mr))dlsym(h, "ibv_reg_dmabuf_mr");
  ibv.fork_init = (int (*)())dlsym(h, "ibv_fork_init");
  return ok;
}

int laneMbps(const ibv_port_attr& a) {
  if (a.active_speed_ex >= 256) return 200000;   // XDR
  switch (a.active_speed) {
    case 1: return 2500; case 2: return 5000; case 4: case 8: return 10000; case 16: return 14000; case 32: return 25000; case 64: return 50000;
    case 128: return 100000; default: return 2500;
  }
}
int widthOf(int code) { switch (code) { case 1: return 1; case 2: return 4; case 4: return 8; case 8: return 12; case 16: return 2; default: return 1; } }

// NCCL_IB_HCA: "mlx5_0,mlx5_1:1" picks by name prefix (and port), "=name" wants the exact name, a leading "^" excludes.
bool hcaWanted(const char* name, int port) {
  const char* spec = getEnv("NCCL_IB_HCA");
  if (!spec || !*spec) return true;
  bool exclude = false, exact = false;
  if (*spec == '^') { exclude = true; ++spec; }
  if (*spec == '=') { exact = true; ++spec; }
  bool match = false;
  std::string s(spec);
  size_t pos = 0;
  while (pos <= s.size()) {
    size_t end = s.find(',', pos);
    if (end == std::string::npos) end = s.size();
    std::string item = s.substr(pos, end - pos);
    pos = end + 1;
    if (item.empty()) continue;
    int wantPort = -1;
    size_t colon = item.find(':');
    if (colon != std::string::npos) { wantPort = atoi(item.c_str() + colon + 1); item.resize(colon); }
    bool nameOk = exact ? item == name : strncmp(name, item.c_str(), item.size()) == 0;
    if (nameOk && (wantPort < 0 || wantPort == port)) match = true;
  }
  return exclude ? !match : match;
}

bool gidInUse(const ibv_gid& g) { static const ibv_gid zero = {}; return memcmp(&g, &zero, sizeof(g)) != 0 && g.global.interface_id != 0; }
bool gidIsV4Mapped(const ibv_gid& g) { return g.global.subnet_prefix == 0 && g.raw[8] == 0 && g.raw[9] == 0 && g.raw[10] == 0xff && g.raw[11] == 0xff; }

// The RoCE version of a GID entry as the kernel reports it ("IB/RoCE v1" or "RoCE v2"); 0 when the file is not there.
int gidRoceVersion(const char* dev, int port, int index) {
  char path[PATH_MAX], line[64] = "";
  snprintf(path, sizeof(path), "/sys/class/infiniband/%s/ports/%d/gid_attrs/types/%d", dev, port, index);
  FILE* f = fopen(path, "r");
  if (!f) return 0;
  if (!fgets(line, sizeof(line), f)) line[0] = 0;
  fclose(f);
  return strstr(line, "v2") ? 2 : 1;
}

int chooseGid(IbDev* d) {
  if (paramIbGidIndex() >= 0) return (int)paramIbGidIndex();
  if (d->attr.link_layer != IBV_LINK_LAYER_ETHERNET) return 0;
  const char* fam = getEnv("NCCL_IB_ADDR_FAMILY");
  const bool wantV6 = fam && strcasecmp(fam, "AF_INET6") == 0;
  int firstUsed = -1, best = -1;
  for (int i = 0; i < d->attr.gid_tbl_len && i < 256; ++i) {
    ibv_gid g;
    if (ibv.query_gid(d->ctx, d->port, i, &g) != 0 || !gidInUse(g)) continue;
    if (firstUsed < 0) firstUsed = i;
    int ver = gidRoceVersion(d->name.c_str(), d->port, i);
    if (ver == (int)paramIbRoceVersion() && gidIsV4Mapped(g) == !wantV6) { best = i; break; }
  }
  return best >= 0 ? best : (firstUsed >= 0 ? firstUsed : 0);
}

void loadDevices() {
  std::lock_guard<std::mutex> g(gInitLock);
  if (gNDevs >= 0) return;
  gNDevs = 0;
  if (paramIbDisable() || !loadVerbs()) return;
  if (ibv.fork_init) ibv.fork_init();
  gPeerMem = access("/sys/kernel/mm/memory_peers/nv_mem/version", F_OK) == 0 || access("/sys/module/nvidia_peermem/version", F_OK) == 0;
  int n = 0;
  ibv_device** list = ibv.get_device_list(&n);
  if (!list) return;
  for (int i = 0; i < n && gNDevs < kMaxIbDevs; ++i) {
    ibv_context* ctx = ibv.open_device(list[i]);
    if (!ctx) continue;
    ibv_device_attr da;
    memset(&da, 0, sizeof(da));
    if (ibv.query_device(ctx, &da) != 0) { ibv.close_device(ctx); continue; }
    int used = 0;
    for (int port = 1; port <= da.phys_port_cnt && gNDevs < kMaxIbDevs; ++port) {
      ibv_port_attr pa;
      memset(&pa, 0, sizeof(pa));
      if (ibv.query_port(ctx, (uint8_t)port, &pa) != 0) continue;
      if (pa.state != IBV_PORT_ACTIVE) continue;
      if (pa.link_layer != IBV_LINK_LAYER_INFINIBAND && pa.link_layer != IBV_LINK_LAYER_ETHERNET) continue;
      const char* name = ibv.get_device_name(list[i]);
      if (!hcaWanted(name, port)) continue;
      IbDev* d = &gDevs[gNDevs];
      d->name = name;
      d->ctx = ctx;
      d->port = port;
      d->attr = pa;
      d->guid = da.node_guid;
      d->maxQp = da.max_qp;
      d->speedMbps = laneMbps(pa) * widthOf(pa.active_width);
      d->gidIndex = chooseGid(d);
      memset(&d->gid, 0, sizeof(d->gid));
      ibv.query_gid(ctx, (uint8_t)port, d->gidIndex, &d->gid);
      char link[PATH_MAX];
      snprintf(link, sizeof(link), "/sys/class/infiniband/%s/device", name);
      if (!realpath(link, d->pciPath)) d->pciPath[0] = 0;
      d->dmaBuf = ibv.reg_dmabuf_mr != nullptr;
      gNDevs++;
      used++;
      INFO(SUB_NET | SUB_INIT, "NET/IB : device %d %s:%d %s, %d Mbps, lid %u, gid index %d", gNDevs - 1, name, port,
           pa.link_layer == IBV_LINK_LAYER_ETHERNET ? "RoCE" : "InfiniBand", d->speedMbps, pa.lid, d->gidIndex);
    }
    if (!used) ibv.close_device(ctx);
  }
  ibv.free_device_list(list);
}

ncclResult_t devPd(IbDev* d) {
  std::lock_guard<std::mutex> g(d->lock);
  if (!d->pd) d->pd = ibv.alloc_pd(d->ctx);
  if (!d->pd) { WARN("NET/IB : cannot allocate a protection domain on %s", d->name.c_str()); return ncclSystemError; }
  return ncclSuccess;
}

// Region that covers [p, p+bytes) on this device: an existing registration is shared, else the page-aligned range is registered.
ncclResult_t mrGet(IbDev* d, const void* p, size_t bytes, ibv_mr** out) {
  uintptr_t start = (uintptr_t)p & ~(uintptr_t)(kPage - 1);
  size_t len = (((uintptr_t)p + bytes + kPage - 1) & ~(uintptr_t)(kPage - 1)) - start;
  std::lock_guard<std::mutex> g(d->lock);
  for (auto& e : d->mrs)
    if (e.start <= start && start + len <= e.start + e.bytes) { e.refs++; *out = e.mr; return ncclSuccess; }
  const int access = IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ;
  ibv_mr* mr = paramIbRelaxedOrdering() ? ibv.reg_mr(d->pd, (void*)start, len, access | IBV_ACCESS_RELAXED_ORDERING) : nullptr;
  if (!mr) mr = ibv.reg_mr(d->pd, (void*)start, len, access);
  if (!mr) { WARN("NET/IB : registration of %zu bytes at %p failed on %s (locked-memory limit?)", len, (void*)start, d->name.c_str()); return ncclSystemError; }
  d->mrs.push_back(MrEntry{start, len, mr, 1});
  *out = mr;
  return ncclSuccess;
}
void mrPut(IbDev* d, ibv_mr* mr) {
  std::lock_guard<std::mutex> g(d->lock);
  for (size_t i = 0; i < d->mrs.size(); ++i) {
    if (d->mrs[i].mr != mr) continue;
    if (--d->mrs[i].refs == 0) { ibv.dereg_mr(mr); d->mrs.erase(d->mrs.begin() + i); }
    return;
  }
  ibv.dereg_mr(mr);   // a dma-buf registration: never shared
}

struct Handle {              // what listen() hands out; the dialling side keeps its progress in `stage`
  SockAddr addr;
  uint64_t magic;
  void* stage;
};
static_assert(sizeof(Handle) <= NCCL_NET_HANDLE_MAXSIZE, "handle too large");

struct PeerInfo {            // exchanged over the side channel, both directions
  uint32_t nQps;             // dialling side: what it offers; listening side: what both will use
  uint32_t qpn[kMaxQps];
  uint16_t lid;
  uint8_t linkLayer, mtu;
  ibv_gid gid;
  uint64_t creditAddr;       // dialling side: where the listener writes credits
  uint32_t creditKey;
  uint32_t eagerBytes;       // listening side: size of its eager buffers
};

struct Credit {              // one entry of the sender's credit table
  uint64_t addr;
  uint32_t key, capacity, tag;
  volatile uint32_t seq;     // sequence number + 1 of the receive it belongs to: written last (same write, ascending addresses)
};

struct Comm;
struct Request {
  bool used = false, done = false, isSend = false;
  Comm* comm = nullptr;
  size_t size = 0;           // send: bytes; receive: capacity, then bytes received
  char* data = nullptr;
  ibv_mr* tmpMr = nullptr;   // registered for this request only
  uint32_t seq = 0;
  int pending = 0;           // send: completions still to come (one per queue pair that carries a part)
  void* prof = nullptr;      // event of this request at the profiler
  ncclProfilerNetIbDescr_v1_t profDescr;
};

struct Arrival { bool eager; uint32_t bytes; uint32_t seq; int buffer; };

struct Comm {
  IbDev* dev = nullptr;
  bool isSend = false;
  Socket sock;
  ibv_cq* cq = nullptr;
  ibv_qp* qps[kMaxQps] = {};   // qps[0] carries eager messages, credits and the first part of every RDMA-write message
  int nQps = 1;
  int maxInline = 0;
  size_t eagerBytes = 0;
  Request reqs[kMaxReqs];
  int inflight = 0;
  uint32_t seq = 0;          // next message of this connection
  bool failed = false;
  // sending side
  Credit* credits = nullptr;   // written by the receiver
  ibv_mr* creditMr = nullptr;
  char* stage = nullptr;       // eager payloads that came without a registration
  ibv_mr* stageMr = nullptr;
  // receiving side
  char* bounce = nullptr;      // eager landing buffers, one per posted receive
  ibv_mr* bounceMr = nullptr;
  Credit* outCredits = nullptr;   // source of the credit writes
  ibv_mr* outCreditMr = nullptr;
  uint64_t remoteCreditAddr = 0;
  uint32_t remoteCreditKey = 0;
  std::deque<Request*> waiting;   // receives in order
  std::deque<Arrival> arrived[kMaxQps];   // completed receives of each queue pair, in order
  int creditWrites = 0;           // signalled credit writes not yet polled
  uint32_t idlePolls = 0;         // polls since something last completed (liveness check of the side channel)
};

struct ListenComm {
  IbDev* dev = nullptr;
  int devIndex = 0;
  Socket sock;
  Comm* pending = nullptr;   // accepted over TCP, waiting for the dialling side's "ready"
};

struct ConnectStage { Comm* comm; PeerInfo theirs; int got; };

void* pageAlloc(size_t bytes) {
  void* p = nullptr;
  if (posix_memalign(&p, kPage, (bytes + kPage - 1) & ~(kPage - 1)) != 0) return nullptr;
  memset(p, 0, bytes);
  return p;
}

void commFree(Comm* c) {
  if (!c) return;
  for (ibv_qp* q : c->qps) if (q) ibv.destroy_qp(q);
  if (c->cq) ibv.destroy_cq(c->cq);
  for (auto& r : c->reqs) {
    if (r.used && r.prof && gProf) gProf(&r.prof, ncclProfilerNetEventStop, nullptr, 0, nullptr);
    if (r.used && r.tmpMr) mrPut(c->dev, r.tmpMr);
  }
  for (ibv_mr* m : {c->creditMr, c->stageMr, c->bounceMr, c->outCreditMr}) if (m) ibv.dereg_mr(m);
  free(c->credits); free(c->stage); free(c->bounce); free(c->outCredits);
  sockClose(&c->sock);
  delete c;
}

ncclResult_t commCreate(IbDev* d, bool isSend, size_t eagerBytes, Comm** out) {
  NCCLCHECK(devPd(d));
  Comm* c = new Comm;
  c->dev = d;
  c->isSend = isSend;
  c->eagerBytes = eagerBytes;
  c->cq = ibv.create_cq(d->ctx, 4 * kSlots * kMaxQps, nullptr, nullptr, 0);
  if (!c->cq) { WARN("NET/IB : cannot create a completion queue on %s", d->name.c_str()); commFree(c); return ncclSystemError; }
  c->nQps = (int)std::min<int64_t>(std::max<int64_t>(paramIbQps(), 1), kMaxQps);
  c->maxInline = 0;
  for (int i = 0; i < c->nQps; ++i) {
    ibv_qp_init_attr ia;
    memset(&ia, 0, sizeof(ia));
    ia.send_cq = ia.recv_cq = c->cq;
    ia.qp_type = IBV_QPT_RC;
    ia.cap.max_send_wr = 2 * kSlots;
    ia.cap.max_recv_wr = isSend ? 1 : kSlots;
    ia.cap.max_send_sge = ia.cap.max_recv_sge = 1;
    ia.cap.max_inline_data = paramIbUseInline() && i == 0 ? (uint32_t)sizeof(Credit) : 0;
    c->qps[i] = ibv.create_qp(d->pd, &ia);
    if (!c->qps[i] && ia.cap.max_inline_data) { ia.cap.max_inline_data = 0; c->qps[i] = ibv.create_qp(d->pd, &ia); }
    if (!c->qps[i]) { WARN("NET/IB : cannot create a queue pair on %s", d->name.c_str()); commFree(c); return ncclSystemError; }
    if (i == 0) c->maxInline = paramIbUseInline() ? (int)ia.cap.max_inline_data : 0;
    ibv_qp_attr a;
    memset(&a, 0, sizeof(a));
    a.qp_state = IBV_QPS_INIT;
    a.pkey_index = (uint16_t)paramIbPkey();
    a.port_num = (uint8_t)d->port;
    a.qp_access_flags = IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE;
    if (ibv.modify_qp(c->qps[i], &a, IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS) != 0) {
      WARN("NET/IB : queue pair to INIT failed on %s", d->name.c_str());
      commFree(c);
      return ncclSystemError;
    }
  }
  const int plain = IBV_ACCESS_LOCAL_WRITE, remote = IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE;
  bool ok = true;
  if (isSend) {
    c->credits = (Credit*)pageAlloc(kSlots * sizeof(Credit));
    c->stage = (char*)pageAlloc(kSlots * eagerBytes);
    ok = c->credits && c->stage && (c->creditMr = ibv.reg_mr(d->pd, c->credits, kSlots * sizeof(Credit), remote)) &&
         (c->stageMr = ibv.reg_mr(d->pd, c->stage, kSlots * eagerBytes, plain));
  } else {
    c->bounce = (char*)pageAlloc(kSlots * eagerBytes);
    c->outCredits = (Credit*)pageAlloc(kSlots * sizeof(Credit));
    ok = c->bounce && c->outCredits && (c->bounceMr = ibv.reg_mr(d->pd, c->bounce, kSlots * eagerBytes, plain)) &&
         (c->outCreditMr = ibv.reg_mr(d->pd, c->outCredits, kSlots * sizeof(Credit), plain));
  }
  if (!ok) { WARN("NET/IB : cannot register the connection's own buffers on %s", d->name.c_str()); commFree(c); return ncclSystemError; }
  *out = c;
  return ncclSuccess;
}

void myInfo(Comm* c, PeerInfo* pi) {
  memset(pi, 0, sizeof(*pi));
  pi->nQps = (uint32_t)c->nQps;
  for (int i = 0; i < c->nQps; ++i) pi->qpn[i] = c->qps[i]->qp_num;
  pi->lid = c->dev->attr.lid;
  pi->linkLayer = c->dev->attr.link_layer;
  pi->mtu = (uint8_t)c->dev->attr.active_mtu;
  pi->gid = c->dev->gid;
  if (c->isSend) { pi->creditAddr = (uint64_t)(uintptr_t)c->credits; pi->creditKey = c->creditMr->rkey; }
  pi->eagerBytes = (uint32_t)c->eagerBytes;
}

ncclResult_t commWire(Comm* c, const PeerInfo& peer) {
  IbDev* d = c->dev;
  if (peer.linkLayer != d->attr.link_layer) { WARN("NET/IB : %s is %s and the peer's port is not", d->name.c_str(), d->attr.link_layer == IBV_LINK_LAYER_ETHERNET ? "RoCE" : "InfiniBand"); return ncclSystemError; }
  // both ends use the smaller number of queue pairs; the ones beyond it stay unconnected until the connection is closed
  c->nQps = (int)std::min<uint32_t>((uint32_t)c->nQps, std::max<uint32_t>(peer.nQps, 1));
  for (int i = 0; i < c->nQps; ++i) {
    ibv_qp_attr a;
    memset(&a, 0, sizeof(a));
    a.qp_state = IBV_QPS_RTR;
    a.path_mtu = std::min<int>(d->attr.active_mtu, peer.mtu);
    a.dest_qp_num = peer.qpn[i];
    a.rq_psn = 0;
    a.max_dest_rd_atomic = 1;
    a.min_rnr_timer = 12;
    a.ah_attr.port_num = (uint8_t)d->port;
    a.ah_attr.sl = (uint8_t)paramIbSl();
    a.ah_attr.dlid = peer.lid;
    if (d->attr.link_layer == IBV_LINK_LAYER_ETHERNET || peer.gid.global.subnet_prefix != d->gid.global.subnet_prefix) {
      a.ah_attr.is_global = 1;
      a.ah_attr.grh.dgid = peer.gid;
      a.ah_attr.grh.sgid_index = (uint8_t)d->gidIndex;
      a.ah_attr.grh.hop_limit = 255;
      a.ah_attr.grh.traffic_class = (uint8_t)paramIbTc();
    }
    if (ibv.modify_qp(c->qps[i], &a, IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN | IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER) != 0) {
      WARN("NET/IB : queue pair to RTR failed on %s", d->name.c_str());
      return ncclSystemError;
    }
    memset(&a, 0, sizeof(a));
    a.qp_state = IBV_QPS_RTS;
    a.timeout = (uint8_t)paramIbTimeout();
    a.retry_cnt = (uint8_t)paramIbRetryCnt();
    a.rnr_retry = 7;
    a.sq_psn = 0;
    a.max_rd_atomic = 1;
    if (ibv.modify_qp(c->qps[i], &a, IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN | IBV_QP_MAX_QP_RD_ATOMIC) != 0) {
      WARN("NET/IB : queue pair to RTS failed on %s", d->name.c_str());
      return ncclSystemError;
    }
  }
  return ncclSuccess;
}

ncclResult_t postBounce(Comm* c, int i) {
  ibv_sge sge = {(uint64_t)(uintptr_t)(c->bounce + (size_t)i * c->eagerBytes), (uint32_t)c->eagerBytes, c->bounceMr->lkey};
  ibv_recv_wr wr, *bad = nullptr;
  memset(&wr, 0, sizeof(wr));
  wr.wr_id = (uint64_t)i;
  wr.sg_list = &sge;
  wr.num_sge = 1;
  if (ibv_post_recv(c->qps[0], &wr, &bad) != 0) { WARN("NET/IB : posting a receive failed"); return ncclSystemError; }
  return ncclSuccess;
}

// Queue pairs beyond the first only carry RDMA writes with immediate: their receives have no buffer.
ncclResult_t postEmpty(Comm* c, int qp, int i) {
  ibv_recv_wr wr, *bad = nullptr;
  memset(&wr, 0, sizeof(wr));
  wr.wr_id = (uint64_t)i;
  if (ibv_post_recv(c->qps[qp], &wr, &bad) != 0) { WARN("NET/IB : posting a receive failed"); return ncclSystemError; }
  return ncclSuccess;
}

Request* reqGet(Comm* c) {
  for (auto& r : c->reqs)
    if (!r.used) { r = Request(); r.used = true; r.comm = c; return &r; }
  return nullptr;
}

ncclResult_t ibInit(void** ctx, uint64_t, ncclNetCommConfig_t*, ncclDebugLogger_t log, ncclProfilerCallback_t prof) {
  gLog = log;
  if (prof) gProf = prof;
  loadDevices();
  if (ctx) *ctx = nullptr;
  return ncclSuccess;
}
ncclResult_t ibDevices(int* n) { loadDevices(); *n = gNDevs; return ncclSuccess; }

ncclResult_t ibGetProperties(int dev, ncclNetProperties_t* p) {
  if (dev < 0 || dev >= gNDevs) return ncclInvalidArgument;
  IbDev* d = &gDevs[dev];
  memset(p, 0, sizeof(*p));
  p->name = (char*)d->name.c_str();
  p->pciPath = d->pciPath[0] ? d->pciPath : nullptr;
  p->guid = d->guid;
  p->ptrSupport = NCCL_PTR_HOST | (gPeerMem ? NCCL_PTR_CUDA : 0) | (d->dmaBuf ? NCCL_PTR_DMABUF : 0);
  p->regIsGlobal = 1;
  p->speed = d->speedMbps;
  p->port = d->port;
  p->latency = 0;
  p->maxComms = d->maxQp;
  p->maxRecvs = 1;
  p->netDeviceType = NCCL_NET_DEVICE_HOST;
  p->vProps.ndevs = 1;
  p->vProps.devs[0] = dev;
  p->maxP2pBytes = 1u << 30;
  p->maxCollBytes = 1u << 30;
  p->maxMultiRequestSize = 1;
  p->railId = p->planeId = -1;
  return ncclSuccess;
}

ncclResult_t ibListen(void*, int dev, void* handle, void** listenComm) {
  if (dev < 0 || dev >= gNDevs) return ncclInvalidArgument;
  Handle* h = (Handle*)handle;
  memset(h, 0, NCCL_NET_HANDLE_MAXSIZE);
  ListenComm* lc = new ListenComm;
  lc->dev = &gDevs[dev];
  lc->devIndex = dev;
  SockAddr addr;
  char ifName[64];
  ncclResult_t r = bootstrapInterface(&addr, ifName);
  if (r == ncclSuccess) r = sockInit(&lc->sock, &addr, kIbMagic, SOCK_NETIB);
  if (r == ncclSuccess) r = sockListen(&lc->sock);
  if (r != ncclSuccess) { delete lc; return r; }
  h->addr = lc->sock.addr;
  h->magic = kIbMagic;
  *listenComm = lc;
  return ncclSuccess;
}

ncclResult_t ibConnect(void*, int dev, void* handle, void** sendComm, ncclNetDeviceHandle_t** devComm) {
  if (dev < 0 || dev >= gNDevs) return ncclInvalidArgument;
  Handle* h = (Handle*)handle;
  *sendComm = nullptr;
  if (devComm) *devComm = nullptr;
  ConnectStage* st = (ConnectStage*)h->stage;
  if (!st) {
    Comm* c = nullptr;
    NCCLCHECK(commCreate(&gDevs[dev], true, (size_t)std::max<int64_t>(paramIbEagerBytes(), 64), &c));
    ncclResult_t r = sockInit(&c->sock, &h->addr, h->magic, SOCK_NETIB);
    if (r == ncclSuccess) r = sockConnect(&c->sock);
    PeerInfo mine;
    myInfo(c, &mine);
    if (r == ncclSuccess) r = sockSend(&c->sock, &mine, sizeof(mine));
    if (r != ncclSuccess) { commFree(c); return r; }
    st = new ConnectStage{c, {}, 0};
    h->stage = st;
  }
  ncclResult_t r = sockProgress(SOCK_OP_RECV, &st->comm->sock, &st->theirs, sizeof(PeerInfo), &st->got);
  if (r != ncclSuccess) { commFree(st->comm); delete st; h->stage = nullptr; return r; }
  if (st->got < (int)sizeof(PeerInfo)) return ncclSuccess;   // the listener has not answered yet: call again
  Comm* c = st->comm;
  const PeerInfo theirs = st->theirs;
  delete st;
  h->stage = nullptr;
  c->eagerBytes = std::min<size_t>(c->eagerBytes, theirs.eagerBytes);
  r = commWire(c, theirs);
  char ready = 1;
  if (r == ncclSuccess) r = sockSend(&c->sock, &ready, 1);
  if (r != ncclSuccess) { commFree(c); return r; }
  *sendComm = c;
  return ncclSuccess;
}

ncclResult_t ibAccept(void* listenComm, void** recvComm, ncclNetDeviceHandle_t** devComm) {
  ListenComm* lc = (ListenComm*)listenComm;
  *recvComm = nullptr;
  if (devComm) *devComm = nullptr;
  if (!lc->pending) {
    struct pollfd pfd = {lc->sock.fd, POLLIN, 0};
    if (poll(&pfd, 1, 0) <= 0) return ncclSuccess;   // nobody is dialling right now: call again
    Comm* c = nullptr;
    NCCLCHECK(commCreate(lc->dev, false, (size_t)std::max<int64_t>(paramIbEagerBytes(), 64), &c));
    PeerInfo theirs, mine;
    ncclResult_t r = sockAccept(&c->sock, &lc->sock);
    if (r == ncclSuccess) r = sockRecv(&c->sock, &theirs, sizeof(theirs));
    // both ends use the smaller of their eager sizes (the receiver posts no credit for a buffer that the sender would fill eagerly)
    if (r == ncclSuccess && theirs.eagerBytes >= 64) c->eagerBytes = std::min<size_t>(c->eagerBytes, theirs.eagerBytes);
    if (r == ncclSuccess) r = commWire(c, theirs);
    for (int i = 0; i < kSlots && r == ncclSuccess; ++i) r = postBounce(c, i);
    for (int q = 1; q < c->nQps; ++q)
      for (int i = 0; i < kSlots && r == ncclSuccess; ++i) r = postEmpty(c, q, i);
    c->remoteCreditAddr = theirs.creditAddr;
    c->remoteCreditKey = theirs.creditKey;
    myInfo(c, &mine);
    if (r == ncclSuccess) r = sockSend(&c->sock, &mine, sizeof(mine));
    if (r != ncclSuccess) { commFree(c); return r; }
    lc->pending = c;
  }
  char ready = 0;
  int got = 0;
  ncclResult_t r = sockProgress(SOCK_OP_RECV, &lc->pending->sock, &ready, 1, &got);
  if (r != ncclSuccess) { commFree(lc->pending); lc->pending = nullptr; return r; }
  if (got < 1) return ncclSuccess;
  *recvComm = lc->pending;
  lc->pending = nullptr;
  return ncclSuccess;
}

struct MrHandle { ibv_mr* mr; IbDev* dev; };

ncclResult_t ibRegMr(void* comm, void* data, size_t size, int type, void** mhandle) {
  Comm* c = (Comm*)comm;
  if (type == NCCL_PTR_CUDA && !gPeerMem) { WARN("NET/IB : device memory cannot be registered here (no peer-memory kernel module)"); return ncclInvalidUsage; }
  ibv_mr* mr = nullptr;
  NCCLCHECK(mrGet(c->dev, data, size, &mr));
  *mhandle = new MrHandle{mr, c->dev};
  return ncclSuccess;
}
ncclResult_t ibRegMrDmaBuf(void* comm, void* data, size_t size, int type, uint64_t offset, int fd, void** mhandle) {
  Comm* c = (Comm*)comm;
  if (!ibv.reg_dmabuf_mr) return ibRegMr(comm, data, size, type, mhandle);
  ibv_mr* mr = ibv.reg_dmabuf_mr(c->dev->pd, offset, size, (uint64_t)(uintptr_t)data, fd, IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ);
  if (!mr) { WARN("NET/IB : dma-buf registration of %zu bytes failed on %s", size, c->dev->name.c_str()); return ncclSystemError; }
  *mhandle = new MrHandle{mr, c->dev};
  return ncclSuccess;
}
ncclResult_t ibDeregMr(void*, void* mhandle) {
  MrHandle* h = (MrHandle*)mhandle;
  if (!h) return ncclSuccess;
  mrPut(h->dev, h->mr);
  delete h;
  return ncclSuccess;
}

// One profiler event per request: the work request on the first queue pair stands for the message.
void profRequest(Request* r, void* phandle, int opcode, size_t length) {
  if (!gProf || !phandle) return;
  r->profDescr.type = ncclProfileQp;
  r->profDescr.qp.device = (int)(r->comm->dev - gDevs);
  r->profDescr.qp.wr_id = (uint64_t)(r - r->comm->reqs);
  r->profDescr.qp.opcode = opcode;
  r->profDescr.qp.qpNum = (int)r->comm->qps[0]->qp_num;
  r->profDescr.qp.length = length;
  gProf(&r->prof, ncclProfilerNetEventStart, phandle, NCCL_PROFILER_NET_TYPE_IB | NCCL_PROFILER_NET_IB_VER, &r->profDescr);
}

// A queue pair says nothing while nothing moves: when the other end's process dies between two messages, a sender waits for a
// credit and a receiver for data that will never come. The TCP side channel of the connection stays open for its whole life,
// so its end-of-file is the sign that the peer is gone; it is looked at once in a while when a request makes no progress.
bool peerGone(Comm* c) {
  if ((++c->idlePolls & 0x3fff) != 0 || c->sock.fd < 0) return false;
  char b;
  ssize_t n = recv(c->sock.fd, &b, 1, MSG_PEEK | MSG_DONTWAIT);
  return n == 0 || (n < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR);
}

ncclResult_t ibIsend(void* sendComm, void* data, size_t size, int tag, void* mhandle, void* phandle, void** request) {
  Comm* c = (Comm*)sendComm;
  *request = nullptr;
  if (c->failed) return ncclRemoteError;
  if (size > (1u << 30)) { WARN("NET/IB : a message of %zu bytes exceeds the 1 GiB limit of one send", size); return ncclInvalidArgument; }
  if (c->inflight >= kSlots) return ncclSuccess;
  const int slot = (int)(c->seq % kSlots);
  ibv_sge sge = {(uint64_t)(uintptr_t)data, (uint32_t)size, 0};
  ibv_send_wr wr, *bad = nullptr;
  memset(&wr, 0, sizeof(wr));
  wr.sg_list = &sge;
  wr.num_sge = size ? 1 : 0;
  wr.send_flags = IBV_SEND_SIGNALED;
  ibv_mr* tmp = nullptr;
  if (size <= c->eagerBytes) {
    wr.opcode = IBV_WR_SEND_WITH_IMM;
    wr.imm_data = htonl(c->seq);
    if ((int)size <= c->maxInline) wr.send_flags |= IBV_SEND_INLINE;
    else if (mhandle) sge.lkey = ((MrHandle*)mhandle)->mr->lkey;
    else {
      char* st = c->stage + (size_t)slot * c->eagerBytes;
      memcpy(st, data, size);
      sge.addr = (uint64_t)(uintptr_t)st;
      sge.lkey = c->stageMr->lkey;
    }
  } else {
    Credit* cr = &c->credits[slot];
    if (cr->seq != c->seq + 1) {   // the matching receive has not been posted yet
      if (peerGone(c)) { WARN("NET/IB : the process at the other end of a connection on %s is gone", c->dev->name.c_str()); c->failed = true; return ncclRemoteError; }
      return ncclSuccess;
    }
    c->idlePolls = 0;
    __sync_synchronize();
    if (size > cr->capacity) { WARN("NET/IB : a send of %zu bytes meets a receive of %u bytes", size, cr->capacity); return ncclInvalidUsage; }
    if (mhandle) sge.lkey = ((MrHandle*)mhandle)->mr->lkey;
    else { NCCLCHECK(mrGet(c->dev, data, size, &tmp)); sge.lkey = tmp->lkey; }
    wr.opcode = IBV_WR_RDMA_WRITE_WITH_IMM;
    wr.imm_data = htonl((uint32_t)size);
    wr.wr.rdma.remote_addr = cr->addr;
    wr.wr.rdma.rkey = cr->key;
  }
  Request* r = reqGet(c);
  if (!r) { if (tmp) mrPut(c->dev, tmp); return ncclSuccess; }
  r->isSend = true;
  r->size = size;
  r->tmpMr = tmp;
  r->seq = c->seq;
  wr.wr_id = (uint64_t)(r - c->reqs);
  (void)tag;
  const int parts = wr.opcode == IBV_WR_RDMA_WRITE_WITH_IMM ? c->nQps : 1;
  r->pending = parts;
  // a message that travels by RDMA write is cut into one part per queue pair (the later ones may be empty: every queue pair
  // sees exactly one write with immediate per such message, which is what the receiver counts); the first carries the size
  const size_t per = parts > 1 ? ((size + parts - 1) / parts + 127) & ~(size_t)127 : size;
  for (int q = 0; q < parts; ++q) {
    if (parts > 1) {
      const size_t off = std::min(size, (size_t)q * per), len = std::min(per, size - off);
      sge.addr = (uint64_t)(uintptr_t)data + off;
      sge.length = (uint32_t)len;
      wr.num_sge = len ? 1 : 0;
      wr.wr.rdma.remote_addr = c->credits[slot].addr + off;
      wr.imm_data = htonl(q == 0 ? (uint32_t)size : (uint32_t)len);
    }
    if (ibv_post_send(c->qps[q], &wr, &bad) != 0) {
      WARN("NET/IB : posting a send of %zu bytes failed", size);
      c->failed = true;   // parts already posted cannot be taken back
      if (q == 0) { if (tmp) mrPut(c->dev, tmp); r->used = false; }
      return ncclSystemError;
    }
  }
  profRequest(r, phandle, wr.opcode, size);
  c->seq++;
  c->inflight++;
  *request = r;
  return ncclSuccess;
}

ncclResult_t ibIrecv(void* recvComm, int n, void** data, size_t* sizes, int* tags, void** mhandles, void** phandles, void** request) {
  Comm* c = (Comm*)recvComm;
  *request = nullptr;
  if (n != 1) { WARN("NET/IB : grouped receives are not offered (maxRecvs is 1)"); return ncclInvalidArgument; }
  if (c->failed) return ncclRemoteError;
  if ((int)c->waiting.size() >= kSlots || c->creditWrites >= kSlots) return ncclSuccess;
  Request* r = reqGet(c);
  if (!r) return ncclSuccess;
  r->size = sizes[0];
  r->data = (char*)data[0];
  r->seq = c->seq;
  if (sizes[0] > c->eagerBytes) {
    // a message that does not fit an eager buffer comes by RDMA write: tell the sender where to
    uint32_t key;
    if (mhandles && mhandles[0]) key = ((MrHandle*)mhandles[0])->mr->rkey;
    else {
      ncclResult_t res = mrGet(c->dev, data[0], sizes[0], &r->tmpMr);
      if (res != ncclSuccess) { r->used = false; return res; }
      key = r->tmpMr->rkey;
    }
    const int slot = (int)(c->seq % kSlots);
    Credit* cr = &c->outCredits[slot];
    cr->addr = (uint64_t)(uintptr_t)data[0];
    cr->key = key;
    cr->capacity = (uint32_t)std::min<size_t>(sizes[0], 1u << 30);
    cr->tag = tags ? (uint32_t)tags[0] : 0;
    cr->seq = c->seq + 1;
    ibv_sge sge = {(uint64_t)(uintptr_t)cr, (uint32_t)sizeof(Credit), c->outCreditMr->lkey};
    ibv_send_wr wr, *bad = nullptr;
    memset(&wr, 0, sizeof(wr));
    wr.wr_id = kCreditWrId;
    wr.sg_list = &sge;
    wr.num_sge = 1;
    wr.opcode = IBV_WR_RDMA_WRITE;
    wr.send_flags = IBV_SEND_SIGNALED | ((int)sizeof(Credit) <= c->maxInline ? IBV_SEND_INLINE : 0);
    wr.wr.rdma.remote_addr = c->remoteCreditAddr + (uint64_t)slot * sizeof(Credit);
    wr.wr.rdma.rkey = c->remoteCreditKey;
    if (ibv_post_send(c->qps[0], &wr, &bad) != 0) {
      WARN("NET/IB : posting a credit failed");
      if (r->tmpMr) mrPut(c->dev, r->tmpMr);
      r->used = false;
      return ncclSystemError;
    }
    c->creditWrites++;
  }
  profRequest(r, phandles ? phandles[0] : nullptr, IBV_WC_RECV, sizes[0]);
  c->seq++;
  c->waiting.push_back(r);
  *request = r;
  return ncclSuccess;
}

ncclResult_t ibIflush(void*, int, void**, int*, void**, void** request) {
  *request = nullptr;   // host memory needs no flush; device memory is only offered with a peer-memory module, whose writes are ordered by the completion
  return ncclSuccess;
}

ncclResult_t progress(Comm* c) {
  ibv_wc wcs[16];
  for (;;) {
    int n = ibv_poll_cq(c->cq, 16, wcs);
    if (n < 0) { WARN("NET/IB : polling the completion queue failed"); c->failed = true; return ncclSystemError; }
    if (n == 0) break;
    for (int i = 0; i < n; ++i) {
      const ibv_wc& wc = wcs[i];
      if (wc.status != IBV_WC_SUCCESS) {
        WARN("NET/IB : completion with status %d (vendor error 0x%x) on %s, %s side, work request %llu", wc.status, wc.vendor_err, c->dev->name.c_str(),
             c->isSend ? "sending" : "receiving", (unsigned long long)wc.wr_id);
        c->failed = true;
        return ncclRemoteError;
      }
      if (wc.opcode & IBV_WC_RECV) {
        int q = 0;
        while (q < c->nQps && c->qps[q]->qp_num != wc.qp_num) ++q;
        if (q == c->nQps) { WARN("NET/IB : completion of an unknown queue pair %u", wc.qp_num); c->failed = true; return ncclInternalError; }
        Arrival a;
        a.eager = wc.opcode == IBV_WC_RECV;
        a.bytes = a.eager ? wc.byte_len : ntohl(wc.imm_data);
        a.seq = a.eager ? ntohl(wc.imm_data) : 0;
        a.buffer = (int)wc.wr_id;
        c->arrived[q].push_back(a);
      } else if (wc.wr_id == kCreditWrId) {
        c->creditWrites--;
      } else if (wc.wr_id < (uint64_t)kMaxReqs) {
        Request* r = &c->reqs[wc.wr_id];
        if (--r->pending <= 0) {
          r->done = true;
          c->inflight--;
        }
      }
    }
  }
  // The oldest receive meets the oldest arrival of the first queue pair; a message that came by RDMA write is complete once
  // every other queue pair has delivered its part of it as well (their arrivals are in message order too).
  while (!c->isSend && !c->arrived[0].empty() && !c->waiting.empty()) {
    Arrival a = c->arrived[0].front();
    Request* r = c->waiting.front();
    if (a.eager) {
      if (a.seq != r->seq) { WARN("NET/IB : eager message %u arrived where %u was expected", a.seq, r->seq); c->failed = true; return ncclInternalError; }
      if (a.bytes > r->size) { WARN("NET/IB : a message of %u bytes meets a receive of %zu bytes", a.bytes, r->size); c->failed = true; return ncclInvalidUsage; }
      if (a.bytes) memcpy(r->data, c->bounce + (size_t)a.buffer * c->eagerBytes, a.bytes);
    } else {
      bool all = true;
      for (int q = 1; q < c->nQps; ++q) all = all && !c->arrived[q].empty();
      if (!all) break;
      for (int q = 1; q < c->nQps; ++q) {
        NCCLCHECK(postEmpty(c, q, c->arrived[q].front().buffer));
        c->arrived[q].pop_front();
      }
    }
    NCCLCHECK(postBounce(c, a.buffer));
    r->size = a.bytes;
    r->done = true;
    c->arrived[0].pop_front();
    c->waiting.pop_front();
  }
  return ncclSuccess;
}

ncclResult_t ibTest(void* request, int* done, int* sizes) {
  Request* r = (Request*)request;
  *done = 0;
  if (!r->done) NCCLCHECK(progress(r->comm));
  if (!r->done) {
    if (peerGone(r->comm)) {
      WARN("NET/IB : the process at the other end of a connection on %s is gone", r->comm->dev->name.c_str());
      r->comm->failed = true;
      return ncclRemoteError;
    }
    return ncclSuccess;
  }
  r->comm->idlePolls = 0;
  *done = 1;
  if (sizes) sizes[0] = (int)r->size;
  if (r->prof && gProf) gProf(&r->prof, ncclProfilerNetEventStop, nullptr, 0, nullptr);
  if (r->tmpMr) mrPut(r->comm->dev, r->tmpMr);
  r->tmpMr = nullptr;
  r->used = false;
  return ncclSuccess;
}

ncclResult_t ibCloseComm(void* comm) { commFree((Comm*)comm); return ncclSuccess; }
ncclResult_t ibCloseListen(void* listenComm) {
  ListenComm* lc = (ListenComm*)listenComm;
  if (!lc) return ncclSuccess;
  if (lc->pending) commFree(lc->pending);
  sockClose(&lc->sock);
  delete lc;
  return ncclSuccess;
}
ncclResult_t ibGetDeviceMr(void*, void*, void**) { return ncclInternalError; }
ncclResult_t ibIrecvConsumed(void*, int, void*) { return ncclSuccess; }
ncclResult_t ibMakeVDevice(int*, ncclNetVDeviceProps_t*) { return ncclInvalidUsage; }
ncclResult_t ibFinalize(void*) { return ncclSuccess; }
ncclResult_t ibSetNetAttr(void*, ncclNetAttr_t*) { return ncclSuccess; }

}  // namespace

ncclNet_t netIbBackend = {"IB", ibInit, ibDevices, ibGetProperties, ibListen, ibConnect, ibAccept, ibRegMr, ibRegMrDmaBuf, ibDeregMr, ibIsend, ibIrecv,
                          ibIflush, ibTest, ibCloseComm, ibCloseComm, ibCloseListen, ibGetDeviceMr, ibIrecvConsumed, ibMakeVDevice, ibFinalize, ibSetNetAttr};

}  // namespace b200
