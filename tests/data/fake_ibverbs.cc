// A stand-in for libibverbs for tests on machines without RDMA hardware: devices "fakeib0..", reliable-connected queue
// pairs whose traffic travels over abstract UNIX stream sockets between (or inside) processes. It implements what the
// InfiniBand backend calls: device / port / GID queries, protection domains, memory regions with key and bounds checks,
// completion queues, queue-pair state changes, and the operations SEND, SEND with immediate, RDMA WRITE and RDMA WRITE
// with immediate, with receiver-not-ready handled by waiting for a posted receive.
// Addressing: a port's LID (and the low bits of its GID) name the owning process; a process listens on "\0fakeib-<lid>".
// Environment: FAKE_IB_DEVICES (count, default 2), FAKE_IB_LINK (IB or ETH, default ETH), FAKE_IB_INLINE (max inline bytes, default 64).
// Protocol violations by the caller (bad keys, out-of-bounds, wrong state order) are counted: fake_ib_errors().
#include <errno.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "ibv_abi.h"

namespace {

std::atomic<int> gErrors{0};
// attributes of the last state changes, for tests of how the caller's settings reach the queue pair
std::atomic<int> gLastPkey{-1}, gLastSgid{-1}, gLastTc{-1}, gLastSl{-1}, gLastTimeout{-1}, gLastRetry{-1}, gLastMtu{-1};
void fail(const char* what) {
  gErrors++;
  fprintf(stderr, "fake_ibverbs[%d]: %s\n", (int)getpid(), what);
}

struct FakeCq {
  ibv_cq base;
  std::mutex lock;
  std::deque<ibv_wc> done;
  void push(const ibv_wc& wc) { std::lock_guard<std::mutex> g(lock); done.push_back(wc); }
};

struct RecvWr { uint64_t id; std::vector<ibv_sge> sge; };

struct FakeQp {
  ibv_qp base;
  std::mutex lock;
  std::condition_variable posted;
  std::deque<RecvWr> recvq;
  uint32_t destQpn = 0;
  uint32_t destKey = 0;      // process key (LID) of the other end
  int maxInline = 0;
  int fd = -1;               // stream to the other end's process, opened by the first send
  bool dead = false;
};

struct Mr { char* addr; size_t len; int access; };

std::mutex gLock;
std::map<uint32_t, FakeQp*> gQps;
std::map<uint32_t, Mr> gMrs;
uint32_t gNextQpn = 0, gNextKey = 0x1000;
uint32_t gProcKey = 0;
std::once_flag gServiceOnce;
int gListenFd = -1;

uint32_t procKey() { return 1 + (uint32_t)getpid() % 65000; }

struct Wire { uint32_t dstQpn, opcode, rkey, imm, len, srcQpn; uint64_t raddr; };

bool readAll(int fd, void* p, size_t n) {
  char* c = (char*)p;
  while (n) { ssize_t r = read(fd, c, n); if (r <= 0) { if (r < 0 && errno == EINTR) continue; return false; } c += r; n -= r; }
  return true;
}
bool writeAll(int fd, const void* p, size_t n) {
  const char* c = (const char*)p;
  while (n) { ssize_t r = send(fd, c, n, MSG_NOSIGNAL); if (r <= 0) { if (r < 0 && errno == EINTR) continue; return false; } c += r; n -= r; }
  return true;
}

void sockName(sockaddr_un* a, socklen_t* len, uint32_t key) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  int n = snprintf(a->sun_path + 1, sizeof(a->sun_path) - 1, "fakeib-%u", key);
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

bool checkMr(uint32_t key, uint64_t addr, size_t len, int needAccess) {
  if (len == 0) return true;
  std::lock_guard<std::mutex> g(gLock);
  auto it = gMrs.find(key);
  if (it == gMrs.end()) return false;
  const Mr& m = it->second;
  return (char*)addr >= m.addr && (char*)addr + len <= m.addr + m.len && (m.access & needAccess) == needAccess;
}

// One incoming stream: operations of one remote queue pair, in order.
void serve(int fd) {
  std::vector<char> payload;
  for (;;) {
    Wire w;
    if (!readAll(fd, &w, sizeof(w))) break;
    payload.resize(w.len);
    if (w.len && !readAll(fd, payload.data(), w.len)) break;
    FakeQp* qp = nullptr;
    {
      std::lock_guard<std::mutex> g(gLock);
      auto it = gQps.find(w.dstQpn);
      if (it != gQps.end()) qp = it->second;
    }
    if (!qp) { fail("operation for an unknown queue pair"); continue; }
    if (qp->base.state != IBV_QPS_RTR && qp->base.state != IBV_QPS_RTS) { fail("operation for a queue pair that is not ready to receive"); continue; }
    if (qp->destQpn != w.srcQpn) { fail("operation from a queue pair this one is not connected to"); continue; }
    const bool write = w.opcode == IBV_WR_RDMA_WRITE || w.opcode == IBV_WR_RDMA_WRITE_WITH_IMM;
    const bool consumes = w.opcode != IBV_WR_RDMA_WRITE;
    if (write) {
      if (!checkMr(w.rkey, w.raddr, w.len, IBV_ACCESS_REMOTE_WRITE)) { fail("RDMA write outside a region registered for remote writing"); continue; }
      if (w.len) memcpy((void*)w.raddr, payload.data(), w.len);
    }
    if (!consumes) continue;
    RecvWr rw;
    {
      std::unique_lock<std::mutex> g(qp->lock);
      qp->posted.wait(g, [&] { return !qp->recvq.empty() || qp->dead; });   // receiver not ready: wait for a posted receive
      if (qp->dead) break;
      rw = qp->recvq.front();
      qp->recvq.pop_front();
    }
    ibv_wc wc;
    memset(&wc, 0, sizeof(wc));
    wc.wr_id = rw.id;
    wc.qp_num = qp->base.qp_num;
    wc.src_qp = w.srcQpn;
    wc.byte_len = w.len;
    wc.opcode = write ? IBV_WC_RECV_RDMA_WITH_IMM : IBV_WC_RECV;
    if (w.opcode == IBV_WR_RDMA_WRITE_WITH_IMM || w.opcode == IBV_WR_SEND_WITH_IMM) { wc.wc_flags = IBV_WC_WITH_IMM; wc.imm_data = w.imm; }
    if (!write) {
      size_t off = 0;
      for (auto& s : rw.sge) {
        size_t n = std::min<size_t>(s.length, w.len - off);
        if (n && !checkMr(s.lkey, s.addr, n, IBV_ACCESS_LOCAL_WRITE)) { fail("receive buffer outside its region"); wc.status = IBV_WC_LOC_PROT_ERR; break; }
        if (n) memcpy((void*)s.addr, payload.data() + off, n);
        off += n;
      }
      if (wc.status == IBV_WC_SUCCESS && off < w.len) { fail("message longer than the posted receive"); wc.status = IBV_WC_LOC_LEN_ERR; }
    }
    ((FakeCq*)qp->base.recv_cq)->push(wc);
  }
  close(fd);
}

void service() {
  for (;;) {
    int fd = accept(gListenFd, nullptr, nullptr);
    if (fd < 0) { if (errno == EINTR) continue; return; }
    std::thread(serve, fd).detach();
  }
}

void startService() {
  std::call_once(gServiceOnce, [] {
    gProcKey = procKey();
    gNextQpn = 0x100 + ((uint32_t)getpid() % 1000) * 0x1000;
    gListenFd = socket(AF_UNIX, SOCK_STREAM, 0);
    sockaddr_un a;
    socklen_t len;
    sockName(&a, &len, gProcKey);
    if (bind(gListenFd, (sockaddr*)&a, len) != 0 || listen(gListenFd, 256) != 0) { fail("cannot listen (another process with the same key?)"); return; }
    std::thread(service).detach();
  });
}

int fakePoll(ibv_cq* cq, int n, ibv_wc* wc) {
  FakeCq* c = (FakeCq*)cq;
  std::lock_guard<std::mutex> g(c->lock);
  int k = 0;
  while (k < n && !c->done.empty()) { wc[k++] = c->done.front(); c->done.pop_front(); }
  return k;
}

int fakePostRecv(ibv_qp* q, ibv_recv_wr* wr, ibv_recv_wr** bad) {
  FakeQp* qp = (FakeQp*)q;
  if (q->state == IBV_QPS_RESET) { fail("receive posted to a queue pair in reset"); *bad = wr; return EINVAL; }
  for (; wr; wr = wr->next) {
    RecvWr r;
    r.id = wr->wr_id;
    for (int i = 0; i < wr->num_sge; ++i) r.sge.push_back(wr->sg_list[i]);
    std::lock_guard<std::mutex> g(qp->lock);
    qp->recvq.push_back(r);
    qp->posted.notify_all();
  }
  return 0;
}

int fakePostSend(ibv_qp* q, ibv_send_wr* wr, ibv_send_wr** bad) {
  FakeQp* qp = (FakeQp*)q;
  for (; wr; wr = wr->next) {
    if (q->state != IBV_QPS_RTS) { fail("send posted to a queue pair that is not ready to send"); *bad = wr; return EINVAL; }
    if (wr->opcode > IBV_WR_SEND_WITH_IMM) { fail("operation the fake does not implement"); *bad = wr; return EINVAL; }
    size_t len = 0;
    for (int i = 0; i < wr->num_sge; ++i) len += wr->sg_list[i].length;
    if ((wr->send_flags & IBV_SEND_INLINE) && (int)len > qp->maxInline) { fail("inline send longer than max_inline_data"); *bad = wr; return ENOMEM; }
    std::vector<char> buf(len);
    size_t off = 0;
    for (int i = 0; i < wr->num_sge; ++i) {
      const ibv_sge& s = wr->sg_list[i];
      if (!(wr->send_flags & IBV_SEND_INLINE) && !checkMr(s.lkey, s.addr, s.length, 0)) { fail("send buffer outside the region of its key"); *bad = wr; return EINVAL; }
      if (s.length) memcpy(buf.data() + off, (void*)s.addr, s.length);
      off += s.length;
    }
    std::lock_guard<std::mutex> g(qp->lock);
    if (qp->fd < 0) {
      qp->fd = socket(AF_UNIX, SOCK_STREAM, 0);
      sockaddr_un a;
      socklen_t alen;
      sockName(&a, &alen, qp->destKey);
      if (connect(qp->fd, (sockaddr*)&a, alen) != 0) { fail("the other end's process is not reachable"); close(qp->fd); qp->fd = -1; *bad = wr; return ENETUNREACH; }
    }
    Wire w = {qp->destQpn, (uint32_t)wr->opcode, wr->wr.rdma.rkey, wr->imm_data, (uint32_t)len, q->qp_num, wr->wr.rdma.remote_addr};
    ibv_wc wc;
    memset(&wc, 0, sizeof(wc));
    wc.wr_id = wr->wr_id;
    wc.qp_num = q->qp_num;
    wc.opcode = (wr->opcode == IBV_WR_SEND || wr->opcode == IBV_WR_SEND_WITH_IMM) ? IBV_WC_SEND : IBV_WC_RDMA_WRITE;
    if (!writeAll(qp->fd, &w, sizeof(w)) || (len && !writeAll(qp->fd, buf.data(), len))) wc.status = IBV_WC_RETRY_EXC_ERR;
    if ((wr->send_flags & IBV_SEND_SIGNALED) || wc.status != IBV_WC_SUCCESS) ((FakeCq*)q->send_cq)->push(wc);
  }
  return 0;
}

struct FakeDev {
  ibv_device dev;
  ibv_context ctx;
  int index;
};
std::vector<FakeDev*> gDevs;
std::once_flag gDevOnce;

void makeDevices() {
  std::call_once(gDevOnce, [] {
    const char* e = getenv("FAKE_IB_DEVICES");
    int n = e ? atoi(e) : 2;
    for (int i = 0; i < n; ++i) {
      FakeDev* d = new FakeDev();
      memset(&d->dev, 0, sizeof(d->dev));
      memset(&d->ctx, 0, sizeof(d->ctx));
      snprintf(d->dev.name, sizeof(d->dev.name), "fakeib%d", i);
      snprintf(d->dev.ibdev_path, sizeof(d->dev.ibdev_path), "/sys/class/infiniband/fakeib%d", i);
      d->ctx.device = &d->dev;
      d->ctx.ops[IBV_OP_POLL_CQ] = (void*)fakePoll;
      d->ctx.ops[IBV_OP_POST_SEND] = (void*)fakePostSend;
      d->ctx.ops[IBV_OP_POST_RECV] = (void*)fakePostRecv;
      d->index = i;
      gDevs.push_back(d);
    }
  });
}

bool linkIsIb() { const char* e = getenv("FAKE_IB_LINK"); return e && strcmp(e, "IB") == 0; }

}  // namespace

extern "C" {

int fake_ib_errors() { return gErrors.load(); }
// what: 0 pkey index, 1 source GID index, 2 traffic class, 3 service level, 4 time-out, 5 retry count, 6 path MTU
int fake_ib_last(int what) {
  switch (what) {
    case 0: return gLastPkey; case 1: return gLastSgid; case 2: return gLastTc; case 3: return gLastSl; case 4: return gLastTimeout; case 5: return gLastRetry;
    case 6: return gLastMtu; default: return -1;
  }
}

ibv_device** ibv_get_device_list(int* n) {
  makeDevices();
  ibv_device** list = (ibv_device**)calloc(gDevs.size() + 1, sizeof(ibv_device*));
  for (size_t i = 0; i < gDevs.size(); ++i) list[i] = &gDevs[i]->dev;
  if (n) *n = (int)gDevs.size();
  return list;
}
void ibv_free_device_list(ibv_device** list) { free(list); }
const char* ibv_get_device_name(ibv_device* d) { return d->name; }
ibv_context* ibv_open_device(ibv_device* d) {
  startService();
  for (auto* f : gDevs) if (&f->dev == d) return &f->ctx;
  return nullptr;
}
int ibv_close_device(ibv_context*) { return 0; }
int ibv_fork_init() { return 0; }

int ibv_query_device(ibv_context* c, ibv_device_attr* a) {
  memset(a, 0, offsetof(ibv_device_attr, spare));
  FakeDev* d = nullptr;
  for (auto* f : gDevs) if (&f->ctx == c) d = f;
  if (!d) return EINVAL;
  a->node_guid = 0xfa4e000000000000ULL + ((uint64_t)procKey() << 8) + d->index;
  a->max_qp = 4096;
  a->max_qp_wr = 1024;
  a->max_cqe = 65536;
  a->max_sge = 4;
  a->max_mr = 65536;
  a->phys_port_cnt = 1;
  return 0;
}
int ibv_query_port(ibv_context*, uint8_t port, ibv_port_attr* a) {
  if (port != 1) return EINVAL;
  memset(a, 0, offsetof(ibv_port_attr, spare));
  a->state = IBV_PORT_ACTIVE;
  a->max_mtu = a->active_mtu = IBV_MTU_4096;
  a->gid_tbl_len = 4;
  a->lid = linkIsIb() ? (uint16_t)procKey() : 0;
  a->link_layer = linkIsIb() ? IBV_LINK_LAYER_INFINIBAND : IBV_LINK_LAYER_ETHERNET;
  a->active_width = 2;    // 4x
  a->active_speed = 64;   // NDR
  a->max_msg_sz = 1u << 30;
  return 0;
}
int ibv_query_gid(ibv_context* c, uint8_t port, int index, ibv_gid* gid) {
  if (port != 1 || index < 0 || index >= 4) return EINVAL;
  FakeDev* d = nullptr;
  for (auto* f : gDevs) if (&f->ctx == c) d = f;
  memset(gid, 0, sizeof(*gid));
  gid->raw[0] = 0xfe;
  gid->raw[1] = 0x80;
  gid->raw[8] = (uint8_t)index;
  gid->raw[9] = d ? (uint8_t)d->index : 0;
  uint32_t k = procKey();
  gid->raw[12] = (uint8_t)(k >> 24); gid->raw[13] = (uint8_t)(k >> 16); gid->raw[14] = (uint8_t)(k >> 8); gid->raw[15] = (uint8_t)k;
  return 0;
}

ibv_pd* ibv_alloc_pd(ibv_context* c) { ibv_pd* p = (ibv_pd*)calloc(1, sizeof(ibv_pd)); p->context = c; return p; }
int ibv_dealloc_pd(ibv_pd* p) { free(p); return 0; }

ibv_mr* ibv_reg_mr(ibv_pd* pd, void* addr, size_t len, int access) {
  if ((access & IBV_ACCESS_REMOTE_WRITE) && !(access & IBV_ACCESS_LOCAL_WRITE)) { fail("remote write access without local write access"); errno = EINVAL; return nullptr; }
  ibv_mr* m = (ibv_mr*)calloc(1, sizeof(ibv_mr));
  m->context = pd->context;
  m->pd = pd;
  m->addr = addr;
  m->length = len;
  std::lock_guard<std::mutex> g(gLock);
  m->lkey = m->rkey = m->handle = gNextKey++;
  gMrs[m->lkey] = Mr{(char*)addr, len, access};
  return m;
}
int ibv_dereg_mr(ibv_mr* m) {
  { std::lock_guard<std::mutex> g(gLock); if (!gMrs.erase(m->lkey)) fail("deregistration of an unknown region"); }
  free(m);
  return 0;
}

ibv_cq* ibv_create_cq(ibv_context* c, int cqe, void* cq_context, void* channel, int) {
  FakeCq* q = new FakeCq();
  memset(&q->base, 0, sizeof(q->base));
  q->base.context = c;
  q->base.cq_context = cq_context;
  q->base.channel = channel;
  q->base.cqe = cqe;
  return &q->base;
}
int ibv_destroy_cq(ibv_cq* cq) { delete (FakeCq*)cq; return 0; }

ibv_qp* ibv_create_qp(ibv_pd* pd, ibv_qp_init_attr* a) {
  if (a->qp_type != IBV_QPT_RC) { fail("only reliable-connected queue pairs exist here"); errno = EINVAL; return nullptr; }
  FakeQp* q = new FakeQp();
  memset(&q->base, 0, sizeof(q->base));
  q->base.context = pd->context;
  q->base.pd = pd;
  q->base.send_cq = a->send_cq;
  q->base.recv_cq = a->recv_cq;
  q->base.qp_type = a->qp_type;
  q->base.state = IBV_QPS_RESET;
  const char* e = getenv("FAKE_IB_INLINE");
  q->maxInline = e ? atoi(e) : 64;
  if ((int)a->cap.max_inline_data > q->maxInline) { delete q; errno = EINVAL; return nullptr; }
  a->cap.max_inline_data = q->maxInline;
  std::lock_guard<std::mutex> g(gLock);
  q->base.qp_num = q->base.handle = ++gNextQpn;
  gQps[q->base.qp_num] = q;
  return &q->base;
}

int ibv_modify_qp(ibv_qp* q, ibv_qp_attr* a, int mask) {
  FakeQp* qp = (FakeQp*)q;
  if (!(mask & IBV_QP_STATE)) return 0;
  const int from = q->state, to = a->qp_state;
  const bool ok = (to == IBV_QPS_INIT && from == IBV_QPS_RESET) || (to == IBV_QPS_RTR && from == IBV_QPS_INIT) || (to == IBV_QPS_RTS && from == IBV_QPS_RTR) ||
                  to == IBV_QPS_ERR || to == IBV_QPS_RESET;
  if (!ok) { fail("queue pair state change out of order"); return EINVAL; }
  if (to == IBV_QPS_INIT && (mask & (IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS)) != (IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS)) { fail("INIT without port, key index and access flags"); return EINVAL; }
  if (to == IBV_QPS_INIT) gLastPkey = a->pkey_index;
  if (to == IBV_QPS_RTR) {
    gLastSl = a->ah_attr.sl;
    gLastMtu = a->path_mtu;
    if (a->ah_attr.is_global) { gLastSgid = a->ah_attr.grh.sgid_index; gLastTc = a->ah_attr.grh.traffic_class; }
    const int need = IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN | IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER;
    if ((mask & need) != need) { fail("RTR without its required attributes"); return EINVAL; }
    qp->destQpn = a->dest_qp_num;
    if (a->ah_attr.is_global) {
      const uint8_t* r = a->ah_attr.grh.dgid.raw;
      qp->destKey = ((uint32_t)r[12] << 24) | ((uint32_t)r[13] << 16) | ((uint32_t)r[14] << 8) | r[15];
    } else {
      if (!linkIsIb()) { fail("an Ethernet port needs a global route"); return EINVAL; }
      qp->destKey = a->ah_attr.dlid;
    }
  }
  if (to == IBV_QPS_RTS) {
    gLastTimeout = a->timeout;
    gLastRetry = a->retry_cnt;
    const int need = IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN | IBV_QP_MAX_QP_RD_ATOMIC;
    if ((mask & need) != need) { fail("RTS without its required attributes"); return EINVAL; }
  }
  q->state = to;
  return 0;
}

int ibv_destroy_qp(ibv_qp* q) {
  FakeQp* qp = (FakeQp*)q;
  {
    std::lock_guard<std::mutex> g(gLock);
    gQps.erase(q->qp_num);
  }
  {
    std::lock_guard<std::mutex> g(qp->lock);
    qp->dead = true;
    if (qp->fd >= 0) close(qp->fd);
    qp->posted.notify_all();
  }
  // a serving thread may still hold the pointer for a moment: the object is kept (a test process is short-lived)
  return 0;
}

}  // extern "C"
