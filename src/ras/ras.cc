// RAS thread of a process. One listening socket for the other processes of the job (its
// address travels in the bootstrap ring record of every rank), one for clients on
// NCCL_RAS_ADDR (default localhost:28028; the first process of a host that binds it serves it).
//
// Between processes (length-prefixed text frames):
//   PING            -> PONG                        keep-alive; each process pings its successor in
//                                                  the address-sorted ring of known processes
//   DEAD <addr>     -> OK                          a process that saw a peer die tells the others
//   COMMS           -> one line per communicator   local state for a status report
// Client protocol (line based, the one the ncclras tool speaks):
//   CLIENT PROTOCOL <n> -> SERVER PROTOCOL 2 | TIMEOUT <s> -> OK | SET FORMAT text|json -> OK
//   STATUS | VERBOSE STATUS -> report, then the server closes the connection
//   MONITOR [groups]        -> OK, then one line per event ("<seconds> <group> <text>") until the client goes away;
//                              groups: comma-separated from lifecycle (communicators come and go), peers (processes
//                              declared dead), all (default)
// A status report is a collective over processes: the serving process asks every known process
// for its communicators (in a worker thread, so the RAS thread keeps answering others), marks
// the ones that do not answer in time, and compares operation counts across the ranks of each
// communicator to point at ranks that lag behind.
// Reference parity: src/ras/ras.cc (thread, poll loop :581-683), rasnet.cc (keep-alives, retry),
// peers.cc (dead peers), collectives.cc (status gathering with time-outs), client_support.cc
// (report layout), ras_internal.h (port 28028 :11, timing constants :200-235).
#include "ras.h"

#include <fcntl.h>
#include <netdb.h>
#include <poll.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <deque>
#include <set>
#include <sstream>

#include "../core/socket.h"

namespace b200 {

B200_PARAM(RasKeepAliveMs, "B200_RAS_KEEPALIVE_MS", 1000, "interval of RAS keep-alive pings, milliseconds");
B200_PARAM(RasTimeoutFactor, "RAS_TIMEOUT_FACTOR", 1, "multiplier applied to every RAS time-out");
B200_PARAM(RasDeadAfter, "B200_RAS_DEAD_AFTER", 5, "missed keep-alives after which a process is declared dead");

namespace {

struct CommRec {
  ncclComm* comm;
  uint64_t hash;
  int rank, nRanks, cudaDev;
  std::vector<RasRankInit> ranks;   // RAS record of every rank
};

struct PeerProc {
  SockAddr addr;
  int pid = 0;
  uint64_t hostHash = 0;
  int missed = 0;
  bool dead = false;
};

struct Ras {
  std::mutex lock;
  std::thread thread;
  bool started = false, stop = false;
  int peerFd = -1, clientFd = -1, wakeFd[2] = {-1, -1};
  SockAddr peerAddr{};
  std::vector<CommRec> comms;
  std::map<std::string, PeerProc> peers;   // keyed by "ip:port" of the peer's RAS socket
  std::set<std::string> deadNotified;
  // events for clients in monitor mode: a bounded log with running sequence numbers
  std::deque<std::pair<uint64_t, std::string>> events;
  uint64_t nextEvent = 1;
};
Ras gRas;

// Appends an event (caller holds gRas.lock). Group is "lifecycle" or "peers".
void eventLocked(const char* group, const std::string& text) {
  char head[64];
  snprintf(head, sizeof(head), "%.3f %s ", (double)std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::system_clock::now().time_since_epoch()).count() / 1e3, group);
  gRas.events.emplace_back(gRas.nextEvent++, std::string(head) + text);
  while (gRas.events.size() > 1024) gRas.events.pop_front();
}

int64_t scaled(int64_t ms) { return ms * std::max<int64_t>(paramRasTimeoutFactor(), 1); }

// ---- small blocking-with-deadline socket helpers (RAS must never hang on a sick peer)
bool waitFd(int fd, short ev, int64_t ms) {
  struct pollfd p = {fd, ev, 0};
  return poll(&p, 1, (int)ms) > 0 && (p.revents & ev);
}
int connectTo(const SockAddr& a, int64_t ms) {
  int fd = socket(a.sa.sa_family, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK);
  int r = connect(fd, &a.sa, sockAddrLen(&a));
  if (r != 0 && errno != EINPROGRESS) { close(fd); return -1; }
  if (r != 0) {
    if (!waitFd(fd, POLLOUT, ms)) { close(fd); return -1; }
    int err = 0;
    socklen_t l = sizeof(err);
    getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &l);
    if (err) { close(fd); return -1; }
  }
  return fd;
}
bool sendAll(int fd, const void* p, size_t n, int64_t ms) {
  size_t off = 0;
  while (off < n) {
    ssize_t k = send(fd, (const char*)p + off, n - off, MSG_NOSIGNAL | MSG_DONTWAIT);
    if (k > 0) { off += k; continue; }
    if (k < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) { if (!waitFd(fd, POLLOUT, ms)) return false; continue; }
    return false;
  }
  return true;
}
bool recvAll(int fd, void* p, size_t n, int64_t ms) {
  size_t off = 0;
  while (off < n) {
    ssize_t k = recv(fd, (char*)p + off, n - off, MSG_DONTWAIT);
    if (k > 0) { off += k; continue; }
    if (k < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) { if (!waitFd(fd, POLLIN, ms)) return false; continue; }
    return false;
  }
  return true;
}
bool sendFrame(int fd, const std::string& s, int64_t ms) {
  uint32_t n = (uint32_t)s.size();
  return sendAll(fd, &n, 4, ms) && sendAll(fd, s.data(), n, ms);
}
bool recvFrame(int fd, std::string* s, int64_t ms) {
  uint32_t n = 0;
  if (!recvAll(fd, &n, 4, ms) || n > (64u << 20)) return false;
  s->resize(n);
  return n == 0 || recvAll(fd, &(*s)[0], n, ms);
}
bool recvLine(int fd, std::string* line, int64_t ms) {
  line->clear();
  char c;
  while (line->size() < 4096) {
    if (!recvAll(fd, &c, 1, ms)) return !line->empty();
    if (c == '\n') return true;
    if (c != '\r') line->push_back(c);
  }
  return true;
}
// request/response with a peer process; false when it did not answer in time
bool ask(const SockAddr& a, const std::string& req, std::string* resp, int64_t ms) {
  int fd = connectTo(a, ms);
  if (fd < 0) return false;
  bool ok = sendFrame(fd, req, ms) && recvFrame(fd, resp, ms);
  close(fd);
  return ok;
}

int listenOnAddr(SockAddr* a) {
  int fd = socket(a->sa.sa_family, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  if (bind(fd, &a->sa, sockAddrLen(a)) != 0 || listen(fd, 256) != 0) { close(fd); return -1; }
  socklen_t l = sizeof(*a);
  getsockname(fd, &a->sa, &l);
  fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK);
  return fd;
}

std::string localCommsText() {
  std::ostringstream o;
  std::lock_guard<std::mutex> g(gRas.lock);
  for (auto& c : gRas.comms) {
    ncclComm* k = c.comm;
    const bool aborted = k->abortFlag && *k->abortFlag;
    o << std::hex << c.hash << std::dec << ' ' << c.rank << ' ' << c.nRanks << ' ' << k->opCount.load() << ' ' << k->asyncResult.load() << ' ' << (aborted ? 1 : 0)
      << ' ' << c.cudaDev << ' ' << (int)getpid() << ' ' << k->nNodes << '\n';
  }
  return o.str();
}

void markDead(const std::string& key, bool notify) {
  std::vector<SockAddr> others;
  {
    std::lock_guard<std::mutex> g(gRas.lock);
    auto it = gRas.peers.find(key);
    if (it == gRas.peers.end() || it->second.dead) return;
    it->second.dead = true;
    eventLocked("peers", "process " + key + " (pid " + std::to_string(it->second.pid) + ") declared dead");
    if (notify && gRas.deadNotified.insert(key).second)
      for (auto& p : gRas.peers) if (!p.second.dead && sockAddrToString(&p.second.addr) != sockAddrToString(&gRas.peerAddr)) others.push_back(p.second.addr);
  }
  WARN("RAS: process at %s does not answer keep-alives any more; declaring it dead", key.c_str());
  for (auto& a : others) {
    std::string r;
    ask(a, "DEAD " + key, &r, scaled(500));
  }
}

void servePeer(int fd) {
  std::string req;
  if (!recvFrame(fd, &req, scaled(1000))) { close(fd); return; }
  std::string resp = "ERR";
  if (req == "PING") resp = "PONG";
  else if (req == "COMMS") resp = localCommsText();
  else if (req.compare(0, 5, "DEAD ") == 0) { markDead(req.substr(5), false); resp = "OK"; }
  sendFrame(fd, resp, scaled(1000));
  close(fd);
}

// ---- status report
struct RankState { uint64_t opCount = 0; int asyncError = 0, aborted = 0, cudaDev = -1, pid = 0; bool seen = false; std::string proc; };
struct CommState { int nRanks = 0, nNodes = 1; std::map<int, RankState> ranks; };

void buildReport(bool verbose, bool json, int64_t timeoutMs, std::string* out) {
  std::map<std::string, PeerProc> peers;
  std::string self;
  {
    std::lock_guard<std::mutex> g(gRas.lock);
    peers = gRas.peers;
    self = sockAddrToString(&gRas.peerAddr);
  }
  std::map<uint64_t, CommState> comms;
  std::vector<std::string> unresponsive, dead;
  std::set<uint64_t> hosts;
  int nProcs = 0, nGpus = 0;
  auto absorb = [&](const std::string& key, const std::string& text) {
    std::istringstream in(text);
    std::string line;
    while (std::getline(in, line)) {
      std::istringstream l(line);
      uint64_t hash;
      int rank, n, async, ab, dev, pid, nodes;
      uint64_t ops;
      if (!(l >> std::hex >> hash >> std::dec >> rank >> n >> ops >> async >> ab >> dev >> pid >> nodes)) continue;
      CommState& cs = comms[hash];
      cs.nRanks = n;
      cs.nNodes = nodes;
      RankState& rs = cs.ranks[rank];
      rs.opCount = ops; rs.asyncError = async; rs.aborted = ab; rs.cudaDev = dev; rs.pid = pid; rs.seen = true; rs.proc = key;
      if (dev >= 0) ++nGpus;
    }
  };
  for (auto& p : peers) {
    hosts.insert(p.second.hostHash);
    if (p.second.dead) { dead.push_back(p.first); continue; }
    ++nProcs;
    if (p.first == self) { absorb(p.first, localCommsText()); continue; }
    std::string resp;
    if (ask(p.second.addr, "COMMS", &resp, timeoutMs)) absorb(p.first, resp);
    else unresponsive.push_back(p.first);
  }
  // findings
  std::vector<std::string> errors;
  for (auto& d : dead) errors.push_back("process " + d + " is DEAD (stopped answering keep-alives)");
  for (auto& u : unresponsive) errors.push_back("process " + u + " did not answer the status request in time (UNRESPONSIVE)");
  std::ostringstream commLines, commJson;
  int gi = 0;
  for (auto& c : comms) {
    CommState& cs = c.second;
    uint64_t maxOps = 0;
    int missing = 0, errs = 0, aborted = 0;
    for (auto& r : cs.ranks) maxOps = std::max(maxOps, r.second.opCount);
    std::vector<int> lagging;
    for (int r = 0; r < cs.nRanks; ++r) {
      auto it = cs.ranks.find(r);
      if (it == cs.ranks.end()) { ++missing; continue; }
      if (it->second.asyncError != 0 && it->second.asyncError != (int)ncclInProgress) ++errs;
      if (it->second.aborted) ++aborted;
      if (it->second.opCount < maxOps) lagging.push_back(r);
    }
    const char* status = missing ? "INCOMPLETE" : aborted ? "ABORTED" : errs ? "ERROR" : "RUNNING";
    std::ostringstream e;
    if (missing) e << missing << " rank(s) not reporting; ";
    if (errs) e << errs << " rank(s) with an asynchronous error; ";
    if (!lagging.empty()) {
      e << "operation count MISMATCH, behind:";
      for (int r : lagging) e << ' ' << r;
    }
    std::string es = e.str().empty() ? "OK" : e.str();
    char line[512];
    snprintf(line, sizeof(line), "%5d  0x%016llx  %5d  %5d  %10llu  %-10s  %s\n", gi, (unsigned long long)c.first, cs.nRanks, cs.nNodes, (unsigned long long)maxOps, status, es.c_str());
    commLines << line;
    if (verbose)
      for (auto& r : cs.ranks) {
        snprintf(line, sizeof(line), "         rank %d: pid %d cudaDev %d opCount %llu asyncError %d%s (process %s)\n", r.first, r.second.pid, r.second.cudaDev,
                 (unsigned long long)r.second.opCount, r.second.asyncError, r.second.aborted ? " ABORTED" : "", r.second.proc.c_str());
        commLines << line;
      }
    if (es != "OK") { char h[32]; snprintf(h, sizeof(h), "0x%llx", (unsigned long long)c.first); errors.push_back(std::string("communicator ") + h + ": " + es); }
    commJson << (gi ? "," : "") << "{\"hash\":\"0x" << std::hex << c.first << std::dec << "\",\"nranks\":" << cs.nRanks << ",\"nnodes\":" << cs.nNodes << ",\"op_count\":" << maxOps
             << ",\"status\":\"" << status << "\",\"missing_ranks\":" << missing << ",\"lagging_ranks\":[";
    for (size_t i = 0; i < lagging.size(); ++i) commJson << (i ? "," : "") << lagging[i];
    commJson << "]}";
    ++gi;
  }
  std::ostringstream o;
  int rtv = 0, drv = 0;
  cudaRuntimeGetVersion(&rtv);
  cudaDriverGetVersion(&drv);
  (void)cudaGetLastError();
  if (json) {
    o << "{\"nccl_version\":\"" << NCCL_MAJOR << '.' << NCCL_MINOR << '.' << NCCL_PATCH << NCCL_SUFFIX << "\",\"cuda_runtime\":" << rtv << ",\"cuda_driver\":" << drv
      << ",\"job\":{\"nodes\":" << hosts.size() << ",\"processes\":" << nProcs << ",\"gpus\":" << nGpus << ",\"dead_processes\":" << dead.size()
      << ",\"unresponsive_processes\":" << unresponsive.size() << "},\"communicators\":[" << commJson.str() << "],\"errors\":[";
    for (size_t i = 0; i < errors.size(); ++i) o << (i ? "," : "") << '"' << errors[i] << '"';
    o << "]}\n";
  } else {
    o << "NCCL version " << NCCL_MAJOR << '.' << NCCL_MINOR << '.' << NCCL_PATCH << NCCL_SUFFIX << " compiled with CUDA " << CUDART_VERSION / 1000 << '.' << (CUDART_VERSION % 1000) / 10 << "\n";
    o << "CUDA runtime version " << rtv << ", driver version " << drv << "\n\n";
    o << "Job summary\n===========\n\n  Nodes  Processes   GPUs  Dead  Unresponsive\n";
    char line[256];
    snprintf(line, sizeof(line), "  %5zu  %9d  %5d  %4zu  %12zu\n\n", hosts.size(), nProcs, nGpus, dead.size(), unresponsive.size());
    o << line;
    o << "Communicators\n=============\n\nGroup  Hash                Ranks  Nodes    Op count  Status      Errors\n" << commLines.str() << "\n";
    o << "Errors\n======\n\n";
    if (errors.empty()) o << "  none\n";
    for (auto& e : errors) o << "  " << e << "\n";
  }
  *out = o.str();
}

void serveClient(int fd) {
  int64_t timeoutMs = scaled(5000);
  bool json = false;
  std::string line;
  while (recvLine(fd, &line, 30000)) {
    if (line.compare(0, 15, "CLIENT PROTOCOL") == 0) sendAll(fd, "SERVER PROTOCOL 2\n", 18, 1000);
    else if (line.compare(0, 8, "TIMEOUT ") == 0) { timeoutMs = std::max(1, atoi(line.c_str() + 8)) * 1000; sendAll(fd, "OK\n", 3, 1000); }
    else if (line == "SET FORMAT json") { json = true; sendAll(fd, "OK\n", 3, 1000); }
    else if (line == "SET FORMAT text") { json = false; sendAll(fd, "OK\n", 3, 1000); }
    else if (line == "STATUS" || line == "VERBOSE STATUS") {
      std::string rep;
      buildReport(line[0] == 'V', json, timeoutMs, &rep);
      sendAll(fd, rep.data(), rep.size(), 5000);
      break;
    } else if (line.compare(0, 7, "MONITOR") == 0) {
      const std::string groups = line.size() > 8 ? line.substr(8) : "all";
      const bool all = groups.find("all") != std::string::npos;
      uint64_t seen;
      { std::lock_guard<std::mutex> g(gRas.lock); seen = gRas.nextEvent - 1; }
      if (!sendAll(fd, "OK\n", 3, 1000)) break;
      // events from now on; the loop ends when the client closes its end (the send fails) or RAS stops
      for (;;) {
        std::vector<std::string> out;
        bool stop;
        {
          std::lock_guard<std::mutex> g(gRas.lock);
          stop = gRas.stop;
          for (auto& e : gRas.events) {
            if (e.first <= seen) continue;
            seen = e.first;
            const size_t sp = e.second.find(' ');
            const std::string grp = e.second.substr(sp + 1, e.second.find(' ', sp + 1) - sp - 1);
            if (all || groups.find(grp) != std::string::npos) out.push_back(e.second);
          }
        }
        bool ok = true;
        for (auto& l : out) ok = ok && sendAll(fd, (l + "\n").data(), l.size() + 1, 1000);
        char c;
        if (!ok || stop || (waitFd(fd, POLLIN, 200) && recv(fd, &c, 1, MSG_DONTWAIT) == 0)) break;
      }
      break;
    } else if (line.empty()) break;
    else { const char* e = "ERROR: unknown command\n"; sendAll(fd, e, strlen(e), 1000); }
  }
  close(fd);
}

void keepAlive() {
  // ping the successor in the address-sorted ring of live processes
  std::string self, nextKey;
  SockAddr next{};
  {
    std::lock_guard<std::mutex> g(gRas.lock);
    self = sockAddrToString(&gRas.peerAddr);
    std::vector<std::string> live;
    for (auto& p : gRas.peers) if (!p.second.dead) live.push_back(p.first);
    if (live.size() < 2) return;
    auto it = std::find(live.begin(), live.end(), self);
    if (it == live.end()) return;
    nextKey = live[(it - live.begin() + 1) % live.size()];
    next = gRas.peers[nextKey].addr;
  }
  std::string r;
  bool ok = ask(next, "PING", &r, scaled(std::max<int64_t>(paramRasKeepAliveMs() / 2, 100))) && r == "PONG";
  bool nowDead = false;
  {
    std::lock_guard<std::mutex> g(gRas.lock);
    PeerProc& p = gRas.peers[nextKey];
    if (ok) p.missed = 0;
    else if (++p.missed >= paramRasDeadAfter()) nowDead = true;
  }
  if (nowDead) markDead(nextKey, true);
}

void rasMain() {
  setThreadName("NCCL RAS");
  uint64_t lastPing = nowNs();
  for (;;) {
    struct pollfd fds[3] = {{gRas.peerFd, POLLIN, 0}, {gRas.clientFd, POLLIN, 0}, {gRas.wakeFd[0], POLLIN, 0}};
    poll(fds, 3, (int)std::min<int64_t>(scaled(paramRasKeepAliveMs()), 1000));
    {
      std::lock_guard<std::mutex> g(gRas.lock);
      if (gRas.stop) return;
    }
    if (fds[0].revents & POLLIN) {
      int fd;
      while ((fd = accept(gRas.peerFd, nullptr, nullptr)) >= 0) servePeer(fd);
    }
    if (gRas.clientFd >= 0 && (fds[1].revents & POLLIN)) {
      int fd;
      while ((fd = accept(gRas.clientFd, nullptr, nullptr)) >= 0) std::thread(serveClient, fd).detach();
    }
    if (fds[2].revents & POLLIN) { char b[16]; (void)!read(gRas.wakeFd[0], b, sizeof(b)); }
    if (nowNs() - lastPing >= (uint64_t)scaled(paramRasKeepAliveMs()) * 1000000ull) {
      lastPing = nowNs();
      keepAlive();
      if (gRas.clientFd < 0) {
        // the process that served the client port may be gone: try to take the port over
        const char* ra = getEnv("NCCL_RAS_ADDR");
        SockAddr ca;
        if (sockAddrFromString(&ca, ra && *ra ? ra : "127.0.0.1:28028") == ncclSuccess) gRas.clientFd = listenOnAddr(&ca);
        if (gRas.clientFd >= 0) INFO(SUB_RAS, "RAS client socket taken over on %s", sockAddrToString(&ca).c_str());
      }
    }
  }
}

void startLocked() {
  if (gRas.started) return;
  SockAddr a;
  char ifname[64];
  if (bootstrapInterface(&a, ifname) != ncclSuccess) return;
  if (a.sa.sa_family == AF_INET) a.sin.sin_port = 0; else a.sin6.sin6_port = 0;
  gRas.peerFd = listenOnAddr(&a);
  if (gRas.peerFd < 0) return;
  gRas.peerAddr = a;
  // client socket: NCCL_RAS_ADDR=host:port, default localhost:28028; only one process per host can own it
  const char* ra = getEnv("NCCL_RAS_ADDR");
  SockAddr ca;
  if (sockAddrFromString(&ca, ra && *ra ? ra : "127.0.0.1:28028") == ncclSuccess) gRas.clientFd = listenOnAddr(&ca);
  if (gRas.clientFd >= 0) INFO(SUB_RAS, "RAS client socket listening on %s", sockAddrToString(&ca).c_str());
  if (pipe(gRas.wakeFd) != 0) { gRas.wakeFd[0] = gRas.wakeFd[1] = -1; }
  gRas.started = true;
  gRas.stop = false;
  gRas.thread = std::thread(rasMain);
  atexit([] { rasShutdown(); });
}

}  // namespace

bool rasListenAddr(SockAddr* out) {
  std::lock_guard<std::mutex> g(gRas.lock);
  startLocked();
  if (!gRas.started) return false;
  *out = gRas.peerAddr;
  return true;
}

void rasCommAdd(ncclComm* comm) {
  std::lock_guard<std::mutex> g(gRas.lock);
  startLocked();
  if (!gRas.started || !comm->bootstrap) return;
  CommRec rec;
  rec.comm = comm;
  rec.hash = comm->commHash;
  rec.rank = comm->rank;
  rec.nRanks = comm->nRanks;
  rec.cudaDev = comm->hostOnly ? -1 : comm->cudaDev;
  const BootstrapRingData* peers = bootstrapPeers(comm->bootstrap);
  for (int r = 0; r < comm->nRanks; ++r) {
    rec.ranks.push_back(peers[r].rasRank);
    const RasRankInit& ri = peers[r].rasRank;
    if (ri.addr.sa.sa_family != AF_INET && ri.addr.sa.sa_family != AF_INET6) continue;
    uint16_t port = ri.addr.sa.sa_family == AF_INET ? ri.addr.sin.sin_port : ri.addr.sin6.sin6_port;
    if (port == 0) continue;   // that rank runs without RAS
    std::string key = sockAddrToString(&ri.addr);
    if (!gRas.peers.count(key)) {
      PeerProc p;
      p.addr = ri.addr;
      p.pid = ri.pid;
      p.hostHash = ri.hostHash;
      gRas.peers[key] = p;
    }
  }
  gRas.comms.push_back(rec);
  char h[32];
  snprintf(h, sizeof(h), "%llx", (unsigned long long)rec.hash);
  eventLocked("lifecycle", std::string("communicator ") + h + " rank " + std::to_string(rec.rank) + " of " + std::to_string(rec.nRanks) + " created");
}

void rasCommRemove(ncclComm* comm) {
  std::lock_guard<std::mutex> g(gRas.lock);
  for (size_t i = 0; i < gRas.comms.size(); ++i)
    if (gRas.comms[i].comm == comm) {
      char h[32];
      snprintf(h, sizeof(h), "%llx", (unsigned long long)gRas.comms[i].hash);
      eventLocked("lifecycle", std::string("communicator ") + h + " rank " + std::to_string(gRas.comms[i].rank) + " destroyed");
      gRas.comms.erase(gRas.comms.begin() + i);
      break;
    }
}

void rasShutdown() {
  {
    std::lock_guard<std::mutex> g(gRas.lock);
    if (!gRas.started) return;
    gRas.stop = true;
    if (gRas.wakeFd[1] >= 0) (void)!write(gRas.wakeFd[1], "x", 1);
  }
  if (gRas.thread.joinable()) gRas.thread.join();
  std::lock_guard<std::mutex> g(gRas.lock);
  for (int* fd : {&gRas.peerFd, &gRas.clientFd, &gRas.wakeFd[0], &gRas.wakeFd[1]}) {
    if (*fd >= 0) close(*fd);
    *fd = -1;
  }
  gRas.started = false;
  gRas.comms.clear();
  gRas.peers.clear();
}

}  // namespace b200
