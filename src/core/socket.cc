// TCP socket layer. See socket.h for the wire contract.
// Reference parity: src/misc/socket.cc (retry policy :19-23, listen backlog :148,
// interface search order :190-232, handshake :327-421, send/recv helpers :622-722).
#include "socket.h"

#include <errno.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netdb.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdio.h>
#include <unistd.h>

namespace b200 {

B200_PARAM(SocketRetryCnt, "SOCKET_RETRY_CNT", 34, "Connection attempts before giving up")
B200_PARAM(SocketRetrySleepMsec, "SOCKET_RETRY_SLEEP_MSEC", 100, "Base sleep between connection attempts (ms)")
B200_PARAM(SocketTimeoutMs, "B200_SOCKET_TIMEOUT_MS", 0,
           "Give up on a socket send/recv/accept that makes no progress for this long (0 = wait forever)")

std::string sockAddrToString(const SockAddr* a) {
  char host[NI_MAXHOST] = "?", serv[NI_MAXSERV] = "?";
  if (a->sa.sa_family != AF_INET && a->sa.sa_family != AF_INET6) return "<unset>";
  getnameinfo(&a->sa, sockAddrLen(a), host, sizeof(host), serv, sizeof(serv), NI_NUMERICHOST | NI_NUMERICSERV);
  return std::string(host) + "<" + serv + ">";
}

int sockAddrLen(const SockAddr* a) {
  return a->sa.sa_family == AF_INET6 ? sizeof(struct sockaddr_in6) : sizeof(struct sockaddr_in);
}

ncclResult_t sockAddrFromString(SockAddr* a, const char* ipPort) {
  memset(a, 0, sizeof(*a));
  std::string s(ipPort);
  std::string host, port;
  if (!s.empty() && s[0] == '[') {
    size_t close = s.find(']');
    if (close == std::string::npos) return ncclInvalidArgument;
    host = s.substr(1, close - 1);
    if (close + 2 <= s.size() && s[close + 1] == ':') port = s.substr(close + 2);
  } else {
    size_t colon = s.rfind(':');
    if (colon == std::string::npos) return ncclInvalidArgument;
    host = s.substr(0, colon);
    port = s.substr(colon + 1);
  }
  struct addrinfo hints, *res = nullptr;
  memset(&hints, 0, sizeof(hints));
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(host.c_str(), port.empty() ? nullptr : port.c_str(), &hints, &res) != 0 || !res) {
    WARN("Could not resolve address %s", ipPort);
    return ncclInvalidArgument;
  }
  memcpy(a, res->ai_addr, res->ai_addrlen);
  freeaddrinfo(res);
  return ncclSuccess;
}

static bool matchPrefixList(const char* name, const char* list, bool exact) {
  std::string l(list);
  size_t pos = 0;
  while (pos <= l.size()) {
    size_t c = l.find(',', pos);
    std::string tok = l.substr(pos, c == std::string::npos ? std::string::npos : c - pos);
    if (!tok.empty()) {
      if (exact ? tok == name : strncmp(name, tok.c_str(), tok.size()) == 0) return true;
    }
    if (c == std::string::npos) break;
    pos = c + 1;
  }
  return false;
}

static bool sameSubnet(const struct ifaddrs* ifa, const SockAddr* remote) {
  if (ifa->ifa_addr->sa_family != remote->sa.sa_family || !ifa->ifa_netmask) return false;
  if (remote->sa.sa_family == AF_INET) {
    uint32_t m = ((struct sockaddr_in*)ifa->ifa_netmask)->sin_addr.s_addr;
    return ((((struct sockaddr_in*)ifa->ifa_addr)->sin_addr.s_addr ^ remote->sin.sin_addr.s_addr) & m) == 0;
  }
  const uint8_t* a = ((struct sockaddr_in6*)ifa->ifa_addr)->sin6_addr.s6_addr;
  const uint8_t* m = ((struct sockaddr_in6*)ifa->ifa_netmask)->sin6_addr.s6_addr;
  const uint8_t* r = remote->sin6.sin6_addr.s6_addr;
  for (int i = 0; i < 16; ++i) if ((a[i] ^ r[i]) & m[i]) return false;
  return true;
}

// One pass over the interface list keeping those accepted by `pred`.
template <typename Pred>
static int collectIfs(struct ifaddrs* list, int family, char names[][64], SockAddr* addrs, int maxIfs, Pred pred) {
  int found = 0;
  for (struct ifaddrs* i = list; i && found < maxIfs; i = i->ifa_next) {
    if (!i->ifa_addr) continue;
    int fam = i->ifa_addr->sa_family;
    if (fam != AF_INET && fam != AF_INET6) continue;
    if (family != -1 && fam != family) continue;
    if (!(i->ifa_flags & IFF_UP)) continue;
    if (fam == AF_INET6) {
      const struct sockaddr_in6* s6 = (const struct sockaddr_in6*)i->ifa_addr;
      if (IN6_IS_ADDR_LOOPBACK(&s6->sin6_addr) && strncmp(i->ifa_name, "lo", 2) != 0) continue;
    }
    if (!pred(i)) continue;
    bool dup = false;
    for (int k = 0; k < found; ++k) if (!strcmp(names[k], i->ifa_name)) dup = true;
    if (dup) continue;
    snprintf(names[found], 64, "%s", i->ifa_name);
    memset(&addrs[found], 0, sizeof(SockAddr));
    memcpy(&addrs[found], i->ifa_addr, fam == AF_INET ? sizeof(struct sockaddr_in) : sizeof(struct sockaddr_in6));
    ++found;
  }
  return found;
}

int findInterfaces(char names[][64], SockAddr* addrs, int maxIfs) {
  struct ifaddrs* list = nullptr;
  if (getifaddrs(&list) != 0) return 0;
  int family = -1;
  const char* fam = getEnv("NCCL_SOCKET_FAMILY");
  if (fam) family = !strcmp(fam, "AF_INET") ? AF_INET : (!strcmp(fam, "AF_INET6") ? AF_INET6 : -1);
  int n = 0;
  const char* user = getEnv("NCCL_SOCKET_IFNAME");
  if (user && *user) {
    bool exclude = user[0] == '^';
    if (exclude) ++user;
    bool exact = user[0] == '=';
    if (exact) ++user;
    n = collectIfs(list, family, names, addrs, maxIfs, [&](struct ifaddrs* i) {
      return matchPrefixList(i->ifa_name, user, exact) != exclude;
    });
  } else {
    n = collectIfs(list, family, names, addrs, maxIfs, [](struct ifaddrs* i) { return !strncmp(i->ifa_name, "ib", 2); });
    const char* commId = getEnv("NCCL_COMM_ID");
    if (n == 0 && commId && *commId) {
      SockAddr remote;
      if (sockAddrFromString(&remote, commId) == ncclSuccess)
        n = collectIfs(list, family, names, addrs, maxIfs, [&](struct ifaddrs* i) { return sameSubnet(i, &remote); });
    }
    auto special = [](const char* nm) {
      return !strncmp(nm, "docker", 6) || !strncmp(nm, "lo", 2) || !strncmp(nm, "virbr", 5);
    };
    if (n == 0) n = collectIfs(list, family, names, addrs, maxIfs, [&](struct ifaddrs* i) { return !special(i->ifa_name); });
    if (n == 0) n = collectIfs(list, family, names, addrs, maxIfs, [](struct ifaddrs* i) { return !strncmp(i->ifa_name, "docker", 6); });
    if (n == 0) n = collectIfs(list, family, names, addrs, maxIfs, [](struct ifaddrs* i) { return !strncmp(i->ifa_name, "lo", 2); });
    if (n == 0) n = collectIfs(list, family, names, addrs, maxIfs, [](struct ifaddrs* i) { return !strncmp(i->ifa_name, "virbr", 5); });
  }
  freeifaddrs(list);
  return n;
}

ncclResult_t bootstrapInterface(SockAddr* addr, char* nameOut) {
  char names[1][64];
  SockAddr addrs[1];
  if (findInterfaces(names, addrs, 1) < 1) {
    WARN("Bootstrap: no socket interface found");
    return ncclSystemError;
  }
  *addr = addrs[0];
  if (nameOut) snprintf(nameOut, 64, "%s", names[0]);
  return ncclSuccess;
}

ncclResult_t sockInit(Socket* s, const SockAddr* addr, uint64_t magic, SockType type, volatile uint32_t* abortFlag) {
  s->fd = -1;
  memset(&s->addr, 0, sizeof(s->addr));
  if (addr) s->addr = *addr;
  s->magic = magic;
  s->type = type;
  s->abortFlag = abortFlag;
  s->ready = false;
  return ncclSuccess;
}

B200_PARAM(SocketRcvBuf, "SOCKET_RCVBUF", -1, "Receive buffer of every TCP socket in bytes (-1: the system's default)")
B200_PARAM(SocketSndBuf, "SOCKET_SNDBUF", -1, "Send buffer of every TCP socket in bytes (-1: the system's default)")

static void setFdOptions(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  if (paramSocketRcvBuf() > 0) { int v = (int)paramSocketRcvBuf(); setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &v, sizeof(v)); }
  if (paramSocketSndBuf() > 0) { int v = (int)paramSocketSndBuf(); setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &v, sizeof(v)); }
  int fl = fcntl(fd, F_GETFL);
  fcntl(fd, F_SETFL, fl | O_NONBLOCK);
  fcntl(fd, F_SETFD, FD_CLOEXEC);
}

ncclResult_t sockListen(Socket* s) {
  int fam = s->addr.sa.sa_family;
  if (fam != AF_INET && fam != AF_INET6) {
    WARN("sockListen: address family not set");
    return ncclInvalidArgument;
  }
  int fd = socket(fam, SOCK_STREAM, 0);
  if (fd < 0) { WARN("socket() failed: %s", strerror(errno)); return ncclSystemError; }
  int one = 1;
  // A fixed port (NCCL_COMM_ID root) may be re-used right after a previous job.
  uint16_t port = fam == AF_INET ? s->addr.sin.sin_port : s->addr.sin6.sin6_port;
  if (port) setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  if (bind(fd, &s->addr.sa, sockAddrLen(&s->addr)) != 0) {
    WARN("bind(%s) failed: %s", sockAddrToString(&s->addr).c_str(), strerror(errno));
    close(fd);
    return ncclSystemError;
  }
  socklen_t len = sockAddrLen(&s->addr);
  getsockname(fd, &s->addr.sa, &len);
  if (listen(fd, 16384) != 0) {
    WARN("listen() failed: %s", strerror(errno));
    close(fd);
    return ncclSystemError;
  }
  int fl = fcntl(fd, F_GETFL);
  fcntl(fd, F_SETFL, fl | O_NONBLOCK);
  fcntl(fd, F_SETFD, FD_CLOEXEC);
  s->fd = fd;
  s->ready = true;
  return ncclSuccess;
}

static inline bool aborted(Socket* s) { return s->abortFlag && __atomic_load_n(s->abortFlag, __ATOMIC_RELAXED); }

// Moves up to n bytes; *off advances. Returns ncclRemoteError when the peer closed.
static ncclResult_t progressOnce(SockOpKind kind, Socket* s, void* p, int n, int* off, int* closed) {
  if (closed) *closed = 0;
  while (*off < n) {
    ssize_t r = kind == SOCK_OP_SEND ? send(s->fd, (char*)p + *off, n - *off, MSG_NOSIGNAL | MSG_DONTWAIT)
                                     : recv(s->fd, (char*)p + *off, n - *off, MSG_DONTWAIT);
    if (r > 0) { *off += (int)r; continue; }
    if (r == 0 && kind == SOCK_OP_RECV) {
      if (closed) { *closed = 1; return ncclSuccess; }
      INFO(SUB_NET, "socket: peer %s closed the connection", sockAddrToString(&s->addr).c_str());
      return ncclRemoteError;
    }
    if (r < 0 && (errno == EINTR)) continue;
    if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) return ncclSuccess;
    if (r < 0 && (errno == ECONNRESET || errno == EPIPE)) {
      if (closed) { *closed = 1; return ncclSuccess; }
      INFO(SUB_NET, "socket: connection to %s lost: %s", sockAddrToString(&s->addr).c_str(), strerror(errno));
      return ncclRemoteError;
    }
    WARN("socket %s failed: %s", kind == SOCK_OP_SEND ? "send" : "recv", strerror(errno));
    return ncclSystemError;
  }
  return ncclSuccess;
}

ncclResult_t sockProgress(SockOpKind kind, Socket* s, void* p, int n, int* off) { return progressOnce(kind, s, p, n, off, nullptr); }

static ncclResult_t waitAll(SockOp* ops, int n) {
  uint64_t lastProgress = nowNs();
  int64_t timeoutMs = paramSocketTimeoutMs();
  for (;;) {
    bool all = true;
    int before = 0, after = 0;
    std::vector<struct pollfd> pfd;
    for (int i = 0; i < n; ++i) {
      before += ops[i].done;
      if (ops[i].done < ops[i].size) NCCLCHECK(progressOnce(ops[i].kind, ops[i].sock, ops[i].data, ops[i].size, &ops[i].done, nullptr));
      after += ops[i].done;
      if (ops[i].done < ops[i].size) {
        all = false;
        pfd.push_back({ops[i].sock->fd, (short)(ops[i].kind == SOCK_OP_SEND ? POLLOUT : POLLIN), 0});
      }
    }
    if (all) return ncclSuccess;
    if (after != before) lastProgress = nowNs();
    for (int i = 0; i < n; ++i) if (aborted(ops[i].sock)) return ncclInternalError;
    if (timeoutMs > 0 && (nowNs() - lastProgress) / 1000000 > (uint64_t)timeoutMs) {
      WARN("socket: no progress for %lld ms, giving up", (long long)timeoutMs);
      return ncclTimeout;
    }
    poll(pfd.data(), pfd.size(), 50);
  }
}

ncclResult_t sockSend(Socket* s, const void* p, int n) {
  SockOp op{SOCK_OP_SEND, s, (void*)p, n, 0};
  return waitAll(&op, 1);
}
ncclResult_t sockRecv(Socket* s, void* p, int n) {
  SockOp op{SOCK_OP_RECV, s, p, n, 0};
  return waitAll(&op, 1);
}
ncclResult_t sockTryRecv(Socket* s, void* p, int n, int* closed, bool blocking) {
  int off = 0;
  *closed = 0;
  NCCLCHECK(progressOnce(SOCK_OP_RECV, s, p, n, &off, closed));
  if (*closed) return ncclSuccess;
  if (off == 0 && !blocking) return ncclInProgress;
  if (off < n) {
    SockOp op{SOCK_OP_RECV, s, p, n, off};
    return waitAll(&op, 1);
  }
  return ncclSuccess;
}
ncclResult_t sockSendRecv(Socket* ss, const void* sp, int sn, Socket* rs, void* rp, int rn) {
  SockOp ops[2] = {{SOCK_OP_SEND, ss, (void*)sp, sn, 0}, {SOCK_OP_RECV, rs, rp, rn, 0}};
  return waitAll(ops, 2);
}
ncclResult_t sockMultiOp(SockOp* ops, int n) {
  for (int i = 0; i < n; ++i) ops[i].done = 0;
  return waitAll(ops, n);
}

ncclResult_t sockConnect(Socket* s) {
  int retries = 0;
  const int maxRetries = (int)paramSocketRetryCnt();
  const int sleepMs = (int)paramSocketRetrySleepMsec();
  for (;;) {
    if (aborted(s)) return ncclInternalError;
    int fd = socket(s->addr.sa.sa_family, SOCK_STREAM, 0);
    if (fd < 0) { WARN("socket() failed: %s", strerror(errno)); return ncclSystemError; }
    int rc;
    do { rc = connect(fd, &s->addr.sa, sockAddrLen(&s->addr)); } while (rc != 0 && errno == EINTR);
    if (rc == 0) {
      setFdOptions(fd);
      s->fd = fd;
      break;
    }
    int err = errno;
    close(fd);
    if ((err == ECONNREFUSED || err == ETIMEDOUT || err == EHOSTUNREACH || err == EAGAIN) && ++retries <= maxRetries) {
      if (retries % 8 == 0) INFO(SUB_NET, "connect to %s: %s, retrying (%d/%d)", sockAddrToString(&s->addr).c_str(), strerror(err), retries, maxRetries);
      usleep((useconds_t)sleepMs * 1000 * (retries < 10 ? retries : 10));
      continue;
    }
    WARN("connect to %s failed: %s", sockAddrToString(&s->addr).c_str(), strerror(err));
    return err == ECONNREFUSED ? ncclRemoteError : ncclSystemError;
  }
  NCCLCHECK(sockSend(s, &s->magic, sizeof(s->magic)));
  int type = s->type;
  NCCLCHECK(sockSend(s, &type, sizeof(type)));
  s->ready = true;
  return ncclSuccess;
}

ncclResult_t sockAccept(Socket* s, Socket* l) {
  uint64_t start = nowNs();
  int64_t timeoutMs = paramSocketTimeoutMs();
  for (;;) {
    if (aborted(l)) return ncclInternalError;
    struct pollfd pfd{l->fd, POLLIN, 0};
    int rc = poll(&pfd, 1, 50);
    if (rc <= 0) {
      if (timeoutMs > 0 && (nowNs() - start) / 1000000 > (uint64_t)timeoutMs) {
        WARN("socket: accept timed out after %lld ms", (long long)timeoutMs);
        return ncclTimeout;
      }
      continue;
    }
    socklen_t len = sizeof(SockAddr);
    SockAddr peer{};
    int fd = accept(l->fd, &peer.sa, &len);
    if (fd < 0) {
      if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR || errno == ECONNABORTED) continue;
      WARN("accept() failed: %s", strerror(errno));
      return ncclSystemError;
    }
    setFdOptions(fd);
    Socket cand;
    cand.fd = fd;
    cand.addr = peer;
    cand.magic = l->magic;
    cand.type = l->type;
    cand.abortFlag = l->abortFlag;
    // Handshake: wrong magic or type means a stray or stale peer; drop it and keep listening.
    uint64_t magic = 0;
    int type = -1;
    int closed = 0;
    ncclResult_t r = sockTryRecv(&cand, &magic, sizeof(magic), &closed, true);
    if (r != ncclSuccess || closed || magic != l->magic) {
      INFO(SUB_NET, "accept: dropping connection from %s (bad magic)", sockAddrToString(&peer).c_str());
      close(fd);
      if (r == ncclInternalError) return r;  // aborted
      continue;
    }
    r = sockTryRecv(&cand, &type, sizeof(type), &closed, true);
    if (r != ncclSuccess || closed || type != l->type) {
      INFO(SUB_NET, "accept: dropping connection from %s (socket type %d, expected %d)", sockAddrToString(&peer).c_str(), type, l->type);
      close(fd);
      if (r == ncclInternalError) return r;
      continue;
    }
    *s = cand;
    s->ready = true;
    return ncclSuccess;
  }
}

ncclResult_t sockShutdown(Socket* s) {
  if (s->fd >= 0) shutdown(s->fd, SHUT_RDWR);
  return ncclSuccess;
}

ncclResult_t sockClose(Socket* s, bool waitPeer) {
  if (s->fd >= 0) {
    if (waitPeer) {
      // Receiver side of a one-shot message: wait for the sender's FIN so that the
      // sender never sees a reset while its last bytes are in flight.
      shutdown(s->fd, SHUT_WR);
      char tmp;
      uint64_t start = nowNs();
      for (;;) {
        ssize_t r = recv(s->fd, &tmp, 1, MSG_DONTWAIT);
        if (r == 0) break;
        if (r < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) break;
        if (aborted(s) || nowNs() - start > 2000000000ull) break;
        struct pollfd pfd{s->fd, POLLIN, 0};
        poll(&pfd, 1, 20);
      }
    }
    close(s->fd);
  }
  s->fd = -1;
  s->ready = false;
  return ncclSuccess;
}

}  // namespace b200
