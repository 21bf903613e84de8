// File-descriptor passing over abstract Unix-domain datagram sockets.
// Reference parity: src/os/linux_ipcsocket.cc (ncclIpcSocketInit/SendFd/RecvFd).
#include "ipcsocket.h"

#include <errno.h>
#include <poll.h>
#include <stdio.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

namespace b200 {

static socklen_t makeName(struct sockaddr_un* sa, uint64_t id) {
  memset(sa, 0, sizeof(*sa));
  sa->sun_family = AF_UNIX;
  // abstract namespace: first byte of sun_path is NUL, nothing appears in the file system
  int n = snprintf(sa->sun_path + 1, sizeof(sa->sun_path) - 1, "b200-ipc-%016llx", (unsigned long long)id);
  return (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + n);
}

ncclResult_t ipcOpen(IpcSocket* s, uint64_t id) {
  int fd = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (fd < 0) { WARN("UDS: socket() failed: %s", strerror(errno)); return ncclSystemError; }
  struct sockaddr_un sa;
  socklen_t len = makeName(&sa, id);
  if (bind(fd, (struct sockaddr*)&sa, len) != 0) {
    WARN("UDS: bind failed: %s", strerror(errno));
    close(fd);
    return ncclSystemError;
  }
  s->fd = fd;
  s->id = id;
  return ncclSuccess;
}

ncclResult_t ipcSendFd(IpcSocket* s, uint64_t peerId, int sendFd, const IpcMsg& msg) {
  struct sockaddr_un sa;
  socklen_t len = makeName(&sa, peerId);
  struct msghdr mh;
  memset(&mh, 0, sizeof(mh));
  struct iovec iov;
  IpcMsg copy = msg;
  iov.iov_base = &copy;
  iov.iov_len = sizeof(copy);
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  mh.msg_name = &sa;
  mh.msg_namelen = len;
  union { struct cmsghdr h; char buf[CMSG_SPACE(sizeof(int))]; } ctl;
  if (sendFd >= 0) {
    memset(&ctl, 0, sizeof(ctl));
    mh.msg_control = ctl.buf;
    mh.msg_controllen = sizeof(ctl.buf);
    struct cmsghdr* c = CMSG_FIRSTHDR(&mh);
    c->cmsg_len = CMSG_LEN(sizeof(int));
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    memcpy(CMSG_DATA(c), &sendFd, sizeof(int));
  }
  for (int attempt = 0;; ++attempt) {
    ssize_t r = sendmsg(s->fd, &mh, 0);
    if (r >= 0) return ncclSuccess;
    // the peer may not have bound its socket yet, or its queue is full: retry for a while
    if ((errno == ECONNREFUSED || errno == ENOENT || errno == EAGAIN || errno == EINTR || errno == ENOBUFS) && attempt < 3000) {
      usleep(1000);
      continue;
    }
    WARN("UDS: sendmsg failed: %s", strerror(errno));
    return ncclSystemError;
  }
}

ncclResult_t ipcRecvFd(IpcSocket* s, int* recvFd, IpcMsg* msg, volatile uint32_t* abortFlag, int timeoutMs) {
  *recvFd = -1;
  int waited = 0;
  for (;;) {
    struct pollfd p{s->fd, POLLIN, 0};
    int rc = poll(&p, 1, 50);
    if (rc > 0) break;
    if (abortFlag && __atomic_load_n((const uint32_t*)abortFlag, __ATOMIC_ACQUIRE)) return ncclInternalError;
    waited += 50;
    if (timeoutMs > 0 && waited >= timeoutMs) { WARN("UDS: timed out waiting for a descriptor"); return ncclTimeout; }
  }
  struct msghdr mh;
  memset(&mh, 0, sizeof(mh));
  struct iovec iov;
  iov.iov_base = msg;
  iov.iov_len = sizeof(*msg);
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  union { struct cmsghdr h; char buf[CMSG_SPACE(sizeof(int))]; } ctl;
  mh.msg_control = ctl.buf;
  mh.msg_controllen = sizeof(ctl.buf);
  ssize_t r;
  do { r = recvmsg(s->fd, &mh, MSG_CMSG_CLOEXEC); } while (r < 0 && errno == EINTR);
  if (r != (ssize_t)sizeof(*msg)) { WARN("UDS: short datagram (%zd bytes)", r); return ncclSystemError; }
  for (struct cmsghdr* c = CMSG_FIRSTHDR(&mh); c; c = CMSG_NXTHDR(&mh, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) memcpy(recvFd, CMSG_DATA(c), sizeof(int));
  }
  return ncclSuccess;
}

void ipcClose(IpcSocket* s) {
  if (s->fd >= 0) close(s->fd);
  s->fd = -1;
}

}  // namespace b200
