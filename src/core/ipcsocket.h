// Unix-domain datagram sockets that carry file descriptors (SCM_RIGHTS) between the ranks of one
// host: the way POSIX-fd handles of cuMem allocations and multicast objects reach their peers.
// Reference parity: src/os/linux_ipcsocket.cc, src/include/ipcsocket.h.
#pragma once
#include "core.h"

namespace b200 {

struct IpcSocket {
  int fd = -1;
  uint64_t id = 0;
};

struct IpcMsg {
  int srcRank;
  int tag;
  uint64_t a, b;   // free-form payload (sizes, offsets)
};

ncclResult_t ipcOpen(IpcSocket* s, uint64_t id);   // binds the abstract name derived from id
ncclResult_t ipcSendFd(IpcSocket* s, uint64_t peerId, int fd, const IpcMsg& msg);
// Receives one datagram; *fd is -1 when it carried no descriptor.
ncclResult_t ipcRecvFd(IpcSocket* s, int* fd, IpcMsg* msg, volatile uint32_t* abortFlag, int timeoutMs);
void ipcClose(IpcSocket* s);

}  // namespace b200
