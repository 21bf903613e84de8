// TCP socket layer used by bootstrap, proxy, RAS and the socket network backend.
// Wire behaviour matches the reference so that either side of a connection may be the
// reference library: a connector first sends the 8-byte magic of the listening socket
// and a 4-byte socket type; an acceptor drops connections whose magic or type differ
// (reference: src/misc/socket.cc:327-421, src/include/socket.h:40-80).
#pragma once
#include <arpa/inet.h>
#include <netinet/in.h>
#include <sys/socket.h>

#include "core.h"

namespace b200 {

constexpr uint64_t kSocketMagic = 0x564ab9f2fc4b9d6cULL;

union SockAddr {
  struct sockaddr sa;
  struct sockaddr_in sin;
  struct sockaddr_in6 sin6;
};
static_assert(sizeof(SockAddr) == 28, "socket address is 28 bytes on the wire");

enum SockType : int { SOCK_UNKNOWN = 0, SOCK_BOOTSTRAP = 1, SOCK_PROXY = 2, SOCK_NET = 3, SOCK_NETIB = 4, SOCK_RAS = 5 };

struct Socket {
  int fd = -1;
  SockAddr addr{};
  uint64_t magic = kSocketMagic;
  int type = SOCK_UNKNOWN;
  volatile uint32_t* abortFlag = nullptr;
  bool ready = false;
};

enum SockOpKind { SOCK_OP_SEND = 0, SOCK_OP_RECV = 1 };
struct SockOp {
  SockOpKind kind;
  Socket* sock;
  void* data;
  int size;
  int done;
};

std::string sockAddrToString(const SockAddr* a);
ncclResult_t sockAddrFromString(SockAddr* a, const char* ipPort);  // "1.2.3.4:567" or "[::1]:567"
int sockAddrLen(const SockAddr* a);

// Picks up to maxIfs interfaces following NCCL_SOCKET_IFNAME / NCCL_SOCKET_FAMILY and the default
// preference order ib* > (subnet of NCCL_COMM_ID) > others > docker* > lo > virbr*.
int findInterfaces(char names[][64], SockAddr* addrs, int maxIfs);
ncclResult_t bootstrapInterface(SockAddr* addr, char* nameOut /* 64 */);

ncclResult_t sockInit(Socket* s, const SockAddr* addr, uint64_t magic, SockType type,
                      volatile uint32_t* abortFlag = nullptr);
ncclResult_t sockListen(Socket* s);            // binds addr (port 0 -> ephemeral), fills s->addr with the bound address
ncclResult_t sockConnect(Socket* s);           // blocking with refused/timeout retries, then handshake
ncclResult_t sockAccept(Socket* s, Socket* listenSock);  // loops until a peer with the right magic+type arrives
ncclResult_t sockSend(Socket* s, const void* p, int n);
ncclResult_t sockRecv(Socket* s, void* p, int n);
ncclResult_t sockTryRecv(Socket* s, void* p, int n, int* closed, bool blocking);
ncclResult_t sockSendRecv(Socket* sendSock, const void* sp, int sn, Socket* recvSock, void* rp, int rn);
// One non-blocking attempt: moves what the kernel accepts right now and advances *off (never waits).
ncclResult_t sockProgress(SockOpKind kind, Socket* s, void* p, int n, int* off);
ncclResult_t sockMultiOp(SockOp* ops, int n);  // progresses all ops concurrently until all complete
ncclResult_t sockClose(Socket* s, bool waitPeer = false);
ncclResult_t sockShutdown(Socket* s);

}  // namespace b200
