// Example collective-network plugin: exports ncclCollNetPlugin_v12 only. Rank 0 of a group plays the
// part of the switch: every rank sends its contribution over a Unix-domain socket, rank 0 reduces
// (or concatenates) and sends the results back. Host memory, one host: it exists to exercise the
// library's collective-network path end to end, as the reference's ext-net examples do for the
// point-to-point interface (ext-net/example).
// Build: part of `make plugins`; use with NCCL_NET_PLUGIN=<path>/star_collnet.so NCCL_COLLNET_ENABLE=1.
// STAR_COLLNET_LOG=<file prefix> makes every rank append one line per collective to <prefix>.<pid>.
#include <errno.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <vector>

#include "plugin/nccl_net.h"

namespace {

ncclDebugLogger_t gLog = nullptr;
std::atomic<int> gSerial{0};

struct Listen { int fd; };
struct Group {
  int nranks, rank;
  std::vector<int> fds;   // rank 0: fds[r] to rank r; other ranks: fds[0] to rank 0
};
struct Request { int size; };

bool sendAll(int fd, const void* p, size_t n) {
  const char* c = (const char*)p;
  while (n) {
    ssize_t k = ::send(fd, c, n, MSG_NOSIGNAL);
    if (k < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    if (k <= 0) return false;
    c += k; n -= (size_t)k;
  }
  return true;
}
bool recvAll(int fd, void* p, size_t n) {
  char* c = (char*)p;
  while (n) {
    ssize_t k = ::recv(fd, c, n, 0);
    if (k < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    if (k <= 0) return false;
    c += k; n -= (size_t)k;
  }
  return true;
}

void note(const char* what, size_t bytes) {
  const char* prefix = getenv("STAR_COLLNET_LOG");
  if (!prefix) return;
  char path[512];
  snprintf(path, sizeof(path), "%s.%d", prefix, (int)getpid());
  if (FILE* f = fopen(path, "a")) { fprintf(f, "%s %zu\n", what, bytes); fclose(f); }
}

template <typename T>
void reduceT(T* acc, const T* in, size_t n, ncclRedOp_t op) {
  for (size_t i = 0; i < n; ++i) {
    switch (op) {
      case ncclSum: acc[i] = acc[i] + in[i]; break;
      case ncclProd: acc[i] = acc[i] * in[i]; break;
      case ncclMax: acc[i] = in[i] > acc[i] ? in[i] : acc[i]; break;
      default: acc[i] = in[i] < acc[i] ? in[i] : acc[i]; break;
    }
  }
}
size_t sizeOf(ncclDataType_t t) { return (t == ncclFloat64 || t == ncclInt64 || t == ncclUint64) ? 8 : 4; }
void reduceInto(void* acc, const void* in, size_t n, ncclDataType_t t, ncclRedOp_t op) {
  switch (t) {
    case ncclFloat32: reduceT((float*)acc, (const float*)in, n, op); break;
    case ncclFloat64: reduceT((double*)acc, (const double*)in, n, op); break;
    case ncclInt32: reduceT((int32_t*)acc, (const int32_t*)in, n, op); break;
    case ncclUint32: reduceT((uint32_t*)acc, (const uint32_t*)in, n, op); break;
    case ncclInt64: reduceT((int64_t*)acc, (const int64_t*)in, n, op); break;
    default: reduceT((uint64_t*)acc, (const uint64_t*)in, n, op); break;
  }
}

// ---- interface functions
ncclResult_t starInit(void** ctx, uint64_t, ncclDebugLogger_t logFunction) {
  gLog = logFunction;
  *ctx = new int(0);
  return ncclSuccess;
}
ncclResult_t starDevices(int* ndev) { *ndev = 1; return ncclSuccess; }
ncclResult_t starProps(int, ncclNetProperties_t* p) {
  memset(p, 0, sizeof(*p));
  static char name[] = "star0";
  p->name = name;
  p->ptrSupport = NCCL_PTR_HOST;
  p->speed = 100000;
  p->latency = 1.0f;
  p->maxComms = 1024;
  p->maxRecvs = 1;
  p->maxCollBytes = (size_t)1 << 30;
  return ncclSuccess;
}
ncclResult_t starListen(void*, int, void* handle, void** listenComm) {
  int fd = socket(AF_UNIX, SOCK_STREAM, 0);
  if (fd < 0) return ncclSystemError;
  sockaddr_un a;
  memset(&a, 0, sizeof(a));
  a.sun_family = AF_UNIX;
  // abstract name (leading NUL): nothing to unlink
  int len = snprintf(a.sun_path + 1, sizeof(a.sun_path) - 1, "nccl-b200-star-%d-%d", (int)getpid(), gSerial++);
  socklen_t alen = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + len);
  if (bind(fd, (sockaddr*)&a, alen) != 0 || listen(fd, 64) != 0) { close(fd); return ncclSystemError; }
  memset(handle, 0, NCCL_NET_HANDLE_MAXSIZE);
  memcpy(handle, a.sun_path + 1, (size_t)len + 1);
  *listenComm = new Listen{fd};
  return ncclSuccess;
}
ncclResult_t starConnect(void* handles[], int nranks, int rank, void* listenComm, void** collComm) {
  Group* g = new Group;
  g->nranks = nranks;
  g->rank = rank;
  if (rank == 0) {
    g->fds.assign(nranks, -1);
    for (int i = 1; i < nranks; ++i) {
      int fd = accept(((Listen*)listenComm)->fd, nullptr, nullptr);
      int32_t who = -1;
      if (fd < 0 || !recvAll(fd, &who, sizeof(who)) || who <= 0 || who >= nranks) { delete g; return ncclSystemError; }
      g->fds[who] = fd;
    }
  } else {
    int fd = socket(AF_UNIX, SOCK_STREAM, 0);
    sockaddr_un a;
    memset(&a, 0, sizeof(a));
    a.sun_family = AF_UNIX;
    size_t len = strlen((const char*)handles[0]);
    memcpy(a.sun_path + 1, handles[0], len);
    socklen_t alen = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + len);
    int32_t who = rank;
    if (fd < 0 || connect(fd, (sockaddr*)&a, alen) != 0 || !sendAll(fd, &who, sizeof(who))) { if (fd >= 0) close(fd); delete g; return ncclSystemError; }
    g->fds.assign(1, fd);
  }
  *collComm = g;
  return ncclSuccess;
}
ncclResult_t starReduceSupport(ncclDataType_t t, ncclRedOp_t op, int* supported) {
  bool typeOk = t == ncclFloat32 || t == ncclFloat64 || t == ncclInt32 || t == ncclUint32 || t == ncclInt64 || t == ncclUint64;
  *supported = typeOk && (op == ncclSum || op == ncclProd || op == ncclMax || op == ncclMin);
  return ncclSuccess;
}
ncclResult_t starRegMr(void*, void* data, size_t, int type, void** mhandle) {
  if (type != NCCL_PTR_HOST) return ncclInvalidUsage;
  *mhandle = data;
  return ncclSuccess;
}
ncclResult_t starRegMrDmaBuf(void*, void*, size_t, int, uint64_t, int, void**) { return ncclInvalidUsage; }
ncclResult_t starDeregMr(void*, void*) { return ncclSuccess; }

// The switch (rank 0) collects `bytes` from every rank into `all` ([nranks][bytes], own part copied).
bool collect(Group* g, const void* mine, size_t bytes, std::vector<char>* all) {
  all->resize(bytes * g->nranks);
  memcpy(all->data(), mine, bytes);
  for (int r = 1; r < g->nranks; ++r)
    if (!recvAll(g->fds[r], all->data() + (size_t)r * bytes, bytes)) return false;
  return true;
}

ncclResult_t starAllReduce(void* collComm, void* sendData, void* recvData, size_t count, ncclDataType_t type, ncclRedOp_t op, void*, void*, void** request) {
  Group* g = (Group*)collComm;
  const size_t bytes = count * sizeOf(type);
  if (g->rank == 0) {
    std::vector<char> all;
    if (!collect(g, sendData, bytes, &all)) return ncclSystemError;
    for (int r = 1; r < g->nranks; ++r) reduceInto(all.data(), all.data() + (size_t)r * bytes, count, type, op);   // rank order
    memcpy(recvData, all.data(), bytes);
    for (int r = 1; r < g->nranks; ++r) if (!sendAll(g->fds[r], recvData, bytes)) return ncclSystemError;
  } else {
    if (!sendAll(g->fds[0], sendData, bytes) || !recvAll(g->fds[0], recvData, bytes)) return ncclSystemError;
  }
  note("allreduce", bytes);
  *request = new Request{(int)bytes};
  return ncclSuccess;
}
ncclResult_t starAllGather(void* collComm, void* sendData, int nRecvParts, ncclNetSGE_v12_t* recvParts, size_t bytesPerRank, size_t, size_t, void*, void** request) {
  Group* g = (Group*)collComm;
  if (nRecvParts != 1 || recvParts[0].size < bytesPerRank * g->nranks) return ncclInvalidUsage;
  char* out = (char*)recvParts[0].address;
  if (g->rank == 0) {
    std::vector<char> all;
    if (!collect(g, sendData, bytesPerRank, &all)) return ncclSystemError;
    memcpy(out, all.data(), all.size());
    for (int r = 1; r < g->nranks; ++r) if (!sendAll(g->fds[r], out, all.size())) return ncclSystemError;
  } else {
    if (!sendAll(g->fds[0], sendData, bytesPerRank) || !recvAll(g->fds[0], out, bytesPerRank * g->nranks)) return ncclSystemError;
  }
  note("allgather", bytesPerRank);
  *request = new Request{(int)bytesPerRank};
  return ncclSuccess;
}
ncclResult_t starReduceScatter(void* collComm, int nSendParts, ncclNetSGE_v12_t* sendParts, void* recvData, size_t bytesPerRank, size_t, size_t,
                               ncclDataType_t type, ncclRedOp_t op, void*, void** request) {
  Group* g = (Group*)collComm;
  const size_t total = bytesPerRank * g->nranks;
  if (nSendParts != 1 || sendParts[0].size < total) return ncclInvalidUsage;
  if (g->rank == 0) {
    std::vector<char> all;
    if (!collect(g, sendParts[0].address, total, &all)) return ncclSystemError;
    for (int r = 1; r < g->nranks; ++r) reduceInto(all.data(), all.data() + (size_t)r * total, total / sizeOf(type), type, op);
    memcpy(recvData, all.data(), bytesPerRank);
    for (int r = 1; r < g->nranks; ++r) if (!sendAll(g->fds[r], all.data() + (size_t)r * bytesPerRank, bytesPerRank)) return ncclSystemError;
  } else {
    if (!sendAll(g->fds[0], sendParts[0].address, total) || !recvAll(g->fds[0], recvData, bytesPerRank)) return ncclSystemError;
  }
  note("reducescatter", bytesPerRank);
  *request = new Request{(int)bytesPerRank};
  return ncclSuccess;
}
ncclResult_t starFlush(void*, void*, int, void*, void** request) { *request = new Request{0}; return ncclSuccess; }
ncclResult_t starTest(void* request, int* done, int* size) {
  Request* r = (Request*)request;
  *done = 1;
  if (size) *size = r->size;
  delete r;
  return ncclSuccess;
}
ncclResult_t starCloseColl(void* collComm) {
  Group* g = (Group*)collComm;
  for (int fd : g->fds) if (fd >= 0) close(fd);
  delete g;
  return ncclSuccess;
}
ncclResult_t starCloseListen(void* listenComm) {
  Listen* l = (Listen*)listenComm;
  close(l->fd);
  delete l;
  return ncclSuccess;
}
ncclResult_t starMakeVDevice(int*, ncclNetVDeviceProps_t*) { return ncclInvalidUsage; }
ncclResult_t starFinalize(void* ctx) { delete (int*)ctx; return ncclSuccess; }

}  // namespace

extern "C" {
__attribute__((visibility("default"))) ncclCollNet_v12_t ncclCollNetPlugin_v12 = {
    "Star", starInit, starDevices, starProps, starListen, starConnect, starReduceSupport, starRegMr, starRegMrDmaBuf, starDeregMr,
    starAllReduce, starAllGather, starReduceScatter, starFlush, starTest, starCloseColl, starCloseListen, starMakeVDevice, starFinalize};
}
