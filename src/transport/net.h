// Network transport of the host data plane: the ncclNet_t table in use (an external plugin or
// the built-in TCP backend), per-peer send/receive connections, and the proxy thread that
// progresses posted operations.
// Reference parity: src/transport/net.cc (proxy progress :1304-1765), src/proxy.cc (progress
// thread :954), src/plugin/net.cc (plugin choice), src/transport/net_socket.cc (TCP backend).
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include "../comm/comm.h"
#include "../plugin/plugin.h"
#include "plugin/nccl_net.h"
#include "plugin/nccl_profiler_net.h"

namespace b200 {

extern ncclNet_t netSocketBackend;                 // transport/net_socket.cc
extern ncclNet_t netIbBackend;                     // transport/net_ib.cc (no device unless libibverbs and an active port are there)

// Resolves the network backend once per process: NCCL_NET_PLUGIN (library), NCCL_NET (name); without either, the
// InfiniBand backend when it finds a device, else TCP sockets.
ncclResult_t netSelect(ncclNet_t** net, bool* external);
ncclCollNet_t* netCollNetTable();                  // collective-network table of the loaded plugin, or nullptr

// Collective network (in-network reduction) of a communicator: transport/collnet.cc
struct CollNet;
ncclResult_t collNetCreate(ncclComm* comm, CollNet** out);   // collective over the bootstrap; *out stays nullptr unless every rank can join
void collNetDestroy(CollNet* c);
bool collNetSupports(CollNet* c, ncclDataType_t type, ncclRedOp_t op);
ncclResult_t collNetAllReduce(ncclComm* comm, CollNet* c, const void* send, void* recv, size_t count, ncclDataType_t type, ncclRedOp_t op);
ncclResult_t collNetAllGather(ncclComm* comm, CollNet* c, const void* send, void* recv, size_t bytesPerRank);
ncclResult_t collNetReduceScatter(ncclComm* comm, CollNet* c, const void* send, void* recv, size_t countPerRank, ncclDataType_t type, ncclRedOp_t op);
void pluginLogger(ncclDebugLogLevel level, unsigned long flags, const char* file, int line, const char* fmt, ...);

struct ProxyOp {
  bool isSend;
  int peer;
  char* data;
  size_t bytes;
  size_t posted = 0;        // bytes handed to the network so far
  size_t completed = 0;
  void* requests[NCCL_NET_MAX_REQUESTS] = {};
  size_t reqBytes[NCCL_NET_MAX_REQUESTS] = {};
  int head = 0, tail = 0;   // ring of requests in flight
  std::atomic<int> state{0};   // 0 running, 1 done, <0 failed (ncclResult_t negated)
  void* profHandle = nullptr;
  // One event per slice (ncclProfileProxyStep) under the operation's; the backend's own events hang under the slice's. A slice
  // whose post was refused ("not yet") keeps its event for the next try.
  void* stepHandle[NCCL_NET_MAX_REQUESTS] = {};
  ProfNetParent stepParent[NCCL_NET_MAX_REQUESTS] = {};
  void* nextStep = nullptr;
  int stepsStarted = 0;
  void* mhandle = nullptr;   // the backend's registration of [data, data+bytes), made when the operation starts
  bool regTried = false;
};

struct Proxy {
  ncclComm* comm = nullptr;
  ncclNet_t* net = nullptr;
  bool external = false;
  void* netCtx = nullptr;
  int dev = 0;
  void* listenComm = nullptr;
  std::vector<void*> sendComm, recvComm;   // per peer
  size_t sliceBytes = 0;
  int maxInflight = 0;
  std::thread thread;
  std::mutex lock;
  std::condition_variable wake;
  std::deque<ProxyOp*> ops;
  bool stop = false;
  uint64_t opsDone = 0, bytesMoved = 0, steps = 0;
};

ncclResult_t proxyCreate(ncclComm* comm);      // collective: listen, exchange handles, connect the full mesh, start the thread
void proxyDestroy(ncclComm* comm);
void proxyQuiesce(ncclComm* comm);   // ends the progress thread; connections stay until proxyDestroy
// Posts an operation; the proxy thread progresses it. proxyWait blocks until every op given is done.
ProxyOp* proxyPost(Proxy* p, bool isSend, int peer, void* data, size_t bytes);
ncclResult_t proxyWait(Proxy* p, ProxyOp** ops, int n);

}  // namespace b200
