/*
 * Network plugin interface (`ncclNetPlugin_v12`): point-to-point transfers between hosts.
 * The core calls listen() on the receiver, passes the opaque handle (at most
 * NCCL_NET_HANDLE_MAXSIZE bytes) to the sender out of band, then connect() / accept() (both may
 * return a NULL comm meaning "not yet, call again"), and moves data with isend / irecv / test.
 * The built-in backend "Socket" (transport/net_socket.cc) implements the same table over TCP.
 * Reference parity: src/include/plugin/nccl_net.h, net/net_v12.h; nccl_device/net_device.h.
 */
#ifndef NCCL_B200_PLUGIN_NET_H_
#define NCCL_B200_PLUGIN_NET_H_
#include <stddef.h>

#include "nccl_common.h"

#define NCCL_NET_HANDLE_MAXSIZE 128
#define NCCL_PTR_HOST 0x1
#define NCCL_PTR_CUDA 0x2
#define NCCL_PTR_DMABUF 0x4
#define NCCL_NET_MAX_REQUESTS 32
#define NCCL_NET_MAX_DEVS_PER_NIC 8
#define NCCL_NET_TRAFFIC_CLASS_UNDEF -1
#define NCCL_NET_ATTR_UNDEF -1
#define NCCL_NET_OPTIONAL_RECV_COMPLETION 0x1

typedef enum {
  NCCL_NET_DEVICE_HOST = 0, NCCL_NET_DEVICE_UNPACK = 1, NCCL_NET_DEVICE_GIN_PROXY = 2, NCCL_NET_DEVICE_GIN_GDAKI = 3, NCCL_NET_DEVICE_GIN_GPI = 4
} ncclNetDeviceType;

typedef struct {
  ncclNetDeviceType netDeviceType;
  int netDeviceVersion;
  void* handle;
  size_t size;
  int needsProxyProgress;
} ncclNetDeviceHandle_t;

typedef struct { int ndevs; int devs[NCCL_NET_MAX_DEVS_PER_NIC]; } ncclNetVDeviceProps_t;
typedef struct { int trafficClass; } ncclNetCommConfig_t;

typedef struct {
  char* name;
  char* pciPath;        /* /sys path of the PCI device, NULL for virtual interfaces */
  uint64_t guid;
  int ptrSupport;       /* NCCL_PTR_* bits */
  int regIsGlobal;
  int forceFlush;
  int speed;            /* Mbps */
  int port;
  float latency;        /* microseconds */
  int maxComms;
  int maxRecvs;         /* receives that one irecv may group */
  ncclNetDeviceType netDeviceType;
  int netDeviceVersion;
  ncclNetVDeviceProps_t vProps;
  size_t maxP2pBytes;
  size_t maxCollBytes;
  int maxMultiRequestSize;
  int16_t railId;
  int16_t planeId;
} ncclNetProperties_t;

typedef struct { int32_t maxConcurrentPeers, minConcurrentPeers, maxFlowsPerPeer, minFlowsPerPeer; } ncclNetCommAttr_t;
typedef struct { ncclNetCommAttr_t sendCommAttr, recvCommAttr; uint32_t op, algo, proto; } ncclNetAttr_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(void** ctx, uint64_t commId, ncclNetCommConfig_t* config, ncclDebugLogger_t logFunction, ncclProfilerCallback_t profFunction);
  ncclResult_t (*devices)(int* ndev);
  ncclResult_t (*getProperties)(int dev, ncclNetProperties_t* props);
  ncclResult_t (*listen)(void* ctx, int dev, void* handle, void** listenComm);
  ncclResult_t (*connect)(void* ctx, int dev, void* handle, void** sendComm, ncclNetDeviceHandle_t** sendDevComm);
  ncclResult_t (*accept)(void* listenComm, void** recvComm, ncclNetDeviceHandle_t** recvDevComm);
  ncclResult_t (*regMr)(void* comm, void* data, size_t size, int type, void** mhandle);
  ncclResult_t (*regMrDmaBuf)(void* comm, void* data, size_t size, int type, uint64_t offset, int fd, void** mhandle);
  ncclResult_t (*deregMr)(void* comm, void* mhandle);
  ncclResult_t (*isend)(void* sendComm, void* data, size_t size, int tag, void* mhandle, void* phandle, void** request);
  ncclResult_t (*irecv)(void* recvComm, int n, void** data, size_t* sizes, int* tags, void** mhandles, void** phandles, void** request);
  ncclResult_t (*iflush)(void* recvComm, int n, void** data, int* sizes, void** mhandles, void** request);
  ncclResult_t (*test)(void* request, int* done, int* sizes);
  ncclResult_t (*closeSend)(void* sendComm);
  ncclResult_t (*closeRecv)(void* recvComm);
  ncclResult_t (*closeListen)(void* listenComm);
  ncclResult_t (*getDeviceMr)(void* comm, void* mhandle, void** dptr_mhandle);
  ncclResult_t (*irecvConsumed)(void* recvComm, int n, void* request);
  ncclResult_t (*makeVDevice)(int* d, ncclNetVDeviceProps_t* props);
  ncclResult_t (*finalize)(void* ctx);
  ncclResult_t (*setNetAttr)(void* ctx, ncclNetAttr_t* netAttr);
} ncclNet_v12_t;

typedef ncclNet_v12_t ncclNet_t;
#define NCCL_NET_PLUGIN_SYMBOL "ncclNetPlugin_v12"

/* ---- collective network: a fabric that reduces / gathers on its own (in-network reduction).
 * A net plugin may export this second table; all ranks of a communicator then form one group
 * (listen on every rank, handles exchanged by the library, connect) and hand whole collectives to it. */
typedef struct {
  void* mhandle;
  void* address;
  size_t size;
} ncclNetSGE_v12_t;
typedef ncclNetSGE_v12_t ncclNetSGE_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(void** ctx, uint64_t commId, ncclDebugLogger_t logFunction);
  ncclResult_t (*devices)(int* ndev);                                   /* 0 devices: nothing else needs to be set */
  ncclResult_t (*getProperties)(int dev, ncclNetProperties_t* props);
  ncclResult_t (*listen)(void* ctx, int dev, void* handle, void** listenComm);
  ncclResult_t (*connect)(void* handles[], int nranks, int rank, void* listenComm, void** collComm);
  ncclResult_t (*reduceSupport)(ncclDataType_t dataType, ncclRedOp_t redOp, int* supported);
  ncclResult_t (*regMr)(void* collComm, void* data, size_t size, int type, void** mhandle);
  ncclResult_t (*regMrDmaBuf)(void* collComm, void* data, size_t size, int type, uint64_t offset, int fd, void** mhandle);
  ncclResult_t (*deregMr)(void* collComm, void* mhandle);
  ncclResult_t (*iallreduce)(void* collComm, void* sendData, void* recvData, size_t count, ncclDataType_t dataType,
                             ncclRedOp_t redOp, void* sendMhandle, void* recvMhandle, void** request);
  ncclResult_t (*iallgather)(void* collComm, void* sendData, int nRecvParts, ncclNetSGE_v12_t* recvParts, size_t bytesPerRank,
                             size_t windowOffset, size_t windowBytes, void* sendMhandle, void** request);
  ncclResult_t (*ireducescatter)(void* collComm, int nSendParts, ncclNetSGE_v12_t* sendParts, void* recvData, size_t bytesPerRank,
                                 size_t windowOffset, size_t windowBytes, ncclDataType_t dataType, ncclRedOp_t redOp,
                                 void* recvMhandle, void** request);
  ncclResult_t (*iflush)(void* collComm, void* data, int size, void* mhandle, void** request);
  ncclResult_t (*test)(void* request, int* done, int* size);
  ncclResult_t (*closeColl)(void* collComm);
  ncclResult_t (*closeListen)(void* listenComm);
  ncclResult_t (*makeVDevice)(int* d, ncclNetVDeviceProps_t* props);
  ncclResult_t (*finalize)(void* ctx);
} ncclCollNet_v12_t;

typedef ncclCollNet_v12_t ncclCollNet_t;
#define NCCL_COLLNET_PLUGIN_SYMBOL "ncclCollNetPlugin_v12"

#endif
