/*
 * Interface of plugins that serve GPU-initiated networking (a NIC that kernels drive, or a proxy for one). The entry
 * points and their order follow the reference's v14 table, so a plugin library built for the reference exposes a
 * table this library can read. It is looked up in the network plugin library (NCCL_NET_PLUGIN), as the reference does.
 *
 * This build moves GPU-initiated traffic inside one NVLink domain (peer stores, or its own host proxy thread) and has no
 * network to hand such a plugin; the loader (src/plugin/gin.cc) initialises the plugin, reports its devices and
 * properties (log, ncclCommQueryProperties::railedGinType) and finalises it.
 * Reference parity: src/include/plugin/nccl_gin.h, gin/gin_v14.h.
 */
#ifndef NCCL_GIN_PLUGIN_H_
#define NCCL_GIN_PLUGIN_H_
#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#include "nccl.h"
#include "nccl_net.h"

#define NCCL_GIN_HANDLE_MAXSIZE 128
#define NCCL_GIN_SIGNAL_OP_INC 0x1
#define NCCL_GIN_SIGNAL_OP_ADD 0x2

typedef struct {
  bool supportsStrongSignals;
  bool supportsVASignals;
} ncclGinProperties_v14_t;

typedef struct {
  int nSignals;
  int nCounters;
  int nContexts;
  int queueDepth;
  int trafficClass;
  int backendVersion;
  int rankStride;
} ncclGinConfig_v14_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(void** ctx, uint64_t commId, ncclDebugLogger_t logFunction);
  ncclResult_t (*devices)(int* ndev);
  ncclResult_t (*getGinProperties)(ncclGinProperties_v14_t* ginProps);
  ncclResult_t (*getProperties)(int dev, ncclNetProperties_t* props);
  ncclResult_t (*listen)(void* ctx, int dev, void* handle, void** listenComm);
  ncclResult_t (*connect)(void* ctx, void* handles[], int nranks, int rank, void* listenComm, void** collComm);
  ncclResult_t (*createContext)(void* collComm, ncclGinConfig_v14_t* config, void** ginCtx, void** devHandle);
  ncclResult_t (*regMrSym)(void* collComm, void* data, size_t size, int type, uint64_t mrFlags, void** mhandle, void** ginHandle);
  ncclResult_t (*regMrSymDmaBuf)(void* collComm, void* data, size_t size, int type, uint64_t offset, int fd, uint64_t mrFlags, void** mhandle,
                                 void** ginHandle);
  ncclResult_t (*deregMrSym)(void* collComm, void* mhandle);
  ncclResult_t (*destroyContext)(void* ginCtx);
  ncclResult_t (*closeColl)(void* collComm);
  ncclResult_t (*closeListen)(void* listenComm);
  ncclResult_t (*ginProgress)(void* ginCtx);
  ncclResult_t (*queryLastError)(void* ginCtx, bool* hasError);
  ncclResult_t (*finalize)(void* ctx);
} ncclGin_v14_t;

typedef ncclGin_v14_t ncclGin_t;
typedef ncclGinConfig_v14_t ncclGinConfig_t;
typedef ncclGinProperties_v14_t ncclGinProperties_t;
#define NCCL_GIN_PLUGIN_SYMBOL "ncclGinPlugin_v14"

#endif
