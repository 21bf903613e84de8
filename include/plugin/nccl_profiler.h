/*
 * Profiler plugin interface (`ncclProfiler_v6`). The core opens an event with startEvent(),
 * may report state changes, and closes it with stopEvent(). Events nest through parentObj:
 *   group API -> collective / p2p API -> kernel launch
 *   group -> collective / p2p task -> kernel channel (device timestamps) / proxy op -> proxy step
 * Reference parity: src/include/plugin/nccl_profiler.h, profiler/profiler_v5.h, profiler_v6.h:129-146.
 */
#ifndef NCCL_B200_PLUGIN_PROFILER_H_
#define NCCL_B200_PLUGIN_PROFILER_H_
#include <stdbool.h>
#include <stddef.h>

#include "nccl_common.h"

enum {
  ncclProfileGroup = 1 << 0, ncclProfileColl = 1 << 1, ncclProfileP2p = 1 << 2, ncclProfileProxyOp = 1 << 3, ncclProfileProxyStep = 1 << 4,
  ncclProfileProxyCtrl = 1 << 5, ncclProfileKernelCh = 1 << 6, ncclProfileNetPlugin = 1 << 7, ncclProfileGroupApi = 1 << 8,
  ncclProfileCollApi = 1 << 9, ncclProfileP2pApi = 1 << 10, ncclProfileKernelLaunch = 1 << 11, ncclProfileCeColl = 1 << 12,
  ncclProfileCeSync = 1 << 13, ncclProfileCeBatch = 1 << 14
};

typedef enum {
  ncclProfilerProxyOpSendPosted = 0, ncclProfilerProxyOpSendRemFifoWait = 1, ncclProfilerProxyOpSendTransmitted = 2, ncclProfilerProxyOpSendDone = 3,
  ncclProfilerProxyOpRecvPosted = 4, ncclProfilerProxyOpRecvReceived = 5, ncclProfilerProxyOpRecvTransmitted = 6, ncclProfilerProxyOpRecvDone = 7,
  ncclProfilerProxyStepSendGPUWait = 8, ncclProfilerProxyStepSendWait = 9, ncclProfilerProxyStepRecvWait = 10, ncclProfilerProxyStepRecvFlushWait = 11,
  ncclProfilerProxyStepRecvGPUWait = 12, ncclProfilerProxyCtrlIdle = 13, ncclProfilerProxyCtrlActive = 14, ncclProfilerProxyCtrlSleep = 15,
  ncclProfilerProxyCtrlWakeup = 16, ncclProfilerProxyCtrlAppend = 17, ncclProfilerProxyCtrlAppendEnd = 18, ncclProfilerProxyOpInProgress_v4 = 19,
  ncclProfilerProxyStepSendPeerWait_v4 = 20, ncclProfilerNetPluginUpdate = 21, ncclProfilerKernelChStop = 22, ncclProfilerGroupStartApiStop = 23,
  ncclProfilerGroupEndApiStart = 24, ncclProfilerCeCollStart = 25, ncclProfilerCeCollComplete = 26, ncclProfilerCeSyncStart = 27,
  ncclProfilerCeSyncComplete = 28, ncclProfilerCeBatchStart = 29, ncclProfilerCeBatchComplete = 30
} ncclProfilerEventState_t;

typedef struct {
  uint64_t type;     /* one of the ncclProfile* bits */
  void* parentObj;   /* handle of the enclosing event, or NULL */
  int rank;
  union {
    struct { bool graphCaptured; int groupDepth; } groupApi;
    struct { const char* func; size_t count; const char* datatype; int root; void* stream; bool graphCaptured; } collApi;
    struct { const char* func; size_t count; const char* datatype; void* stream; bool graphCaptured; } p2pApi;
    struct { void* stream; } kernelLaunch;
    struct {
      uint64_t seqNumber; const char* func; void const* sendBuff; void* recvBuff; size_t count; int root; const char* datatype;
      uint8_t nChannels; uint8_t nWarps; const char* algo; const char* proto; void* parentGroup;
    } coll;
    struct { const char* func; void* buff; const char* datatype; size_t count; int peer; uint8_t nChannels; void* parentGroup; } p2p;
    struct { ncclPid_t pid; uint8_t channelId; int peer; int nSteps; int chunkSize; int isSend; } proxyOp;
    struct { int step; } proxyStep;
    struct { uint8_t channelId; uint64_t pTimer; } kernelCh;
    struct { int64_t id; void* data; } netPlugin;
    struct {
      uint64_t seqNumber; const char* func; void const* sendBuff; void* recvBuff; size_t count; int root; const char* datatype;
      const char* syncStrategy; bool intraBatchSync; uint32_t batchSize; uint32_t numBatches; uint32_t ceSeqNum; void* stream;
    } ceColl;
    struct { bool isComplete; int nRanks; } ceCollSync;
    struct { int numOps; size_t totalBytes; bool useIntraSync; } ceCollBatch;
  };
} ncclProfilerEventDescr_t;

typedef union {
  struct { size_t transSize; } proxyStep;
  struct { int appendedProxyOps; } proxyCtrl;
  struct { void* data; } netPlugin;
  struct { uint64_t pTimer; } kernelCh;
} ncclProfilerEventStateArgs_t;

typedef struct {
  const char* name;
  /* eActivationMask: the plugin writes the OR of the event types it wants */
  ncclResult_t (*init)(void** context, uint64_t commId, int* eActivationMask, const char* commName, int nNodes, int nranks, int rank,
                       ncclDebugLogger_t logfn);
  ncclResult_t (*startEvent)(void* context, void** eHandle, ncclProfilerEventDescr_t* eDescr);
  ncclResult_t (*stopEvent)(void* eHandle);
  ncclResult_t (*recordEventState)(void* eHandle, ncclProfilerEventState_t eState, ncclProfilerEventStateArgs_t* eStateArgs);
  ncclResult_t (*finalize)(void* context);
} ncclProfiler_v6_t;

typedef ncclProfiler_v6_t ncclProfiler_t;
#define NCCL_PROFILER_PLUGIN_SYMBOL "ncclProfiler_v6"

#endif
