/*
 * Public host API of the B200-native collective library.
 *
 * The ABI (struct layouts, enum values, entry-point names and their p-prefixed
 * profiling twins) matches NCCL 2.30 (reference: src/nccl.h.in) so that a
 * program built against that header runs against this library unchanged.
 * Every definition below was written from the documented ABI, not copied.
 */
#ifndef NCCL_H_
#define NCCL_H_

#include <cuda_runtime.h>
#include <limits.h>
#include <stddef.h>
#include <stdint.h>

#define NCCL_MAJOR 2
#define NCCL_MINOR 30
#define NCCL_PATCH 7
#define NCCL_SUFFIX "+b200"
#define NCCL_VERSION(X, Y, Z) \
  (((X) <= 2 && (Y) <= 8) ? (X)*1000 + (Y)*100 + (Z) : (X)*10000 + (Y)*100 + (Z))
#define NCCL_VERSION_CODE NCCL_VERSION(NCCL_MAJOR, NCCL_MINOR, NCCL_PATCH)

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ncclComm* ncclComm_t;
typedef struct ncclWindow_vidmem* ncclWindow_t;
#define NCCL_COMM_NULL NULL

#define NCCL_UNIQUE_ID_BYTES 128
typedef struct { char internal[NCCL_UNIQUE_ID_BYTES]; } ncclUniqueId;

typedef enum {
  ncclSuccess = 0,
  ncclUnhandledCudaError = 1,
  ncclSystemError = 2,
  ncclInternalError = 3,
  ncclInvalidArgument = 4,
  ncclInvalidUsage = 5,
  ncclRemoteError = 6,
  ncclInProgress = 7,
  ncclTimeout = 8,
  ncclNumResults = 9
} ncclResult_t;

#define NCCL_CONFIG_UNDEF_INT INT_MIN
#define NCCL_CONFIG_UNDEF_PTR NULL
#define NCCL_SPLIT_NOCOLOR -1
#define NCCL_UNDEF_FLOAT -1.0f
#define NCCL_API_MAGIC 0xcafebeef

/* ncclCommWindowRegister flags */
#define NCCL_WIN_DEFAULT 0x00
#define NCCL_WIN_COLL_SYMMETRIC 0x01
#define NCCL_WIN_STRICT_ORDERING 0x02
#define NCCL_WIN_REQUIRED_ALIGNMENT 4096

/* ncclConfig_t::CTAPolicy */
#define NCCL_CTA_POLICY_DEFAULT 0x00
#define NCCL_CTA_POLICY_EFFICIENCY 0x01
#define NCCL_CTA_POLICY_ZERO 0x02

/* ncclCommShrink / ncclCommRevoke flags */
#define NCCL_SHRINK_DEFAULT 0x00
#define NCCL_SHRINK_ABORT 0x01
#define NCCL_REVOKE_DEFAULT 0x00

typedef struct ncclConfig_v23000 {
  size_t size;
  unsigned int magic;
  unsigned int version;
  int blocking;
  int cgaClusterSize;
  int minCTAs;
  int maxCTAs;
  const char* netName;
  int splitShare;
  int trafficClass;
  const char* commName;
  int collnetEnable;
  int CTAPolicy;
  int shrinkShare;
  int nvlsCTAs;
  int nChannelsPerNetPeer;
  int nvlinkCentricSched;
  int graphUsageMode;
  int numRmaCtx;
  int maxP2pPeers;
  int graphStreamOrdering;
} ncclConfig_t;

#define NCCL_CONFIG_INITIALIZER                                                     \
  { sizeof(ncclConfig_t), NCCL_API_MAGIC, NCCL_VERSION_CODE, NCCL_CONFIG_UNDEF_INT, \
    NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT,            \
    NCCL_CONFIG_UNDEF_PTR, NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT,            \
    NCCL_CONFIG_UNDEF_PTR, NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT,            \
    NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT,            \
    NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT,            \
    NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT }

typedef struct ncclSimInfo_v22200 {
  size_t size;
  unsigned int magic;
  unsigned int version;
  float estimatedTime;
} ncclSimInfo_t;

#define NCCL_SIM_INFO_INITIALIZER \
  { sizeof(ncclSimInfo_t), 0x74685283, NCCL_VERSION_CODE, NCCL_UNDEF_FLOAT }

typedef enum { ncclNumOps_dummy = 5 } ncclRedOp_dummy_t;
typedef enum {
  ncclSum = 0,
  ncclProd = 1,
  ncclMax = 2,
  ncclMin = 3,
  ncclAvg = 4,
  ncclNumOps = 5,
  /* handles returned by ncclRedOpCreatePreMulSum live in [ncclNumOps, ncclMaxRedOp] */
  ncclMaxRedOp = 0x7fffffff >> (32 - 8 * sizeof(ncclRedOp_dummy_t))
} ncclRedOp_t;

typedef enum {
  ncclInt8 = 0, ncclChar = 0,
  ncclUint8 = 1,
  ncclInt32 = 2, ncclInt = 2,
  ncclUint32 = 3,
  ncclInt64 = 4,
  ncclUint64 = 5,
  ncclFloat16 = 6, ncclHalf = 6,
  ncclFloat32 = 7, ncclFloat = 7,
  ncclFloat64 = 8, ncclDouble = 8,
  ncclBfloat16 = 9,
  ncclFloat8e4m3 = 10,
  ncclFloat8e5m2 = 11,
  ncclNumTypes = 12
} ncclDataType_t;

typedef enum { ncclScalarDevice = 0, ncclScalarHostImmediate = 1 } ncclScalarResidence_t;

#define NCCL_SUSPEND_MEM 0x01
typedef enum {
  ncclStatGpuMemSuspend = 0,
  ncclStatGpuMemSuspended = 1,
  ncclStatGpuMemPersist = 2,
  ncclStatGpuMemTotal = 3
} ncclCommMemStat_t;

typedef struct {
  int opCnt;
  int peer;
  int sigIdx;
  int ctx;
} ncclWaitSignalDesc_t;

typedef struct ncclParamHandle* ncclParamHandle_t;

/* Declares NAME and its profiling twin pNAME with the same signature. */
#define NCCL_API_DECL(ret, name, ...) \
  ret name(__VA_ARGS__);              \
  ret p##name(__VA_ARGS__)

/* Memory usable for every optimisation of the library (symmetric windows, multicast). */
NCCL_API_DECL(ncclResult_t, ncclMemAlloc, void** ptr, size_t size);
NCCL_API_DECL(ncclResult_t, ncclMemFree, void* ptr);

NCCL_API_DECL(ncclResult_t, ncclGetVersion, int* version);
NCCL_API_DECL(ncclResult_t, ncclGetUniqueId, ncclUniqueId* uniqueId);
NCCL_API_DECL(ncclResult_t, ncclCommInitRankConfig, ncclComm_t* comm, int nranks, ncclUniqueId commId,
              int rank, ncclConfig_t* config);
NCCL_API_DECL(ncclResult_t, ncclCommInitRank, ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank);
NCCL_API_DECL(ncclResult_t, ncclCommInitAll, ncclComm_t* comm, int ndev, const int* devlist);
NCCL_API_DECL(ncclResult_t, ncclCommInitRankScalable, ncclComm_t* newcomm, int nranks, int myrank, int nId,
              ncclUniqueId* commIds, ncclConfig_t* config);
NCCL_API_DECL(ncclResult_t, ncclCommFinalize, ncclComm_t comm);
NCCL_API_DECL(ncclResult_t, ncclCommDestroy, ncclComm_t comm);
NCCL_API_DECL(ncclResult_t, ncclCommAbort, ncclComm_t comm);
NCCL_API_DECL(ncclResult_t, ncclCommRevoke, ncclComm_t comm, int revokeFlags);
NCCL_API_DECL(ncclResult_t, ncclCommSplit, ncclComm_t comm, int color, int key, ncclComm_t* newcomm,
              ncclConfig_t* config);
NCCL_API_DECL(ncclResult_t, ncclCommShrink, ncclComm_t comm, int* excludeRanksList, int excludeRanksCount,
              ncclComm_t* newcomm, ncclConfig_t* config, int shrinkFlags);
NCCL_API_DECL(ncclResult_t, ncclCommGetUniqueId, ncclComm_t comm, ncclUniqueId* uniqueId);
NCCL_API_DECL(ncclResult_t, ncclCommGrow, ncclComm_t comm, int nRanks, const ncclUniqueId* uniqueId, int rank,
              ncclComm_t* newcomm, ncclConfig_t* config);
NCCL_API_DECL(const char*, ncclGetErrorString, ncclResult_t result);
NCCL_API_DECL(const char*, ncclGetLastError, ncclComm_t comm);
/* Reads the logging environment variables again (kept for source compatibility; deprecated upstream). */
void ncclResetDebugInit(void);
void pncclResetDebugInit(void);
NCCL_API_DECL(ncclResult_t, ncclCommGetAsyncError, ncclComm_t comm, ncclResult_t* asyncError);
NCCL_API_DECL(ncclResult_t, ncclCommCount, const ncclComm_t comm, int* count);
NCCL_API_DECL(ncclResult_t, ncclCommCuDevice, const ncclComm_t comm, int* device);
NCCL_API_DECL(ncclResult_t, ncclCommUserRank, const ncclComm_t comm, int* rank);
NCCL_API_DECL(ncclResult_t, ncclCommRegister, const ncclComm_t comm, void* buff, size_t size, void** handle);
NCCL_API_DECL(ncclResult_t, ncclCommDeregister, const ncclComm_t comm, void* handle);
NCCL_API_DECL(ncclResult_t, ncclCommSuspend, ncclComm_t comm, int flags);
NCCL_API_DECL(ncclResult_t, ncclCommResume, ncclComm_t comm);
NCCL_API_DECL(ncclResult_t, ncclCommMemStats, ncclComm_t comm, ncclCommMemStat_t stat, uint64_t* value);
NCCL_API_DECL(ncclResult_t, ncclCommWindowRegister, ncclComm_t comm, void* buff, size_t size, ncclWindow_t* win,
              int winFlags);
NCCL_API_DECL(ncclResult_t, ncclCommWindowDeregister, ncclComm_t comm, ncclWindow_t win);
NCCL_API_DECL(ncclResult_t, ncclWinGetUserPtr, ncclComm_t comm, ncclWindow_t win, void** outUserPtr);

NCCL_API_DECL(ncclResult_t, ncclRedOpCreatePreMulSum, ncclRedOp_t* op, void* scalar, ncclDataType_t datatype,
              ncclScalarResidence_t residence, ncclComm_t comm);
NCCL_API_DECL(ncclResult_t, ncclRedOpDestroy, ncclRedOp_t op, ncclComm_t comm);

NCCL_API_DECL(ncclResult_t, ncclReduce, const void* sendbuff, void* recvbuff, size_t count,
              ncclDataType_t datatype, ncclRedOp_t op, int root, ncclComm_t comm, cudaStream_t stream);
NCCL_API_DECL(ncclResult_t, ncclBcast, void* buff, size_t count, ncclDataType_t datatype, int root,
              ncclComm_t comm, cudaStream_t stream);
NCCL_API_DECL(ncclResult_t, ncclBroadcast, const void* sendbuff, void* recvbuff, size_t count,
              ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream);
NCCL_API_DECL(ncclResult_t, ncclAllReduce, const void* sendbuff, void* recvbuff, size_t count,
              ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
NCCL_API_DECL(ncclResult_t, ncclReduceScatter, const void* sendbuff, void* recvbuff, size_t recvcount,
              ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
NCCL_API_DECL(ncclResult_t, ncclAllGather, const void* sendbuff, void* recvbuff, size_t sendcount,
              ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream);
NCCL_API_DECL(ncclResult_t, ncclAlltoAll, const void* sendbuff, void* recvbuff, size_t count,
              ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream);
NCCL_API_DECL(ncclResult_t, ncclGather, const void* sendbuff, void* recvbuff, size_t count,
              ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream);
NCCL_API_DECL(ncclResult_t, ncclScatter, const void* sendbuff, void* recvbuff, size_t count,
              ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream);
NCCL_API_DECL(ncclResult_t, ncclSend, const void* sendbuff, size_t count, ncclDataType_t datatype, int peer,
              ncclComm_t comm, cudaStream_t stream);
NCCL_API_DECL(ncclResult_t, ncclRecv, void* recvbuff, size_t count, ncclDataType_t datatype, int peer,
              ncclComm_t comm, cudaStream_t stream);

/* One-sided operations on registered windows. */
NCCL_API_DECL(ncclResult_t, ncclPutSignal, const void* localbuff, size_t count, ncclDataType_t datatype,
              int peer, ncclWindow_t peerWin, size_t peerWinOffset, int sigIdx, int ctx, unsigned int flags,
              ncclComm_t comm, cudaStream_t stream);
NCCL_API_DECL(ncclResult_t, ncclSignal, int peer, int sigIdx, int ctx, unsigned int flags, ncclComm_t comm,
              cudaStream_t stream);
NCCL_API_DECL(ncclResult_t, ncclWaitSignal, int nDesc, ncclWaitSignalDesc_t* signalDescs, ncclComm_t comm,
              cudaStream_t stream);

NCCL_API_DECL(ncclResult_t, ncclGroupStart, void);
NCCL_API_DECL(ncclResult_t, ncclGroupEnd, void);
NCCL_API_DECL(ncclResult_t, ncclGroupSimulateEnd, ncclSimInfo_t* simInfo);

/* Typed parameter registry: query any tunable by key ("NCCL_DEBUG", ...). */
NCCL_API_DECL(ncclResult_t, ncclParamBind, ncclParamHandle_t* out, const char* key);
NCCL_API_DECL(ncclResult_t, ncclParamGetI8, ncclParamHandle_t h, int8_t* out);
NCCL_API_DECL(ncclResult_t, ncclParamGetI16, ncclParamHandle_t h, int16_t* out);
NCCL_API_DECL(ncclResult_t, ncclParamGetI32, ncclParamHandle_t h, int32_t* out);
NCCL_API_DECL(ncclResult_t, ncclParamGetI64, ncclParamHandle_t h, int64_t* out);
NCCL_API_DECL(ncclResult_t, ncclParamGetU8, ncclParamHandle_t h, uint8_t* out);
NCCL_API_DECL(ncclResult_t, ncclParamGetU16, ncclParamHandle_t h, uint16_t* out);
NCCL_API_DECL(ncclResult_t, ncclParamGetU32, ncclParamHandle_t h, uint32_t* out);
NCCL_API_DECL(ncclResult_t, ncclParamGetU64, ncclParamHandle_t h, uint64_t* out);
NCCL_API_DECL(ncclResult_t, ncclParamGetStr, ncclParamHandle_t h, const char** out);
NCCL_API_DECL(ncclResult_t, ncclParamGet, ncclParamHandle_t h, void* out, int maxLen, int* len);
NCCL_API_DECL(ncclResult_t, ncclParamGetParameter, const char* key, const char** value, int* valueLen);
NCCL_API_DECL(ncclResult_t, ncclParamGetAllParameterKeys, const char*** table, int* tableLen);
NCCL_API_DECL(void, ncclParamDumpAll, void);

#ifdef __cplusplus
}
#endif

#endif /* NCCL_H_ */
