/*
 * Tuner plugin interface. A tuner library exports `ncclTunerPlugin_v6` (or `_v5`: the same
 * struct without getChunkSize). For every collective the core fills a cost table
 * [algorithm][protocol] with predicted microseconds (-1 = not available); the plugin may edit the
 * table and the channel count, and the core then takes the cheapest entry.
 * Reference parity: src/include/plugin/nccl_tuner.h, tuner/tuner_v5.h, tuner/tuner_v6.h.
 */
#ifndef NCCL_B200_PLUGIN_TUNER_H_
#define NCCL_B200_PLUGIN_TUNER_H_
#include "nccl_common.h"

#define NCCL_ALGO_UNDEF -1
#define NCCL_ALGO_TREE 0
#define NCCL_ALGO_RING 1
#define NCCL_ALGO_COLLNET_DIRECT 2
#define NCCL_ALGO_COLLNET_CHAIN 3
#define NCCL_ALGO_NVLS 4
#define NCCL_ALGO_NVLS_TREE 5
#define NCCL_ALGO_PAT 6
#define NCCL_NUM_ALGORITHMS 7

#define NCCL_PROTO_UNDEF -1
#define NCCL_PROTO_LL 0
#define NCCL_PROTO_LL128 1
#define NCCL_PROTO_SIMPLE 2
#define NCCL_NUM_PROTOCOLS 3

#define NCCL_ALGO_PROTO_IGNORE -1.0

#define NCCL_HW_NVLINK 0
#define NCCL_HW_PCI 1
#define NCCL_HW_NET 2
#define NCCL_NUM_HW_LINKS 3
#define NCCL_NUM_COMPCAPS 4        /* volta, ampere, hopper, blackwell */
#define NCCL_BLACKWELL_COMPCAP_IDX 3
#define NCCL_NUM_TUNING_SCALES 3   /* 1, 2, 4+ nodes */

typedef struct {
  int nNvlDomains;
  int minRanksPerNvlDomain;
  int maxRanksPerNvlDomain;
} ncclNvlDomainInfo_t;

/* Constants of the analytic model, shown to the plugin at init; it may rewrite them. */
typedef struct {
  double baseLatencies[NCCL_NUM_ALGORITHMS][NCCL_NUM_PROTOCOLS];
  double hwLatencies[NCCL_NUM_HW_LINKS][NCCL_NUM_ALGORITHMS][NCCL_NUM_PROTOCOLS];
  double llMaxBws[NCCL_NUM_COMPCAPS][NCCL_NUM_TUNING_SCALES];
  double perChMaxRingLL128Bws[NCCL_NUM_COMPCAPS][NCCL_NUM_TUNING_SCALES];
  double perChMaxTreeLL128Bws[NCCL_NUM_COMPCAPS][NCCL_NUM_TUNING_SCALES];
  double perChMaxTreeBws[NCCL_NUM_COMPCAPS][NCCL_NUM_TUNING_SCALES];
  double perChMaxNVLSTreeBws[NCCL_NUM_COMPCAPS][NCCL_NUM_TUNING_SCALES];
} ncclTunerConstants_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(void** ctx, uint64_t commId, size_t nRanks, size_t nNodes, ncclDebugLogger_t logFunction, ncclNvlDomainInfo_t* nvlDomainInfo,
                       ncclTunerConstants_t* constants);
  ncclResult_t (*getCollInfo)(void* ctx, ncclFunc_t collType, size_t nBytes, int numPipeOps, float** collCostTable, int numAlgo, int numProto,
                              int regBuff, int* nChannels);
  ncclResult_t (*finalize)(void* ctx);
} ncclTuner_v5_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(void** ctx, uint64_t commId, size_t nRanks, size_t nNodes, ncclDebugLogger_t logFunction, ncclNvlDomainInfo_t* nvlDomainInfo,
                       ncclTunerConstants_t* constants);
  ncclResult_t (*getCollInfo)(void* ctx, ncclFunc_t collType, size_t nBytes, int numPipeOps, float** collCostTable, int numAlgo, int numProto,
                              int regBuff, int* nChannels);
  ncclResult_t (*finalize)(void* ctx);
  /* optional: override the pipeline chunk size chosen for (algo, proto) */
  ncclResult_t (*getChunkSize)(void* ctx, ncclFunc_t collType, size_t nBytes, int algo, int proto, int nChannels, size_t* chunkSize);
} ncclTuner_v6_t;

/* Earlier interfaces, still loaded (reference: src/plugin/tuner/tuner_v2.cc ... tuner_v4.cc).
 * v4 / v3: context comes back from init; v3 has no regBuff argument; v2 names its choice directly. */
typedef struct {
  const char* name;
  ncclResult_t (*init)(size_t nRanks, size_t nNodes, ncclDebugLogger_t logFunction, void** ctx);
  ncclResult_t (*getCollInfo)(void* ctx, ncclFunc_t collType, size_t nBytes, int numPipeOps, float** collCostTable, int numAlgo, int numProto,
                              int regBuff, int* nChannels);
  ncclResult_t (*destroy)(void* ctx);
} ncclTuner_v4_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(size_t nRanks, size_t nNodes, ncclDebugLogger_t logFunction, void** ctx);
  ncclResult_t (*getCollInfo)(void* ctx, ncclFunc_t collType, size_t nBytes, int numPipeOps, float** collCostTable, int numAlgo, int numProto,
                              int* nChannels);
  ncclResult_t (*destroy)(void* ctx);
} ncclTuner_v3_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(size_t nRanks, size_t nNodes, ncclDebugLogger_t logFunction, void** ctx);
  ncclResult_t (*getCollInfo)(void* ctx, ncclFunc_t collType, size_t nBytes, int collNetSupport, int nvlsSupport, int numPipeOps,
                              int* algorithm, int* protocol, int* nChannels);
  ncclResult_t (*destroy)(void* ctx);
} ncclTuner_v2_t;

typedef ncclTuner_v6_t ncclTuner_t;
#define NCCL_TUNER_PLUGIN_SYMBOL "ncclTunerPlugin_v6"

#endif
