/*
 * Expert-parallel (MoE) dispatch / combine over a communicator.
 *
 * API shape of the reference extension (contrib/nccl_ep/include/nccl_ep.h): tensors are described
 * by ncclEpTensor_t, configuration structs start with {size, magic}, a group owns the symmetric
 * buffers, a handle owns the routing of one batch, dispatch sends tokens to the ranks of their
 * selected experts and combine brings the expert outputs back as a weighted sum.
 *
 * This implementation serves ranks that can map each other's memory (one NVLink domain) with one
 * fused kernel per direction; the layout of dispatched tokens is expert-major:
 *   tokens   [num_local_experts, num_ranks * max_dispatch_tokens_per_rank, hidden]
 *   scales   [num_local_experts, num_ranks * max_dispatch_tokens_per_rank, hidden / 128]  (fp8 dispatch)
 *   expert_counters[num_local_experts] = rows in use per expert.
 * Passing an output `scales` tensor selects fp8 (e4m3, one fp32 scale per 128 channels) dispatch.
 */
#ifndef NCCL_EP_H_
#define NCCL_EP_H_

#include "nccl.h"

#ifdef __cplusplus
extern "C" {
#endif

#define NCCL_EP_MAJOR 0
#define NCCL_EP_MINOR 1
#define NCCL_EP_PATCH 0
#define NCCL_EP_VERSION_CODE (NCCL_EP_MAJOR * 10000 + NCCL_EP_MINOR * 100 + NCCL_EP_PATCH)
#define NCCL_EP_API_VERSION 1
#define NCCL_EP_MAGIC 0xC00FFFEEu
#define NCCL_EP_TENSOR_MAGIC 0xCAFECAFE
#define NCCL_EP_AUTO 0

typedef enum { NCCL_EP_ALGO_LOW_LATENCY = 0, NCCL_EP_ALGO_HIGH_THROUGHPUT = 1 } ncclEpAlgorithm_t;
typedef enum { NCCL_EP_LAYOUT_UNSET = NCCL_EP_AUTO, NCCL_EP_LAYOUT_EXPERT_MAJOR, NCCL_EP_LAYOUT_RANK_MAJOR, NCCL_EP_LAYOUT_FLAT } ncclEpLayout_t;
typedef enum { NCCL_EP_FWD_PASS = 0, NCCL_EP_BWD_PASS = 1 } ncclEpPassDir_t;

typedef struct ncclEpTensor {
  unsigned int size;
  unsigned int magic;
  unsigned int ndim;
  ncclDataType_t datatype;
  void* data;
  ncclWindow_t win_hdl;
  uint64_t win_offset;
  size_t* sizes;
} ncclEpTensor_t;

typedef struct { unsigned int size; unsigned int magic; } ncclEpTensorAllocConfig_t;

typedef cudaError_t (*ncclEpAllocFn_t)(void** ptr, size_t size, void* context);
typedef cudaError_t (*ncclEpFreeFn_t)(void* ptr, void* context);
typedef struct { ncclEpAllocFn_t alloc_fn; ncclEpFreeFn_t free_fn; void* context; } ncclEpAllocConfig_t;

typedef struct {
  unsigned int size;
  unsigned int magic;
  unsigned int version;
  ncclEpAlgorithm_t algorithm;
  unsigned int num_experts;
  unsigned int max_dispatch_tokens_per_rank;
  unsigned int max_recv_tokens_per_rank;
  unsigned int max_token_bytes;          /* bytes of one bf16 token row: 2 * hidden */
  unsigned long int rdma_buffer_size;
  unsigned int num_qp_per_rank;
  unsigned int num_channels;
  unsigned int max_num_sms;
  ncclEpAllocConfig_t alloc;
  unsigned int enable_mask;
  uint64_t timeout_ns;
} ncclEpGroupConfig_t;

typedef struct ncclEpGroup* ncclEpGroup_t;
typedef struct ncclEpHandle* ncclEpHandle_t;

typedef struct {
  unsigned int size;
  unsigned int magic;
  ncclEpTensor_t* expert_counters;
  ncclEpTensor_t* src_rank_counters;
  ncclEpTensor_t* expert_offsets;
  ncclEpTensor_t* recv_total_counter;
} ncclEpLayoutInfo_t;

typedef struct { unsigned int size; unsigned int magic; ncclEpTensor_t* tokens; ncclEpTensor_t* topk_weights; ncclEpTensor_t* scales; } ncclEpDispatchInputs_t;
typedef struct { unsigned int size; unsigned int magic; ncclEpTensor_t* tokens; ncclEpTensor_t* topk_weights; ncclEpTensor_t* scales; ncclEpTensor_t* topk_idx; } ncclEpDispatchOutputs_t;
typedef struct { unsigned int size; unsigned int magic; ncclEpTensor_t* tokens; ncclEpTensor_t* topk_weights; } ncclEpCombineInputs_t;
typedef struct { unsigned int size; unsigned int magic; ncclEpTensor_t* tokens; ncclEpTensor_t* topk_weights; } ncclEpCombineOutputs_t;
typedef struct { unsigned int size; unsigned int magic; size_t dispatch_output_per_expert_alignment; } ncclEpHandleConfig_t;
typedef struct { unsigned int size; unsigned int magic; unsigned int send_only; unsigned int round_scales; ncclEpPassDir_t pass_direction; } ncclEpDispatchConfig_t;
typedef struct { unsigned int size; unsigned int magic; unsigned int send_only; ncclEpPassDir_t pass_direction; } ncclEpCombineConfig_t;
typedef struct ncclEpCompleteConfig { unsigned int size; unsigned int magic; } ncclEpCompleteConfig_t;

ncclResult_t ncclEpGetVersion(int* version);
ncclResult_t ncclEpTensorAlloc(ncclEpTensor_t** tensor, unsigned int ndim, ncclDataType_t datatype, const size_t* sizes, const ncclEpTensorAllocConfig_t* config);
ncclResult_t ncclEpTensorDestroy(ncclEpTensor_t* tensor);
ncclResult_t ncclEpCreateGroup(ncclEpGroup_t* ep_group, ncclComm_t comm, const ncclEpGroupConfig_t* config);
ncclResult_t ncclEpGroupDestroy(ncclEpGroup_t ep_group);
ncclResult_t ncclEpHandleMemSize(ncclEpGroup_t ep_group, ncclEpLayout_t layout, const ncclEpHandleConfig_t* config, size_t* size_out, int num_topk);
ncclResult_t ncclEpInitHandle(ncclEpHandle_t* handle, ncclEpGroup_t ep_group, ncclEpLayout_t layout, const ncclEpHandleConfig_t* config, int num_topk, const ncclEpTensor_t* handle_mem);
ncclResult_t ncclEpUpdateHandle(ncclEpHandle_t handle, const ncclEpTensor_t* topk_idx, const ncclEpLayoutInfo_t* layout_info, cudaStream_t stream);
ncclResult_t ncclEpCreateHandle(ncclEpHandle_t* handle, ncclEpGroup_t ep_group, ncclEpLayout_t layout, const ncclEpTensor_t* topk_idx, const ncclEpLayoutInfo_t* layout_info, const ncclEpHandleConfig_t* config, cudaStream_t stream);
ncclResult_t ncclEpHandleDestroy(ncclEpHandle_t handle);
ncclResult_t ncclEpDispatch(ncclEpHandle_t handle, const ncclEpDispatchInputs_t* inputs, const ncclEpDispatchOutputs_t* outputs, const ncclEpLayoutInfo_t* layout_info, const ncclEpDispatchConfig_t* config, cudaStream_t stream);
ncclResult_t ncclEpCombine(ncclEpHandle_t handle, const ncclEpCombineInputs_t* inputs, const ncclEpCombineOutputs_t* outputs, const ncclEpCombineConfig_t* config, cudaStream_t stream);
ncclResult_t ncclEpComplete(ncclEpHandle_t handle, const ncclEpCompleteConfig_t* config, cudaStream_t stream);
ncclResult_t ncclEpMaskQuery(ncclEpGroup_t ep_group, int* mask_status, cudaStream_t stream);
ncclResult_t ncclEpMaskUpdate(ncclEpGroup_t ep_group, const int* mask, cudaStream_t stream);
ncclResult_t ncclEpMaskClean(ncclEpGroup_t ep_group, cudaStream_t stream);
ncclResult_t ncclEpGetAsyncError(ncclEpGroup_t ep_group, int* error_out);
ncclResult_t ncclEpErrorClear(ncclEpGroup_t ep_group);

#ifdef __cplusplus
}
#endif
#endif
