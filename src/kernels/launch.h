// Host-visible handles of the device kernels (defined in the .cu files of this directory).
#pragma once
#include <cuda_runtime.h>

#include "args.h"
#include "nccl.h"

namespace b200 {

enum KernelId : int {
  KERNEL_REDUCE_P2P = 0,
  KERNEL_ALLREDUCE_LL = 1,
  KERNEL_REDUCE_NVLS = 2,
  KERNEL_COPY = 3,
  KERNEL_P2P = 4,
  KERNEL_SCALE = 5,
  KERNEL_SIGNAL = 6,
  KERNEL_RING = 7,
  KERNEL_TREE = 8,
  KERNEL_COUNT = 9
};

// RedOp values used by the kernels (sum, prod, max, min); avg and pre-multiplied sums are
// lowered by the host to one of these plus a scale (reference: src/enqueue.cc:2479-2583).
const void* reduceKernelFn(int kernelId, ncclDataType_t type, int op);
bool nvlsReduceSupported(ncclDataType_t type, int op);
const void* ringKernelFn(ncclDataType_t type, int op);
const void* treeKernelFn(ncclDataType_t type, int op);
const void* llReduceKernelFn(ncclDataType_t type, int op);   // all-reduce, reduce-scatter, reduce (a.func)
const void* llReduceBatchKernelFn(ncclDataType_t type, int op);   // takes LLBatchArgs: several all-reduces of one group
const void* llCopyKernelFn();
const void* copyKernelFn();
const void* copyBulkKernelFn();              // same arguments as copyKernelFn: bulk-copy engines, 32 threads per CTA, dynamic shared memory
size_t copyBulkSmemBytes();
const void* p2pKernelFn();
const void* reshardKernelFn();                 // takes ReshardArgs: pulls the runs of a mesh-to-mesh reshard with peer loads
const void* scaleKernelFn(ncclDataType_t type);
const void* localCopyKernelFn(int unroll);   // takes ScaleArgs{src, dst, count = bytes}; unroll 4 or 8
const void* localBulkCopyKernelFn();         // same arguments: one thread per CTA drives cp.async.bulk copies through shared memory
size_t localBulkCopySmemBytes();
const void* signalKernelFn();
const void* waitSignalKernelFn();

struct ScaleArgs {
  const void* src;
  void* dst;
  size_t count;
  unsigned long long scalarBits;   // immediate scalar (element type of the buffer)
  const void* scalarPtr;           // device scalar, read by the kernel when non-null
};

struct OneSignalArgs {
  uint64_t* target;                // peer's counter for (me, sigIdx)
};
struct WaitSignalArgs {
  int nDesc;
  const uint64_t* counter[16];     // my counters to watch
  uint64_t* seen[16];              // private: consumed so far
  uint32_t opCnt[16];
  SyncArgs sync;
  int rank;
};

// Launch with the attributes the data plane wants: optional cooperative co-residency (single-GPU
// emulation), programmatic stream serialisation when `pdl`, remote memory-sync domain.
ncclResult_t launchKernel(const void* fn, dim3 grid, dim3 block, size_t smem, void* argStruct, cudaStream_t stream,
                          bool cooperative, bool pdl = false);

}  // namespace b200
