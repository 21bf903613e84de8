// Shared helpers of the example programs: error checks and a thread-per-GPU launcher.
// The examples follow the usage patterns of the reference's examples/ tree (01_communicators ...
// 06_device_api): each program is a complete user of the public headers and the shared library.
#pragma once
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <functional>
#include <thread>
#include <vector>

#include "nccl.h"

#define CUDA_OK(call)                                                                                 \
  do {                                                                                                \
    cudaError_t e_ = (call);                                                                          \
    if (e_ != cudaSuccess) {                                                                          \
      fprintf(stderr, "%s:%d CUDA error: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_));          \
      exit(2);                                                                                        \
    }                                                                                                 \
  } while (0)

#define NCCL_OK(call)                                                                                 \
  do {                                                                                                \
    ncclResult_t r_ = (call);                                                                         \
    if (r_ != ncclSuccess && r_ != ncclInProgress) {                                                  \
      fprintf(stderr, "%s:%d NCCL error: %s (%s)\n", __FILE__, __LINE__, ncclGetErrorString(r_), ncclGetLastError(nullptr)); \
      exit(3);                                                                                        \
    }                                                                                                 \
  } while (0)

// Number of GPUs the example uses: every visible one, or EXAMPLE_GPUS when that is set.
inline int exampleGpus() {
  int n = 0;
  CUDA_OK(cudaGetDeviceCount(&n));
  if (const char* e = getenv("EXAMPLE_GPUS")) n = std::min(n, atoi(e));
  if (n < 1) { fprintf(stderr, "no GPU visible\n"); exit(2); }
  return n;
}

// Runs body(rank, nRanks, comm) on one thread per GPU, each with its own communicator of one
// shared unique id (the layout of a multi-process job, inside one process).
inline void runThreadPerGpu(int n, const std::function<void(int, int, ncclComm_t)>& body) {
  ncclUniqueId id;
  NCCL_OK(ncclGetUniqueId(&id));
  std::vector<std::thread> th;
  for (int r = 0; r < n; ++r)
    th.emplace_back([=, &body] {
      CUDA_OK(cudaSetDevice(r));
      ncclComm_t comm;
      NCCL_OK(ncclCommInitRank(&comm, n, id, r));
      body(r, n, comm);
      NCCL_OK(ncclCommDestroy(comm));
    });
  for (auto& t : th) t.join();
}
