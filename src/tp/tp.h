// Internal interface between the tensor-parallel host code and its sm_100a kernels.
#pragma once
#include "../kernels/args.h"

namespace b200 {

enum TpMode : int {
  TP_MODE_STORE = 0,    // C = A * W^T, stored locally
  TP_MODE_REDUCE = 1,   // GEMM -> reduce-scatter: partial tiles are added into the owner's fp32 buffer
  TP_MODE_GATHER = 2,   // all-gather -> GEMM: comm CTAs pull remote row blocks while the GEMM runs
};

struct TpGemmArgs {
  void* C;                        // bf16 output [M, ldc] (STORE / GATHER)
  int ldc;
  float* accum[kMaxRanks];        // REDUCE: accum[p] = rank p's fp32 buffer [M / nRanks, N], mapped here
  const void* peerA[kMaxRanks];   // GATHER: peerA[p] = rank p's A buffer [M, K] bf16, mapped here
  uint32_t* blockFlags;           // GATHER: one word per 128-row block of A, set to flagEpoch when landed
  uint32_t flagEpoch;
  int M, N, K;
  int mode;
  int rank, nRanks;
  int gemmCtas;                   // GATHER: CTAs [0, gemmCtas) compute, the rest gather
  SyncArgs sync;
};

const void* tpGemmKernelFn();
const void* tpConvertKernelFn();
size_t tpGemmSmemBytes();
int tpGemmThreads();

}  // namespace b200
