// Host side of the fused tensor-parallel GEMMs: contexts, TMA descriptors, launches.
// See include/nccl_tp.h for the API and src/tp/gemm_sm100.cu for the kernels.
#include "tp.h"

#include <cuda.h>

#include <map>

#include "../comm/device_plane.h"
#include "nccl_tp.h"

using namespace b200;

namespace b200 {
B200_PARAM(TpCommCtas, "B200_TP_COMM_CTAS", 16, "CTAs that gather remote rows in all-gather -> GEMM")
}

struct ncclTpContext {
  ncclComm* comm = nullptr;
  int smCount = 0;
  float* accum = nullptr;          // symmetric fp32 window [maxRows / n, maxCols]
  size_t accumBytes = 0;
  SymWindow* accumWin = nullptr;
  uint32_t* blockFlags = nullptr;  // one word per 128-row block (all-gather -> GEMM)
  size_t maxBlocks = 0;
  uint32_t epoch = 0;
  std::map<void*, SymWindow*> gathered;
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encodeFn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = (EncodeTiledFn)p;
    else (void)cudaGetLastError();
  }
  return fn;
}

// Row-major [rows, K] bf16 tensor, tiles of boxRows x 64 elements with 128-byte swizzle.
static ncclResult_t makeMap(CUtensorMap* map, const void* base, int rows, int K, int boxRows) {
  EncodeTiledFn enc = encodeFn();
  if (!enc) { WARN("cuTensorMapEncodeTiled is not available"); return ncclUnhandledCudaError; }
  if ((uintptr_t)base & 15) { WARN("tensor-parallel GEMM operands must be 16-byte aligned"); return ncclInvalidArgument; }
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)boxRows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { WARN("cuTensorMapEncodeTiled failed (%d)", (int)r); return ncclUnhandledCudaError; }
  return ncclSuccess;
}

static ncclResult_t checkShape(int M, int N, int K, int n) {
  if (M <= 0 || N <= 0 || K <= 0 || M % (128 * n) || N % 256 || K % 64) {
    WARN("tensor-parallel GEMM: M=%d must be a multiple of %d, N=%d of 256, K=%d of 64", M, 128 * n, N, K);
    return ncclInvalidArgument;
  }
  return ncclSuccess;
}

static void fillSyncTp(ncclComm* comm, SyncArgs* s) {
  memset(s, 0, sizeof(*s));
  DevicePlane* dp = comm->devPlane;
  if (comm->nRanks > 1 && dp && dp->resWin) {
    for (int p = 0; p < comm->nRanks; ++p) s->inbox[p] = (uint32_t*)dp->resWin->host.peerPtr[p];
    s->epoch[comm->rank] = dp->epochs;
  }
  s->status[comm->rank] = comm->devStatusDev;
  s->abortFlag = comm->abortFlagDev;
  s->timeoutNs = dp ? dp->timeoutNs : 5000000000ull;
}

static ncclResult_t launchGemm(ncclTpContext* tp, const void* A, const void* W, TpGemmArgs* a, int grid, cudaStream_t stream) {
  static bool attrSet = false;
  if (!attrSet) {
    CUDACHECK(cudaFuncSetAttribute(tpGemmKernelFn(), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tpGemmSmemBytes()));
    attrSet = true;
  }
  CUtensorMap tmA, tmB;
  NCCLCHECK(makeMap(&tmA, A, a->M, a->K, 128));
  NCCLCHECK(makeMap(&tmB, W, a->N, a->K, 256));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(tpGemmThreads());
  cfg.dynamicSmemBytes = tpGemmSmemBytes();
  cfg.stream = stream;
  void* args[3] = {&tmA, &tmB, a};
  cudaError_t e = cudaLaunchKernelExC(&cfg, tpGemmKernelFn(), args);
  if (e != cudaSuccess) { WARN("tensor-parallel GEMM launch failed: %s", cudaGetErrorString(e)); (void)cudaGetLastError(); return ncclUnhandledCudaError; }
  if (tp->comm->devPlane) tp->comm->devPlane->launches++;
  return ncclSuccess;
}

extern "C" {

ncclResult_t ncclTpCreate(ncclComm_t comm, size_t maxRows, size_t maxCols, ncclTp_t* out) {
  if (!out) return ncclInvalidArgument;
  *out = nullptr;
  if (!commValid(comm) || comm->hostOnly) { WARN("ncclTpCreate needs a GPU communicator"); return ncclInvalidArgument; }
  NCCLCHECK(commEnsureReady(comm));
  if (comm->nRanks > 1 && !comm->lsaAll) { WARN("ncclTpCreate: ranks must be able to map each other's memory"); return ncclInvalidUsage; }
  if (comm->compCap < 100) { WARN("ncclTpCreate: the fused GEMM kernels need compute capability 10.0 (found %d)", comm->compCap); return ncclInvalidUsage; }
  ncclTpContext* tp = new ncclTpContext;
  tp->comm = comm;
  int cur = -1;
  CUDACHECK(cudaGetDevice(&cur));
  if (cur != comm->cudaDev) CUDACHECK(cudaSetDevice(comm->cudaDev));
  CUDACHECK(cudaDeviceGetAttribute(&tp->smCount, cudaDevAttrMultiProcessorCount, comm->cudaDev));
  const int n = comm->nRanks;
  tp->accumBytes = (maxRows / n) * maxCols * sizeof(float);
  if (tp->accumBytes) {
    NCCLCHECK(memAlloc((void**)&tp->accum, tp->accumBytes, comm->cudaDev));
    if (n > 1) {
      NCCLCHECK(symWindowRegister(comm, tp->accum, tp->accumBytes, &tp->accumWin, NCCL_WIN_COLL_SYMMETRIC));
      if (!tp->accumWin->symmetric) { WARN("ncclTpCreate: accumulation window could not be mapped by the peers"); return ncclInternalError; }
    }
  }
  tp->maxBlocks = maxRows / 128 + 1;
  CUDACHECK(cudaMalloc(&tp->blockFlags, tp->maxBlocks * sizeof(uint32_t)));
  CUDACHECK(cudaMemset(tp->blockFlags, 0, tp->maxBlocks * sizeof(uint32_t)));
  if (cur != comm->cudaDev) cudaSetDevice(cur);
  *out = tp;
  return ncclSuccess;
}

ncclResult_t ncclTpDestroy(ncclTp_t tp) {
  if (!tp) return ncclSuccess;
  cudaDeviceSynchronize();
  for (auto& kv : tp->gathered) {
    if (kv.second) symWindowDeregister(tp->comm, kv.second);
    memFree(kv.first);
  }
  if (tp->accumWin) symWindowDeregister(tp->comm, tp->accumWin);
  if (tp->accum) memFree(tp->accum);
  if (tp->blockFlags) cudaFree(tp->blockFlags);
  delete tp;
  return ncclSuccess;
}

ncclResult_t ncclTpAllocGathered(ncclTp_t tp, size_t rows, size_t cols, void** ptr) {
  if (!tp || !ptr) return ncclInvalidArgument;
  void* p = nullptr;
  NCCLCHECK(memAlloc(&p, rows * cols * 2, tp->comm->cudaDev));
  SymWindow* w = nullptr;
  if (tp->comm->nRanks > 1) {
    NCCLCHECK(symWindowRegister(tp->comm, p, rows * cols * 2, &w, NCCL_WIN_COLL_SYMMETRIC));
    if (!w->symmetric) { WARN("ncclTpAllocGathered: window could not be mapped by the peers"); return ncclInternalError; }
  }
  tp->gathered[p] = w;
  *ptr = p;
  return ncclSuccess;
}

ncclResult_t ncclTpFreeGathered(ncclTp_t tp, void* ptr) {
  if (!tp) return ncclInvalidArgument;
  auto it = tp->gathered.find(ptr);
  if (it == tp->gathered.end()) return ncclInvalidArgument;
  cudaDeviceSynchronize();
  if (it->second) symWindowDeregister(tp->comm, it->second);
  memFree(ptr);
  tp->gathered.erase(it);
  return ncclSuccess;
}

ncclResult_t ncclTpGemm(ncclTp_t tp, const void* A, const void* W, void* C, int M, int N, int K, cudaStream_t stream) {
  if (!tp || !A || !W || !C) return ncclInvalidArgument;
  NCCLCHECK(checkShape(M, N, K, 1));
  TpGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.C = C; a.ldc = N; a.M = M; a.N = N; a.K = K;
  a.mode = TP_MODE_STORE;
  a.rank = tp->comm->rank; a.nRanks = tp->comm->nRanks;
  fillSyncTp(tp->comm, &a.sync);
  int tiles = (M / 128) * (N / 256);
  return launchGemm(tp, A, W, &a, std::min(tp->smCount, tiles), stream);
}

ncclResult_t ncclTpGemmReduceScatter(ncclTp_t tp, const void* A, const void* W, void* out, int M, int N, int K, cudaStream_t stream) {
  if (!tp || !A || !W || !out) return ncclInvalidArgument;
  ncclComm* comm = tp->comm;
  const int n = comm->nRanks;
  NCCLCHECK(checkShape(M, N, K, n));
  NCCLCHECK(devPlaneCheckStatus(comm));
  if (n == 1) return ncclTpGemm(tp, A, W, out, M, N, K, stream);
  const size_t need = (size_t)(M / n) * N * sizeof(float);
  if (need > tp->accumBytes) { WARN("ncclTpGemmReduceScatter: %d x %d exceeds the context's accumulation window", M, N); return ncclInvalidArgument; }
  CUDACHECK(cudaMemsetAsync(tp->accum, 0, need, stream));
  TpGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.M = M; a.N = N; a.K = K;
  a.mode = TP_MODE_REDUCE;
  a.rank = comm->rank; a.nRanks = n;
  for (int p = 0; p < n; ++p) a.accum[p] = (float*)tp->accumWin->host.peerPtr[p];
  fillSyncTp(comm, &a.sync);
  int tiles = (M / 128) * (N / 256);
  NCCLCHECK(launchGemm(tp, A, W, &a, std::min(tp->smCount, tiles), stream));
  // kernel completion implies that every rank's partial sums have landed here
  size_t count = (size_t)(M / n) * N;
  int ctas = (int)std::min<size_t>((count / 8 + 255) / 256, (size_t)tp->smCount * 8);
  const float* acc = tp->accum;
  void* args[3] = {(void*)&acc, &out, &count};
  CUDACHECK(cudaLaunchKernel(tpConvertKernelFn(), dim3(ctas), dim3(256), args, 0, stream));
  if (comm->devPlane) comm->devPlane->launches++;
  return ncclSuccess;
}

ncclResult_t ncclTpAllGatherGemm(ncclTp_t tp, void* gatheredA, const void* W, void* C, int M, int N, int K, cudaStream_t stream) {
  if (!tp || !gatheredA || !W || !C) return ncclInvalidArgument;
  ncclComm* comm = tp->comm;
  const int n = comm->nRanks;
  NCCLCHECK(checkShape(M, N, K, n));
  NCCLCHECK(devPlaneCheckStatus(comm));
  if (n == 1) return ncclTpGemm(tp, gatheredA, W, C, M, N, K, stream);
  auto it = tp->gathered.find(gatheredA);
  if (it == tp->gathered.end() || !it->second) { WARN("ncclTpAllGatherGemm: the activation buffer must come from ncclTpAllocGathered"); return ncclInvalidArgument; }
  if ((size_t)(M / 128) > tp->maxBlocks) { WARN("ncclTpAllGatherGemm: M=%d exceeds the context's row limit", M); return ncclInvalidArgument; }
  TpGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.C = C; a.ldc = N; a.M = M; a.N = N; a.K = K;
  a.mode = TP_MODE_GATHER;
  a.rank = comm->rank; a.nRanks = n;
  for (int p = 0; p < n; ++p) a.peerA[p] = it->second->host.peerPtr[p];
  a.blockFlags = tp->blockFlags;
  a.flagEpoch = ++tp->epoch;
  int commCtas = (int)std::max<int64_t>(1, std::min<int64_t>(paramTpCommCtas(), tp->smCount / 4));
  a.gemmCtas = tp->smCount - commCtas;
  fillSyncTp(comm, &a.sync);
  return launchGemm(tp, gatheredA, W, &a, tp->smCount, stream);
}

}  // extern "C"
