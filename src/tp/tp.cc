// Host side of the fused tensor-parallel GEMMs: contexts, TMA descriptors, launches.
// See include/nccl_tp.h for the API and src/tp/gemm_sm100.cu for the kernels.
#include "tp.h"

#include <cuda.h>

#include <map>

#include "../comm/device_plane.h"
#include "nccl_tp.h"

using namespace b200;

namespace b200 {
B200_PARAM(TpCommCtas, "B200_TP_COMM_CTAS", 0, "CTAs that gather remote rows in all-gather -> GEMM (0: 4 for two ranks, 8 up to four, 16 beyond)")
B200_PARAM(TpPair, "B200_TP_PAIR", 1, "bf16 GEMM on CTA pairs (256 x 256 tiles, tcgen05 cta_group::2) when the row count allows")
}

struct ncclTpContext {
  ncclComm* comm = nullptr;
  int smCount = 0;
  int pairClusters = 0;   // clusters of the CTA-pair GEMM kernel that can be resident at once (0: unavailable)
  void* accum = nullptr;           // symmetric staging window: bf16 [n sources][maxRows / n][maxCols]
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

// Row-major [rows, K] tensor of bf16 (elemBytes 2) or fp8 (1), tiles of boxRows x 128 bytes with 128-byte swizzle.
// Comm CTAs of all-gather -> GEMM: each moves about 33 GB/s (128 KiB of loads in flight over NVLink, measured at two
// ranks); the remote share of the rows and how early the first remote chunk is needed both grow with the number of ranks.
static int tpCommCtas(const ncclTpContext* tp, int nRanks);

static ncclResult_t makeMap(CUtensorMap* map, const void* base, int rows, int K, int boxRows, int elemBytes = 2) {
  EncodeTiledFn enc = encodeFn();
  if (!enc) { WARN("cuTensorMapEncodeTiled is not available"); return ncclUnhandledCudaError; }
  if ((uintptr_t)base & 15) { WARN("tensor-parallel GEMM operands must be 16-byte aligned"); return ncclInvalidArgument; }
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * elemBytes};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elemBytes), (cuuint32_t)boxRows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, elemBytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { WARN("cuTensorMapEncodeTiled failed (%d)", (int)r); return ncclUnhandledCudaError; }
  return ncclSuccess;
}

static int tpCommCtas(const ncclTpContext* tp, int nRanks) {
  int64_t want = paramTpCommCtas();
  if (want <= 0) want = nRanks <= 2 ? 4 : nRanks <= 4 ? 8 : 16;
  return (int)std::max<int64_t>(1, std::min<int64_t>(want, tp->smCount / 4));
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

// Launches the bf16 GEMM kernel in the mode of `a`. Grid: one CTA per SM (fewer when there are fewer
// tiles); in all-gather mode the last CTAs are the comm CTAs. The CTA-pair kernel runs when enabled,
// when its clusters fit and when every rank's rows split into 256-row tiles.
static ncclResult_t launchGemm(ncclTpContext* tp, const void* A, const void* W, TpGemmArgs* a, cudaStream_t stream) {
  const int n = a->nRanks;
  const bool fused = n > 1 && a->mode != TP_MODE_STORE;
  const bool gather = fused && a->mode == TP_MODE_GATHER;
  const bool pair = paramTpPair() != 0 && tp->pairClusters > 0 && a->M % (256 * (fused ? n : 1)) == 0;
  int commCtas = gather ? tpCommCtas(tp, n) : 0;
  int grid;
  if (pair) {
    commCtas = (commCtas + 1) & ~1;   // both CTAs of a cluster have the same role
    const int tiles = (a->M / 256) * (a->N / 256);
    const int pairs = std::max(1, std::min(tp->pairClusters - commCtas / 2, tiles));
    a->gemmCtas = 2 * pairs;
    grid = 2 * pairs + commCtas;
  } else {
    const int tiles = (a->M / 128) * (a->N / 256);
    grid = gather ? tp->smCount : std::min(tp->smCount, tiles);
    a->gemmCtas = grid - commCtas;
  }
  CUtensorMap tmA, tmB;
  NCCLCHECK(makeMap(&tmA, A, a->M, a->K, 128));
  NCCLCHECK(makeMap(&tmB, W, a->N, a->K, pair ? 128 : 256));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(pair ? tpGemmPairThreads() : tpGemmThreads());
  cfg.dynamicSmemBytes = pair ? tpGemmPairSmemBytes() : tpGemmSmemBytes();
  cfg.stream = stream;
  void* args[3] = {&tmA, &tmB, a};
  cudaError_t e = cudaLaunchKernelExC(&cfg, pair ? tpGemmPairKernelFn() : tpGemmKernelFn(), args);
  if (e != cudaSuccess) { WARN("tensor-parallel GEMM launch failed: %s", cudaGetErrorString(e)); (void)cudaGetLastError(); return ncclUnhandledCudaError; }
  if (tp->comm->devPlane) tp->comm->devPlane->launches++;
  return ncclSuccess;
}

static ncclResult_t launchGemmFp8(ncclTpContext* tp, const void* A, const void* W, TpGemmArgs* a, int grid, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  NCCLCHECK(makeMap(&tmA, A, a->M, a->K, 128, 1));
  NCCLCHECK(makeMap(&tmB, W, a->N, a->K, 256, 1));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(tpGemmFp8Threads());
  cfg.dynamicSmemBytes = tpGemmFp8SmemBytes();
  cfg.stream = stream;
  void* args[3] = {&tmA, &tmB, a};
  cudaError_t e = cudaLaunchKernelExC(&cfg, tpGemmFp8KernelFn(), args);
  if (e != cudaSuccess) { WARN("fp8 tensor-parallel GEMM launch failed: %s", cudaGetErrorString(e)); (void)cudaGetLastError(); return ncclUnhandledCudaError; }
  if (tp->comm->devPlane) tp->comm->devPlane->launches++;
  return ncclSuccess;
}

static ncclResult_t checkShapeFp8(int M, int N, int K, int n) {
  if (M <= 0 || N <= 0 || K <= 0 || M % (128 * n) || N % 256 || K % 128) {
    WARN("fp8 tensor-parallel GEMM: M=%d must be a multiple of %d, N=%d of 256, K=%d of 128", M, 128 * n, N, K);
    return ncclInvalidArgument;
  }
  return ncclSuccess;
}

extern "C" {

ncclResult_t ncclTpQuantizeFp8(ncclTp_t tp, const void* x, void* q, float* scales, int rows, int K, int blockRows, cudaStream_t stream) {
  if (!tp || !x || !q || !scales || rows <= 0 || K <= 0 || K % 128 || (blockRows != 1 && blockRows != 128)) return ncclInvalidArgument;
  if (blockRows == 128 && rows % 128) return ncclInvalidArgument;
  if (((uintptr_t)x & 7) || ((uintptr_t)q & 3)) return ncclInvalidArgument;
  void* args[5] = {(void*)&x, &q, &scales, &rows, &K};
  if (blockRows == 1) {
    size_t warps = (size_t)rows * (K / 128);
    int ctas = (int)std::min<size_t>((warps + 7) / 8, (size_t)tp->smCount * 16);
    CUDACHECK(cudaLaunchKernel(tpQuantRowsKernelFn(), dim3(std::max(ctas, 1)), dim3(256), args, 0, stream));
  } else {
    int blocks = (rows / 128) * (K / 128);
    CUDACHECK(cudaLaunchKernel(tpQuantBlocksKernelFn(), dim3(std::min(blocks, tp->smCount * 8)), dim3(256), args, 0, stream));
  }
  if (tp->comm->devPlane) tp->comm->devPlane->launches++;
  return ncclSuccess;
}

ncclResult_t ncclTpGemmFp8(ncclTp_t tp, const void* A, const float* scaleA, const void* W, const float* scaleW, void* C, int M, int N, int K, cudaStream_t stream) {
  if (!tp || !A || !W || !C || !scaleA || !scaleW) return ncclInvalidArgument;
  NCCLCHECK(checkShapeFp8(M, N, K, 1));
  TpGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.C = C; a.ldc = N; a.M = M; a.N = N; a.K = K;
  a.mode = TP_MODE_STORE;
  a.rank = tp->comm->rank; a.nRanks = tp->comm->nRanks;
  a.scaleA = scaleA; a.scaleW = scaleW;
  fillSyncTp(tp->comm, &a.sync);
  int tiles = (M / 128) * (N / 256);
  return launchGemmFp8(tp, A, W, &a, std::min(tp->smCount, tiles), stream);
}

ncclResult_t ncclTpGemmReduceScatterFp8(ncclTp_t tp, const void* A, const float* scaleA, const void* W, const float* scaleW, void* out, int M, int N, int K,
                                        cudaStream_t stream) {
  if (!tp || !A || !W || !out || !scaleA || !scaleW) return ncclInvalidArgument;
  ncclComm* comm = tp->comm;
  const int n = comm->nRanks;
  NCCLCHECK(checkShapeFp8(M, N, K, n));
  NCCLCHECK(devPlaneCheckStatus(comm));
  if (n > 1) NCCLCHECK(devPlaneOrderStreams(comm, stream));   // the fused kernels use the communicator's barrier slots: one kernel of a communicator at a time
  if (n == 1) return ncclTpGemmFp8(tp, A, scaleA, W, scaleW, out, M, N, K, stream);
  const size_t need = (size_t)M * N * 2;
  if (need > tp->accumBytes) { WARN("ncclTpGemmReduceScatterFp8: %d x %d exceeds the context's staging window", M, N); return ncclInvalidArgument; }
  TpGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.M = M; a.N = N; a.K = K;
  a.mode = TP_MODE_REDUCE;
  a.rank = comm->rank; a.nRanks = n;
  a.scaleA = scaleA; a.scaleW = scaleW;
  for (int p = 0; p < n; ++p) a.partial[p] = tp->accumWin->host.peerPtr[p];
  fillSyncTp(comm, &a.sync);
  int tiles = (M / 128) * (N / 256);
  NCCLCHECK(launchGemmFp8(tp, A, W, &a, std::min(tp->smCount, tiles), stream));
  size_t count = (size_t)(M / n) * N;
  int ctas = (int)std::min<size_t>((count / 8 + 255) / 256, (size_t)tp->smCount * 8);
  const void* staged = tp->accum;
  int nSources = n;
  void* args[4] = {(void*)&staged, &out, &count, &nSources};
  CUDACHECK(cudaLaunchKernel(tpReduceKernelFn(), dim3(ctas), dim3(256), args, 0, stream));
  if (comm->devPlane) comm->devPlane->launches++;
  return ncclSuccess;
}

ncclResult_t ncclTpAllocGatheredFp8(ncclTp_t tp, size_t rows, size_t cols, void** q, float** scales) {
  if (!tp || !q || !scales || cols % 128) return ncclInvalidArgument;
  // one window: rows x cols bytes of e4m3, then cols/128 x rows fp32 scales
  const size_t qBytes = (rows * cols + 255) / 256 * 256;
  const size_t bytes = qBytes + (cols / 128) * rows * sizeof(float);
  void* p = nullptr;
  NCCLCHECK(memAlloc(&p, bytes, tp->comm->cudaDev));
  SymWindow* w = nullptr;
  if (tp->comm->nRanks > 1) {
    NCCLCHECK(symWindowRegister(tp->comm, p, bytes, &w, NCCL_WIN_COLL_SYMMETRIC));
    if (!w->symmetric) { WARN("ncclTpAllocGatheredFp8: window could not be mapped by the peers"); return ncclInternalError; }
  }
  tp->gathered[p] = w;
  // activations belong to the caller: a suspend saves them to host memory and a resume brings them back
  memTrack(tp->comm, p, bytes, MEM_OFFLOAD, "gathered activations (fp8)", tp->comm->nRanks > 1 ? &tp->gathered[p] : nullptr, NCCL_WIN_COLL_SYMMETRIC);
  *q = p;
  *scales = (float*)((char*)p + qBytes);
  return ncclSuccess;
}

ncclResult_t ncclTpAllGatherGemmFp8(ncclTp_t tp, void* gatheredA, const void* W, const float* scaleW, void* C, int M, int N, int K, cudaStream_t stream) {
  if (!tp || !gatheredA || !W || !scaleW || !C) return ncclInvalidArgument;
  ncclComm* comm = tp->comm;
  const int n = comm->nRanks;
  NCCLCHECK(checkShapeFp8(M, N, K, n));
  NCCLCHECK(devPlaneCheckStatus(comm));
  const size_t scaleOffset = ((size_t)M * K + 255) / 256 * 256;
  if (n == 1) return ncclTpGemmFp8(tp, gatheredA, (const float*)((char*)gatheredA + scaleOffset), W, scaleW, C, M, N, K, stream);
  auto it = tp->gathered.find(gatheredA);
  if (it == tp->gathered.end() || !it->second) { WARN("ncclTpAllGatherGemmFp8: the activation buffer must come from ncclTpAllocGatheredFp8"); return ncclInvalidArgument; }
  if ((size_t)(M / 128) > tp->maxBlocks) { WARN("ncclTpAllGatherGemmFp8: M=%d exceeds the context's row limit", M); return ncclInvalidArgument; }
  TpGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.C = C; a.ldc = N; a.M = M; a.N = N; a.K = K;
  a.mode = TP_MODE_GATHER;
  a.rank = comm->rank; a.nRanks = n;
  for (int p = 0; p < n; ++p) a.peerA[p] = it->second->host.peerPtr[p];
  a.scaleOffset = scaleOffset;
  a.scaleW = scaleW;
  a.blockFlags = tp->blockFlags;
  a.flagEpoch = ++tp->epoch;
  int commCtas = tpCommCtas(tp, n);
  a.gemmCtas = tp->smCount - commCtas;
  fillSyncTp(comm, &a.sync);
  return launchGemmFp8(tp, gatheredA, W, &a, tp->smCount, stream);
}

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
  // function attributes are per device: set them here, with this context's device current, not once per process
  CUDACHECK(cudaFuncSetAttribute(tpGemmKernelFn(), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tpGemmSmemBytes()));
  CUDACHECK(cudaFuncSetAttribute(tpGemmFp8KernelFn(), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tpGemmFp8SmemBytes()));
  {
    // how many clusters of two CTAs of the pair kernel the device can hold at once: the grid never exceeds it,
    // because its CTAs wait for one another (comm CTAs, cross-GPU barriers)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tp->smCount & ~1);
    cfg.blockDim = dim3(tpGemmPairThreads());
    cfg.dynamicSmemBytes = tpGemmPairSmemBytes();
    int clusters = 0;
    if (cudaFuncSetAttribute(tpGemmPairKernelFn(), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tpGemmPairSmemBytes()) == cudaSuccess &&
        cudaOccupancyMaxActiveClusters(&clusters, tpGemmPairKernelFn(), &cfg) == cudaSuccess)
      tp->pairClusters = std::min(clusters, tp->smCount / 2);
    else
      (void)cudaGetLastError();
    INFO(SUB_INIT, "tensor-parallel GEMM: %d SMs, %d resident CTA pairs", tp->smCount, tp->pairClusters);
  }
  const int n = comm->nRanks;
  tp->accumBytes = n > 1 ? maxRows * maxCols * 2 : 0;   // bf16 staging: one [maxRows / n, maxCols] slot per source rank
  if (tp->accumBytes) {
    NCCLCHECK(memAlloc((void**)&tp->accum, tp->accumBytes, comm->cudaDev));
    if (n > 1) {
      NCCLCHECK(symWindowRegister(comm, tp->accum, tp->accumBytes, &tp->accumWin, NCCL_WIN_COLL_SYMMETRIC));
      if (!tp->accumWin->symmetric) { WARN("ncclTpCreate: accumulation window could not be mapped by the peers"); return ncclInternalError; }
    }
    memTrack(comm, tp->accum, tp->accumBytes, MEM_SCRATCH, "tensor-parallel partial sums", n > 1 ? &tp->accumWin : nullptr, NCCL_WIN_COLL_SYMMETRIC);
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
  if (tp->accum) memUntrack(tp->comm, tp->accum);
  for (auto& kv : tp->gathered) memUntrack(tp->comm, kv.first);
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
  memTrack(tp->comm, p, rows * cols * 2, MEM_OFFLOAD, "gathered activations", tp->comm->nRanks > 1 ? &tp->gathered[p] : nullptr, NCCL_WIN_COLL_SYMMETRIC);
  *ptr = p;
  return ncclSuccess;
}

ncclResult_t ncclTpFreeGathered(ncclTp_t tp, void* ptr) {
  if (!tp) return ncclInvalidArgument;
  auto it = tp->gathered.find(ptr);
  if (it == tp->gathered.end()) return ncclInvalidArgument;
  cudaDeviceSynchronize();
  memUntrack(tp->comm, ptr);
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
  return launchGemm(tp, A, W, &a, stream);
}

ncclResult_t ncclTpGemmReduceScatter(ncclTp_t tp, const void* A, const void* W, void* out, int M, int N, int K, cudaStream_t stream) {
  if (!tp || !A || !W || !out) return ncclInvalidArgument;
  ncclComm* comm = tp->comm;
  const int n = comm->nRanks;
  NCCLCHECK(checkShape(M, N, K, n));
  NCCLCHECK(devPlaneCheckStatus(comm));
  if (n > 1) NCCLCHECK(devPlaneOrderStreams(comm, stream));   // the fused kernels use the communicator's barrier slots: one kernel of a communicator at a time
  if (n == 1) return ncclTpGemm(tp, A, W, out, M, N, K, stream);
  const size_t need = (size_t)M * N * 2;
  if (need > tp->accumBytes) { WARN("ncclTpGemmReduceScatter: %d x %d exceeds the context's staging window", M, N); return ncclInvalidArgument; }
  TpGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.M = M; a.N = N; a.K = K;
  a.mode = TP_MODE_REDUCE;
  a.rank = comm->rank; a.nRanks = n;
  for (int p = 0; p < n; ++p) a.partial[p] = tp->accumWin->host.peerPtr[p];
  fillSyncTp(comm, &a.sync);
  NCCLCHECK(launchGemm(tp, A, W, &a, stream));
  // kernel completion implies that every rank's partial tiles have landed in this rank's staging slots
  size_t count = (size_t)(M / n) * N;
  int ctas = (int)std::min<size_t>((count / 8 + 255) / 256, (size_t)tp->smCount * 8);
  const void* staged = tp->accum;
  int nSources = n;
  void* args[4] = {(void*)&staged, &out, &count, &nSources};
  CUDACHECK(cudaLaunchKernel(tpReduceKernelFn(), dim3(ctas), dim3(256), args, 0, stream));
  if (comm->devPlane) comm->devPlane->launches++;
  return ncclSuccess;
}

ncclResult_t ncclTpAllGatherGemm(ncclTp_t tp, void* gatheredA, const void* W, void* C, int M, int N, int K, cudaStream_t stream) {
  if (!tp || !gatheredA || !W || !C) return ncclInvalidArgument;
  ncclComm* comm = tp->comm;
  const int n = comm->nRanks;
  NCCLCHECK(checkShape(M, N, K, n));
  NCCLCHECK(devPlaneCheckStatus(comm));
  if (n > 1) NCCLCHECK(devPlaneOrderStreams(comm, stream));   // the fused kernels use the communicator's barrier slots: one kernel of a communicator at a time
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
  fillSyncTp(comm, &a.sync);
  return launchGemm(tp, gatheredA, W, &a, stream);
}

}  // extern "C"
