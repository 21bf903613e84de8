// All-reduce over N buffers of one GPU with working memory in a fixed device array (see the header
// for who needs it and for the rules of use). The kernel is the flagged-line one-shot all-reduce of
// reduce.cu with a smaller line capacity and with its epoch and status words inside the same array.
#include "noalloc_allreduce.h"

#include <mutex>

#include "common.cuh"
#include "launch.h"
#include "../core/core.h"

namespace b200 {

constexpr int kNaLines = 512;                                          // 8 payload bytes each
constexpr size_t kNaRegionBytes = (size_t)2 * kMaxRanks * kNaLines * 16;  // [parity][source][line]
constexpr size_t kNaCtrlBytes = 256;                                   // epoch, finished CTAs, status record
constexpr size_t kNaRankBytes = kNaRegionBytes + kNaCtrlBytes;
static_assert(kNaRankBytes * B200_NOALLOC_MAX_RANKS == B200_NOALLOC_SCRATCH_BYTES, "scratch size in the header is stale");
static_assert(kNaLines * 8 == B200_NOALLOC_MAX_BYTES, "payload limit in the header is stale");

// Zero-initialised when the module is loaded on a device. In host code this name is only a
// stand-in for the symbol: the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char gNoAllocScratch[B200_NOALLOC_SCRATCH_BYTES];

struct NoAllocArgs {
  int nRanks;
  size_t count;
  const void* send[kMaxRanks];
  void* recv[kMaxRanks];
  unsigned char* scratch;
  unsigned long long timeoutNs;
};

template <typename T>
__global__ void __launch_bounds__(kCtaThreads, 1) noAllocAllReduceKernel(const __grid_constant__ NoAllocArgs a) {
  const int rank = blockIdx.y;
  const int n = a.nRanks;
  constexpr int N = 8 / sizeof(T);
  unsigned char* mine = a.scratch + (size_t)rank * kNaRankBytes;
  uint32_t* ctrl = (uint32_t*)(mine + kNaRegionBytes);   // [16..19] status record of this rank
  // One epoch for the whole call, kept in the control block of rank 0 whatever nRanks is: every
  // CTA of the grid reads it here and the last CTA of the grid to finish publishes the next value.
  // (An epoch per rank would let ranks that sat out a call with fewer ranks fall behind.)
  uint32_t* call = (uint32_t*)(a.scratch + kNaRegionBytes);   // [0] epoch, [1] finished CTAs
  SyncArgs sync;
  sync.abortFlag = nullptr;
  sync.timeoutNs = a.timeoutNs;
  WaitCtx w{&sync, ctrl + 16};
  uint32_t epoch = call[0] + 1;
  if (epoch == 0) epoch = 1;
  const int parity = epoch & 1;
  const size_t bytes = a.count * sizeof(T);
  const size_t nLines = (bytes + 7) / 8;
  const char* in = (const char*)a.send[rank];
  char* out = (char*)a.recv[rank];
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  auto region = [&](int p, int s) { return (char*)a.scratch + (size_t)p * kNaRankBytes + ((size_t)(parity * kMaxRanks + s) * kNaLines) * 16; };
  auto load8 = [&](size_t l) {
    const char* p = in + l * 8;
    size_t valid = bytes - l * 8;
    if (valid >= 8 && ((uintptr_t)p & 7) == 0) return *(const uint64_t*)p;
    uint64_t v = 0;
    for (size_t b = 0; b < 8 && b < valid; ++b) v |= (uint64_t)(uint8_t)p[b] << (8 * b);
    return v;
  };
  for (size_t l = (size_t)blockIdx.x * blockDim.x + threadIdx.x; l < nLines; l += stride) {
    uint64_t d = load8(l);
    uint4 line = make_uint4((uint32_t)d, epoch, (uint32_t)(d >> 32), epoch);
    for (int p = 0; p < n; ++p)
      if (p != rank) stVolatile16(region(p, rank) + l * 16, line);
  }
  bool ok = true;
  for (size_t l = (size_t)blockIdx.x * blockDim.x + threadIdx.x; l < nLines && ok; l += stride) {
    float acc[N];
    for (int s = 0; s < n; ++s) {
      uint64_t d;
      if (s == rank) {
        d = load8(l);
      } else {
        const char* slot = region(rank, s) + l * 16;
        uint4 v = ldVolatile16(slot);
        if (v.y != epoch || v.w != epoch)
          ok = boundedWait(w, WAIT_LL, (uint32_t)s, epoch, [&] { v = ldVolatile16(slot); return v.y == epoch && v.w == epoch; });
        if (!ok) break;
        d = (uint64_t)v.x | ((uint64_t)v.z << 32);
      }
      union { uint64_t u; T e[N]; } cv;
      cv.u = d;
#pragma unroll
      for (int k = 0; k < N; ++k) {
        float x = Elem<T>::ld(cv.e[k]);
        acc[k] = s == 0 ? x : acc[k] + x;
      }
    }
    if (!ok) break;
    union { uint64_t u; T e[N]; } res;
#pragma unroll
    for (int k = 0; k < N; ++k) res.e[k] = Elem<T>::st(acc[k]);
    char* p = out + l * 8;
    size_t valid = bytes - l * 8;
    if (valid >= 8 && ((uintptr_t)p & 7) == 0) *(uint64_t*)p = res.u;
    else for (size_t b = 0; b < 8 && b < valid; ++b) p[b] = (char)(res.u >> (8 * b));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t done = atomicAdd(&call[1], 1u);
    if (done == gridDim.x * gridDim.y - 1) {
      call[1] = 0;
      call[0] = epoch;
    }
  }
}

static std::mutex gNaLock;
static unsigned char* gNaPtr[64];   // device address of the scratch array, per device

}  // namespace b200

using namespace b200;

extern "C" ncclResult_t b200NoAllocAllReduce(int nRanks, ncclDataType_t type, size_t count, const void* const* send, void* const* recv,
                                             cudaStream_t stream) {
  if (nRanks < 1 || nRanks > B200_NOALLOC_MAX_RANKS) { WARN("b200NoAllocAllReduce: nRanks %d is outside [1, %d]", nRanks, B200_NOALLOC_MAX_RANKS); return ncclInvalidArgument; }
  if (type != ncclFloat32 && type != ncclFloat16 && type != ncclBfloat16) { WARN("b200NoAllocAllReduce: only fp32, fp16 and bf16 are supported"); return ncclInvalidArgument; }
  const size_t es = type == ncclFloat32 ? 4 : 2;
  if (count > B200_NOALLOC_MAX_BYTES / es) {   // compared in elements: count * es could wrap
    WARN("b200NoAllocAllReduce: %zu elements of %zu bytes per buffer exceed the fixed scratch (limit %d bytes)", count, es, B200_NOALLOC_MAX_BYTES);
    return ncclInvalidArgument;
  }
  if (!send || !recv) return ncclInvalidArgument;
  for (int r = 0; r < nRanks; ++r) if (count && (!send[r] || !recv[r])) { WARN("b200NoAllocAllReduce: null buffer for rank %d", r); return ncclInvalidArgument; }
  if (count == 0) return ncclSuccess;
  int dev = -1;
  CUDACHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return ncclInvalidUsage;
  unsigned char* scratch = nullptr;
  {
    // set-up, once per device, with that device current: resolve the symbol to its device address
    std::lock_guard<std::mutex> g(gNaLock);
    if (!gNaPtr[dev]) {
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, gNoAllocScratch);
      if (e != cudaSuccess || !p) {
        WARN("b200NoAllocAllReduce: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        (void)cudaGetLastError();
        return ncclUnhandledCudaError;
      }
      gNaPtr[dev] = (unsigned char*)p;
    }
    scratch = gNaPtr[dev];
  }
  NoAllocArgs a;
  memset(&a, 0, sizeof(a));
  a.nRanks = nRanks;
  a.count = count;
  for (int r = 0; r < nRanks; ++r) { a.send[r] = send[r]; a.recv[r] = recv[r]; }
  a.scratch = scratch;
  a.timeoutNs = 2000000000ull;
  // the status record of every rank must read "ok" when the kernel starts
  for (int r = 0; r < nRanks; ++r)
    CUDACHECK(cudaMemsetAsync(scratch + (size_t)r * kNaRankBytes + kNaRegionBytes + 64, 0, 16, stream));
  const void* fn = type == ncclFloat32 ? (const void*)noAllocAllReduceKernel<float>
                 : type == ncclFloat16 ? (const void*)noAllocAllReduceKernel<__half> : (const void*)noAllocAllReduceKernel<__nv_bfloat16>;
  NCCLCHECK(launchKernel(fn, dim3(1, nRanks), dim3(kCtaThreads), 0, &a, stream, /*cooperative=*/true));
  CUDACHECK(cudaStreamSynchronize(stream));
  for (int r = 0; r < nRanks; ++r) {
    uint32_t st[4] = {0, 0, 0, 0};
    CUDACHECK(cudaMemcpy(st, scratch + (size_t)r * kNaRankBytes + kNaRegionBytes + 64, 16, cudaMemcpyDeviceToHost));
    if (st[0] != DEV_OK) { WARN("b200NoAllocAllReduce: rank %d gave up waiting for rank %u", r, st[2]); return ncclTimeout; }
  }
  return ncclSuccess;
}
