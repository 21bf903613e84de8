// Kernels written against the public device API (nccl_device.h) only: they serve as its tests
// and as the fused all-reduce + residual + RMSNorm building block of tensor-parallel decoders.
//   b200DevApiAllReduce   in-place-capable sum all-reduce of a window slice: every CTA owns one
//                         LSA barrier; each pack is loaded from all peers (or through
//                         multimem.ld_reduce) and stored to all peers (or through multimem.st).
//   b200DevApiArRmsNorm   x = sum over ranks of partial[t,:] + residual[t,:]; residual <- x;
//                         out <- x * rsqrt(mean(x^2) + eps) * weight. One-shot (every rank reduces
//                         every row; peer loads or multimem) or two-shot (rows dealt to ranks, the
//                         owner stores residual and out to every rank).
//   b200DevApiLLSum       low-latency all-to-all session: two floats per slot summed over ranks.
// Reference parity: examples/06_device_api (LSA / multimem all-reduce samples) and
// contrib/nccl_ubx allreduce_2shot_* with residual and RMSNorm epilogue.
#include <cuda_bf16.h>

#include "nccl_device.h"

namespace {

constexpr int kThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kThreads) devApiAllReduceKernel(ncclDevComm_t dc, ncclWindow_t sendWin, size_t sendOff, ncclWindow_t recvWin,
                                                                   size_t recvOff, size_t count, int multimem, int* status) {
  using V = nccl_device::Vec16<T>;
  ncclCoopCta cta;
  ncclLsaBarrierSession<ncclCoopCta> bar(cta, dc, ncclTeamLsa(dc), blockIdx.x);
  if (bar.sync(0, false, false) != ncclSuccess) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    bar.finish();
    return;
  }
  const int n = dc.lsaSize;
  const size_t packs = count / V::N;   // the host checks count % V::N == 0
  const size_t perRank = (packs + n - 1) / n;
  const size_t lo = min(packs, perRank * dc.lsaRank), hi = min(packs, lo + perRank);
  const char* mcIn = (const char*)ncclGetMultimemPointer(sendWin, sendOff);
  char* mcOut = (char*)ncclGetMultimemPointer(recvWin, recvOff);
  for (size_t i = lo + (size_t)blockIdx.x * kThreads + threadIdx.x; i < hi; i += (size_t)gridDim.x * kThreads) {
    uint4 r;
    if (multimem) {
      r = V::mcLoad(mcIn + i * 16);
      ncclMultimemStore16(mcOut + i * 16, r);
    } else {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int p = 0; p < n; ++p) V::add(acc, *(const uint4*)((const char*)ncclGetLsaPointer(sendWin, sendOff, p) + i * 16));
      r = V::pack(acc);
      for (int p = 0; p < n; ++p) *(uint4*)((char*)ncclGetLsaPointer(recvWin, recvOff, (dc.lsaRank + p) % n) + i * 16) = r;
    }
  }
  if (bar.sync(0, true, false) != ncclSuccess && threadIdx.x == 0) atomicExch(status, 2);
  bar.finish();
}

__device__ __forceinline__ float blockSum(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < kThreads / 32 ? smem[threadIdx.x] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) smem[32] = t;
  }
  __syncthreads();
  return smem[32];
}

// mode 0: one-shot, peer loads; 1: one-shot, multimem.ld_reduce; 2: two-shot, peer loads + peer stores
__global__ void __launch_bounds__(kThreads) devApiArRmsNormKernel(ncclDevComm_t dc, ncclWindow_t inWin, size_t inOff, ncclWindow_t resWin, size_t resOff,
                                                                   ncclWindow_t outWin, size_t outOff, const __nv_bfloat16* weight, float eps, int tokens,
                                                                   int hidden, int mode, int* status) {
  using V = nccl_device::Vec16<__nv_bfloat16>;
  __shared__ float red[40];
  ncclCoopCta cta;
  ncclLsaBarrierSession<ncclCoopCta> bar(cta, dc, ncclTeamLsa(dc), blockIdx.x);
  if (bar.sync(0, false, false) != ncclSuccess) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    bar.finish();
    return;
  }
  const int n = dc.lsaSize, me = dc.lsaRank;
  const int packsPerRow = hidden / 8;   // the host checks hidden % 8 == 0 and hidden <= 8 * kThreads * 4
  const size_t rowBytes = (size_t)hidden * 2;
  const int rowStep = mode == 2 ? gridDim.x * n : gridDim.x;
  const int rowStart = mode == 2 ? blockIdx.x * n + me : blockIdx.x;
  char* resLocal = (char*)ncclGetLocalPointer(resWin, resOff);
  char* outLocal = (char*)ncclGetLocalPointer(outWin, outOff);
  const char* mcIn = (const char*)ncclGetMultimemPointer(inWin, inOff);
  for (int t = rowStart; t < tokens; t += rowStep) {
    float x[4][8];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int pk = threadIdx.x + k * kThreads;
#pragma unroll
      for (int j = 0; j < 8; ++j) x[k][j] = 0.0f;
      if (pk < packsPerRow) {
        const size_t o = t * rowBytes + (size_t)pk * 16;
        if (mode == 1) {
          V::add(x[k], V::mcLoad(mcIn + o));
        } else {
          for (int p = 0; p < n; ++p) V::add(x[k], *(const uint4*)((const char*)ncclGetLsaPointer(inWin, inOff, p) + o));
        }
        V::add(x[k], *(const uint4*)(resLocal + o));
        // the residual stream is kept in bf16: normalise exactly what is stored
        const uint4 packed = V::pack(x[k]);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[k][j] = 0.0f;
        V::add(x[k], packed);
        if (mode == 2) {
          for (int p = 0; p < n; ++p) *(uint4*)((char*)ncclGetLsaPointer(resWin, resOff, (me + p) % n) + o) = packed;
        } else {
          *(uint4*)(resLocal + o) = packed;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += x[k][j] * x[k][j];
      }
    }
    const float inv = rsqrtf(blockSum(ss, red) / (float)hidden + eps);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int pk = threadIdx.x + k * kThreads;
      if (pk < packsPerRow) {
        const size_t o = t * rowBytes + (size_t)pk * 16;
        float w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        V::add(w, *(const uint4*)((const char*)weight + (size_t)pk * 16));
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] *= x[k][j] * inv;
        const uint4 packed = V::pack(w);
        if (mode == 2) {
          for (int p = 0; p < n; ++p) *(uint4*)((char*)ncclGetLsaPointer(outWin, outOff, (me + p) % n) + o) = packed;
        } else {
          *(uint4*)(outLocal + o) = packed;
        }
      }
    }
  }
  if (bar.sync(0, true, false) != ncclSuccess && threadIdx.x == 0) atomicExch(status, 2);
  bar.finish();
}

// Exercises ncclLLA2ASession: every rank contributes two floats per slot; each rank receives the sum.
__global__ void __launch_bounds__(256) devApiLLSumKernel(ncclDevComm_t dc, const float2* in, float2* out, int slots, int* status) {
  ncclCoopCta cta;
  ncclLLA2ASession<ncclCoopCta> ll(cta, dc, ncclTeamLsa(dc), blockIdx.x);
  for (int s = threadIdx.x; s < slots; s += blockDim.x) {
    const float2 v = in[blockIdx.x * slots + s];
    ll.bcast(s, (uint64_t)__float_as_uint(v.x) | ((uint64_t)__float_as_uint(v.y) << 32));
    float2 r;
    if (ll.recvReduceFloat2(s, v, &r) != ncclSuccess) {
      atomicExch(status, 3);
      break;
    }
    out[blockIdx.x * slots + s] = r;
  }
  ll.endEpoch();
}

// Exercises ncclGin: every rank puts `bytes` from its send region into the next rank's receive region,
// bumps signal 0 there, and waits until its own signal 0 has reached the call's sequence number.
__global__ void __launch_bounds__(256) devApiGinRingKernel(ncclDevComm_t dc, ncclWindow_t win, size_t sendOff, size_t recvOff, size_t bytes,
                                                           unsigned long long seq, int* status) {
  ncclCoopCta cta;
  ncclGin gin(dc);
  const ncclTeam_t team = ncclTeamLsa(dc);
  const int next = (dc.lsaRank + 1) % dc.lsaSize;
  if (gin.put(cta, team, next, win, recvOff, win, sendOff, bytes, /*signal*/ 0, /*counter*/ 0) != ncclSuccess) {
    if (threadIdx.x == 0) atomicExch(status, 4);
    return;
  }
  if (threadIdx.x == 0 && gin.waitSignal(0, seq) != ncclSuccess) atomicExch(status, 5);
}

int* statusWord() {
  static thread_local int* w[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!w[dev]) {
    if (cudaMalloc(&w[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(w[dev], 0, sizeof(int));
  }
  return w[dev];
}

}  // namespace

extern "C" {

// Sum all-reduce of `count` elements (ncclFloat32 or ncclBfloat16) from sendWin+sendOff into
// recvWin+recvOff on every rank. nCtas must not exceed the device communicator's lsaBarrierCount.
ncclResult_t b200DevApiAllReduce(const ncclDevComm_t* dc, ncclWindow_t sendWin, size_t sendOff, ncclWindow_t recvWin, size_t recvOff, size_t count,
                                 ncclDataType_t type, int multimem, int nCtas, cudaStream_t stream) {
  if (!dc || !sendWin || !recvWin || nCtas < 1 || nCtas > dc->lsaBarrierCount) return ncclInvalidArgument;
  if (type != ncclFloat32 && type != ncclBfloat16) return ncclInvalidArgument;
  const size_t per = type == ncclFloat32 ? 4 : 8;
  if (count % per || sendOff % 16 || recvOff % 16) return ncclInvalidArgument;
  if (multimem && (!sendWin->mcPtr || !recvWin->mcPtr)) return ncclInvalidUsage;
  int* st = statusWord();
  if (!st) return ncclUnhandledCudaError;
  if (type == ncclFloat32)
    devApiAllReduceKernel<float><<<nCtas, kThreads, 0, stream>>>(*dc, sendWin->devSelf, sendOff, recvWin->devSelf, recvOff, count, multimem, st);
  else
    devApiAllReduceKernel<__nv_bfloat16><<<nCtas, kThreads, 0, stream>>>(*dc, sendWin->devSelf, sendOff, recvWin->devSelf, recvOff, count, multimem, st);
  return cudaGetLastError() == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}

ncclResult_t b200DevApiArRmsNorm(const ncclDevComm_t* dc, ncclWindow_t inWin, size_t inOff, ncclWindow_t resWin, size_t resOff, ncclWindow_t outWin,
                                 size_t outOff, const void* weight, float eps, int tokens, int hidden, int mode, int nCtas, cudaStream_t stream) {
  if (!dc || !inWin || !resWin || !outWin || !weight || nCtas < 1 || nCtas > dc->lsaBarrierCount) return ncclInvalidArgument;
  if (hidden % 8 || hidden > 8 * kThreads * 4 || tokens < 0 || mode < 0 || mode > 2) return ncclInvalidArgument;
  if (inOff % 16 || resOff % 16 || outOff % 16 || (uintptr_t)weight % 16) return ncclInvalidArgument;
  if (mode == 1 && !inWin->mcPtr) return ncclInvalidUsage;
  int* st = statusWord();
  if (!st) return ncclUnhandledCudaError;
  devApiArRmsNormKernel<<<nCtas, kThreads, 0, stream>>>(*dc, inWin->devSelf, inOff, resWin->devSelf, resOff, outWin->devSelf, outOff,
                                                        (const __nv_bfloat16*)weight, eps, tokens, hidden, mode, st);
  return cudaGetLastError() == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}

ncclResult_t b200DevApiLLSum(const ncclDevComm_t* dc, const void* in, void* out, int slots, int nCtas, cudaStream_t stream) {
  if (!dc || !in || !out || nCtas < 1 || nCtas > dc->llA2ABlockCount || slots < 1 || slots > dc->llA2ASlotCount) return ncclInvalidArgument;
  int* st = statusWord();
  if (!st) return ncclUnhandledCudaError;
  devApiLLSumKernel<<<nCtas, 256, 0, stream>>>(*dc, (const float2*)in, (float2*)out, slots, st);
  return cudaGetLastError() == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}

// One CTA; needs a device communicator created with at least one GIN signal and counter.
ncclResult_t b200DevApiGinRing(const ncclDevComm_t* dc, ncclWindow_t win, size_t sendOff, size_t recvOff, size_t bytes, unsigned long long seq,
                               cudaStream_t stream) {
  if (!dc || !win || dc->ginSignalCount < 1 || dc->ginCounterCount < 1) return ncclInvalidArgument;
  int* st = statusWord();
  if (!st) return ncclUnhandledCudaError;
  devApiGinRingKernel<<<1, 256, 0, stream>>>(*dc, win->devSelf, sendOff, recvOff, bytes, seq, st);
  return cudaGetLastError() == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}

// 0 when no device-API kernel launched by this thread on the current device gave up a wait,
// otherwise the code of the wait (1 entry barrier, 2 exit barrier, 3 low-latency receive).
// Synchronises the device and clears the word.
int b200DevApiStatus(void) {
  int* st = statusWord();
  if (!st) return -1;
  int v = -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  cudaMemcpy(&v, st, sizeof(int), cudaMemcpyDeviceToHost);
  if (v) cudaMemset(st, 0, sizeof(int));
  return v;
}

}  // extern "C"
