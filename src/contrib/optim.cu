// Fused AdamW over one parameter shard of a sharded (ZeRO-3) optimizer: reads the reduce-scattered
// bf16 gradient once, updates the fp32 master weights and both moments, and writes the bf16 shard
// that the next all-gather publishes. One pass over memory: 2 + 12 bytes read, 12 + 2 written per
// element. Launched on the communication stream right behind the reduce-scatter it consumes.
// The reference has no optimizer; frameworks above it (FSDP, ZeRO) run this step between its
// reduce-scatter and all-gather calls (src/collectives.cc: ncclReduceScatter / ncclAllGather).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "nccl.h"

namespace {

struct AdamArgs {
  float lr, beta1, beta2, eps, weightDecay, gradScale, biasCorr1, biasCorr2Sqrt;
};

__device__ __forceinline__ void adamOne(float& w, float& m, float& v, float g, const AdamArgs& a) {
  g *= a.gradScale;
  m = a.beta1 * m + (1.0f - a.beta1) * g;
  v = a.beta2 * v + (1.0f - a.beta2) * g * g;
  const float mhat = m / a.biasCorr1;
  const float denom = sqrtf(v) / a.biasCorr2Sqrt + a.eps;
  w = w * (1.0f - a.lr * a.weightDecay) - a.lr * mhat / denom;
}

__global__ void __launch_bounds__(256) fusedAdamWKernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                                        const __nv_bfloat16* __restrict__ grad, __nv_bfloat16* __restrict__ param, size_t n, AdamArgs a) {
  const size_t packs = n / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < packs; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 gq = __ldg((const uint4*)grad + i);
    const __nv_bfloat162* g2 = (const __nv_bfloat162*)&gq;
    float4 w0 = ((float4*)master)[2 * i], w1 = ((float4*)master)[2 * i + 1];
    float4 m0 = ((float4*)m)[2 * i], m1 = ((float4*)m)[2 * i + 1];
    float4 v0 = ((float4*)v)[2 * i], v1 = ((float4*)v)[2 * i + 1];
    adamOne(w0.x, m0.x, v0.x, __bfloat162float(g2[0].x), a);
    adamOne(w0.y, m0.y, v0.y, __bfloat162float(g2[0].y), a);
    adamOne(w0.z, m0.z, v0.z, __bfloat162float(g2[1].x), a);
    adamOne(w0.w, m0.w, v0.w, __bfloat162float(g2[1].y), a);
    adamOne(w1.x, m1.x, v1.x, __bfloat162float(g2[2].x), a);
    adamOne(w1.y, m1.y, v1.y, __bfloat162float(g2[2].y), a);
    adamOne(w1.z, m1.z, v1.z, __bfloat162float(g2[3].x), a);
    adamOne(w1.w, m1.w, v1.w, __bfloat162float(g2[3].y), a);
    ((float4*)master)[2 * i] = w0;
    ((float4*)master)[2 * i + 1] = w1;
    ((float4*)m)[2 * i] = m0;
    ((float4*)m)[2 * i + 1] = m1;
    ((float4*)v)[2 * i] = v0;
    ((float4*)v)[2 * i + 1] = v1;
    uint4 pq;
    __nv_bfloat162* p2 = (__nv_bfloat162*)&pq;
    p2[0] = __floats2bfloat162_rn(w0.x, w0.y);
    p2[1] = __floats2bfloat162_rn(w0.z, w0.w);
    p2[2] = __floats2bfloat162_rn(w1.x, w1.y);
    p2[3] = __floats2bfloat162_rn(w1.z, w1.w);
    ((uint4*)param)[i] = pq;
  }
  // tail (n is normally padded to a multiple of 8 by the sharding engine)
  for (size_t e = packs * 8 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
    float w = master[e], mm = m[e], vv = v[e];
    adamOne(w, mm, vv, __bfloat162float(grad[e]), a);
    master[e] = w;
    m[e] = mm;
    v[e] = vv;
    param[e] = __float2bfloat16_rn(w);
  }
}

}  // namespace

extern "C" ncclResult_t b200FusedAdamW(void* master, void* m, void* v, const void* grad, void* param, size_t n, float lr, float beta1, float beta2,
                                       float eps, float weightDecay, float gradScale, int step, cudaStream_t stream) {
  if (!master || !m || !v || !grad || !param || step < 1) return ncclInvalidArgument;
  if (((uintptr_t)master | (uintptr_t)m | (uintptr_t)v | (uintptr_t)grad | (uintptr_t)param) % 16) return ncclInvalidArgument;
  if (n == 0) return ncclSuccess;
  AdamArgs a;
  a.lr = lr;
  a.beta1 = beta1;
  a.beta2 = beta2;
  a.eps = eps;
  a.weightDecay = weightDecay;
  a.gradScale = gradScale;
  a.biasCorr1 = 1.0f - powf(beta1, (float)step);
  a.biasCorr2Sqrt = sqrtf(1.0f - powf(beta2, (float)step));
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  size_t want = (n / 8 + 255) / 256;
  int grid = (int)(want < (size_t)sms * 8 ? (want ? want : 1) : (size_t)sms * 8);
  fusedAdamWKernel<<<grid, 256, 0, stream>>>((float*)master, (float*)m, (float*)v, (const __nv_bfloat16*)grad, (__nv_bfloat16*)param, n, a);
  return cudaGetLastError() == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}
