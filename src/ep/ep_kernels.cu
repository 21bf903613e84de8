// Expert-parallel dispatch and combine, one kernel each.
//   epDispatchKernel  per token: read the bf16 row once, quantise it to e4m3 with one fp32 scale
//                     per 128 channels (or keep bf16), then one warp per selected expert stores the
//                     packed token straight into the landing zone of the rank that owns the expert
//                     (slot claimed with a local atomic, no remote atomics). When every CTA of the
//                     rank has sent, the per-expert counts are published with release stores. The
//                     same kernel then receives: per local expert it waits for the counts of all
//                     source ranks, and packs the landed tokens, their scales and their origin
//                     (source rank, token, k) contiguously per expert: the permutation is fused.
//   epCombineKernel   sends every expert output row back into the (token, k) slot of its source
//                     rank, publishes one flag per destination, waits for the flags of all ranks
//                     and forms the weighted sum over the token's selected experts in fp32.
// Counts and flags carry the call's epoch, so nothing has to be cleared between calls. Every wait
// is bounded and reports through the communicator's status words.
// Reference parity: contrib/nccl_ep/device/low_latency.cu (:105-153 fp8 cast, :520 dispatch, :1527
// combine), contrib/nccl_ubx/csrc/ubx.cu:1307 (quantising dispatch).
#include "ep_kernels.cuh"

#include <cuda_fp8.h>

#include "../kernels/common.cuh"

namespace b200 {

constexpr int kEpThreads = 512;
constexpr int kStCounters = 8;   // first per-expert counter inside state[]

__device__ __forceinline__ void stReleaseSys64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__global__ void __launch_bounds__(kEpThreads, 1) epDispatchKernel(const __grid_constant__ EpArgs a) {
  extern __shared__ uint8_t epSmem[];   // one packed token: payload (+ scales)
  __shared__ int sCnt[kMaxRanks], sOff[kMaxRanks + 1];
  __shared__ int sIsLast;
  const int rank = ctaRank(a.emu, a.rank);
  if (a.emu && ((a.absent >> rank) & 1u)) return;   // a rank that never joins (tests of the waits that run out)
  const int n = a.nRanks, H = a.hidden, K = a.topk, El = a.expertsPerRank, E = a.numExperts;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nWarps = kEpThreads / 32;
  uint32_t* st = a.state[rank];
  uint32_t* mask = a.mask[rank];                    // may be null: nobody is ever left out
  const uint32_t epoch = st[0] + 1;
  const size_t slotBytes = epSlotBytes(H, a.fp8);
  const size_t payload = slotBytes - 16;
  const int T = a.numTokens[rank];
  const __nv_bfloat16* x = a.x[rank];
  WaitCtx w{&a.sync, a.sync.status[rank]};
  // Landing zones and count words exist twice, selected by the parity of the epoch: a rank may start
  // call k+1 while a slower peer still packs call k, but it cannot reach k+2 before that peer has
  // finished k (it needs the peer's counts of k+1, which the peer sends after finishing k).
  const size_t zoneOff = (size_t)(epoch & 1) * ((size_t)El * n * a.maxTokens * slotBytes);
  const size_t cntOff = (size_t)(epoch & 1) * ((size_t)El * n);

  // ---------------------------------------------------------------- send
  const bool sendPhase = (a.phases & 1) != 0, recvPhase = (a.phases & 2) != 0;
  for (int t = blockIdx.x; sendPhase && t < T; t += gridDim.x) {
    const __nv_bfloat16* row = x + (size_t)t * H;
    if (a.fp8) {
      float* scales = (float*)(epSmem + H);
      for (int g = warp; g < H / 128; g += nWarps) {
        uint2 raw = *(const uint2*)(row + g * 128 + lane * 4);
        __nv_bfloat162 p0 = *(__nv_bfloat162*)&raw.x, p1 = *(__nv_bfloat162*)&raw.y;
        float v0 = __bfloat162float(p0.x), v1 = __bfloat162float(p0.y), v2 = __bfloat162float(p1.x), v3 = __bfloat162float(p1.y);
        float amax = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        amax = fmaxf(amax, 1e-4f);
        const float scale = amax * (1.0f / 448.0f), inv = 448.0f / amax;
        uint32_t packed = (uint32_t)__nv_cvt_float_to_fp8(v0 * inv, __NV_SATFINITE, __NV_E4M3) |
                          ((uint32_t)__nv_cvt_float_to_fp8(v1 * inv, __NV_SATFINITE, __NV_E4M3) << 8) |
                          ((uint32_t)__nv_cvt_float_to_fp8(v2 * inv, __NV_SATFINITE, __NV_E4M3) << 16) |
                          ((uint32_t)__nv_cvt_float_to_fp8(v3 * inv, __NV_SATFINITE, __NV_E4M3) << 24);
        *(uint32_t*)(epSmem + g * 128 + lane * 4) = packed;
        if (lane == 0) scales[g] = scale;
      }
    } else {
      for (int i = threadIdx.x; i < H / 8; i += kEpThreads) ((uint4*)epSmem)[i] = ((const uint4*)row)[i];
    }
    __syncthreads();
    for (int k = warp; k < K; k += nWarps) {
      const long long e = a.topkIdx[rank][(size_t)t * K + k];
      if (e < 0 || e >= E) continue;
      const int dst = (int)(e / El), el = (int)(e % El);
      if (mask && mask[dst]) continue;   // that rank is left out
      int s = 0;
      if (lane == 0) s = (int)atomicAdd(&st[kStCounters + e], 1u);
      s = __shfl_sync(0xffffffffu, s, 0);
      if (s >= a.maxTokens) continue;   // cannot happen while numTokens <= maxTokens
      char* slot = a.recvBuf[dst] + zoneOff + ((size_t)(el * n + rank) * a.maxTokens + s) * slotBytes;
      if (lane == 0) *(int4*)slot = make_int4(t * K + k, 0, 0, 0);
      for (size_t i = lane; i < payload / 16; i += 32) st16(slot + 16 + i * 16, ((const uint4*)epSmem)[i]);
    }
    __syncthreads();
  }
  // every CTA of this rank must be done before the counts go out
  __syncthreads();
  if (threadIdx.x == 0) {
    sIsLast = 0;
    if (sendPhase) {
      __threadfence_system();
      sIsLast = atomicAdd(&st[1], 1u) == gridDim.x - 1;
    }
  }
  __syncthreads();
  if (sIsLast) {
    __threadfence();
    for (int e = threadIdx.x; e < E; e += kEpThreads) {
      const uint32_t c = st[kStCounters + e];
      st[kStCounters + e] = 0;
      const int dst = e / El, el = e % El;
      if (mask && mask[dst]) continue;
      stReleaseSys64(a.recvCount[dst] + cntOff + (size_t)el * n + rank, ((unsigned long long)epoch << 32) | c);
    }
  }
  if (!recvPhase) return;   // split-phase call: ncclEpComplete runs the receiving half

  // ---------------------------------------------------------------- receive and pack
  const int cap = n * a.maxTokens;
  const size_t rowBytes = a.fp8 ? (size_t)H : (size_t)H * 2;
  bool ok = true;
  for (int el = blockIdx.x; el < El && ok; el += gridDim.x) {
    if (threadIdx.x < n) {
      const unsigned long long* c = a.recvCount[rank] + cntOff + (size_t)el * n + threadIdx.x;
      unsigned long long v = 0;
      int cnt = 0;
      if (!(mask && mask[threadIdx.x])) {
        const bool quiet = a.enableMask && mask;
        bool got = boundedWait(w, WAIT_TILE, threadIdx.x, epoch, [&] { v = ldRelaxedSys64((const uint64_t*)c); return (uint32_t)(v >> 32) == epoch; }, !quiet);
        fenceSys();
        if (got) cnt = (int)(uint32_t)v;
        else if (quiet && !(a.sync.abortFlag && ldRelaxedSys(a.sync.abortFlag))) { mask[threadIdx.x] = 1; cnt = 0; }   // left out from now on; the call goes on without it
        else cnt = -1;
      }
      sCnt[threadIdx.x] = cnt;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int off = 0;
      for (int s = 0; s < n; ++s) { sOff[s] = off; off += sCnt[s] > 0 ? sCnt[s] : 0; if (sCnt[s] < 0) off = -1 << 30; }
      sOff[n] = off;
      if (off >= 0) a.expertCount[rank][el] = off;
    }
    __syncthreads();
    ok = sOff[n] >= 0;
    if (ok) {
      const int total = sOff[n];
      for (int pos = warp; pos < total; pos += nWarps) {
        int s = 0;
        while (s + 1 < n && pos >= sOff[s + 1]) ++s;
        const int j = pos - sOff[s];
        const char* slot = a.recvBuf[rank] + zoneOff + ((size_t)(el * n + s) * a.maxTokens + j) * slotBytes;
        const size_t o = (size_t)el * cap + pos;
        if (lane == 0) a.srcInfo[rank][o] = make_int2(s, ((const int*)slot)[0]);
        char* dstTok = (char*)a.outTokens[rank] + o * rowBytes;
        {
          const size_t packs = rowBytes / 16;
          size_t i = lane;
          for (; i + 96 < packs; i += 128) {
            uint4 v0 = ldLocal16(slot + 16 + i * 16), v1 = ldLocal16(slot + 16 + (i + 32) * 16);
            uint4 v2 = ldLocal16(slot + 16 + (i + 64) * 16), v3 = ldLocal16(slot + 16 + (i + 96) * 16);
            st16(dstTok + i * 16, v0);
            st16(dstTok + (i + 32) * 16, v1);
            st16(dstTok + (i + 64) * 16, v2);
            st16(dstTok + (i + 96) * 16, v3);
          }
          for (; i < packs; i += 32) st16(dstTok + i * 16, ldLocal16(slot + 16 + i * 16));
        }
        if (a.fp8) {
          const float* sc = (const float*)(slot + 16 + H);
          float* dsc = a.outScales[rank] + o * (H / 128);
          for (int i = lane; i < H / 128; i += 32) dsc[i] = sc[i];
        }
      }
    }
    __syncthreads();
  }
  // the last CTA to finish closes the call
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&st[2], 1u) == gridDim.x - 1) {
      st[1] = 0;
      st[2] = 0;
      st[0] = epoch;
    }
  }
}

__global__ void __launch_bounds__(kEpThreads, 1) epCombineKernel(const __grid_constant__ EpArgs a) {
  __shared__ int sIsLast, sOk;
  const int rank = ctaRank(a.emu, a.rank);
  if (a.emu && ((a.absent >> rank) & 1u)) return;
  const int n = a.nRanks, H = a.hidden, K = a.topk, El = a.expertsPerRank;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nWarps = kEpThreads / 32;
  uint32_t* st = a.state[rank];
  uint32_t* mask = a.mask[rank];
  const bool sendPhase = (a.phases & 1) != 0, recvPhase = (a.phases & 2) != 0;
  const uint32_t epoch = st[4] + 1;
  const int cap = n * a.maxTokens;
  WaitCtx w{&a.sync, a.sync.status[rank]};
  const __nv_bfloat16* y = a.x[rank];
  const size_t combOff = (size_t)(epoch & 1) * ((size_t)a.maxTokens * K * H * 2);   // two landing zones, by epoch parity

  // ---------------------------------------------------------------- send expert outputs home
  for (int el = 0; sendPhase && el < El; ++el) {
    const int total = a.expertCount[rank][el];
    for (int pos = blockIdx.x * nWarps + warp; pos < total; pos += gridDim.x * nWarps) {
      const size_t o = (size_t)el * cap + pos;
      const int2 info = a.srcInfo[rank][o];
      if (mask && mask[info.x]) continue;
      const char* src = (const char*)(y + o * H);
      char* dst = a.combBuf[info.x] + combOff + (size_t)info.y * H * 2;
      // four independent 16-byte loads in flight per lane before the stores that depend on them
      const int packs = H / 8;
      int i = lane;
      for (; i + 96 < packs; i += 128) {
        uint4 v0 = ldLocal16(src + (size_t)i * 16), v1 = ldLocal16(src + (size_t)(i + 32) * 16);
        uint4 v2 = ldLocal16(src + (size_t)(i + 64) * 16), v3 = ldLocal16(src + (size_t)(i + 96) * 16);
        st16(dst + (size_t)i * 16, v0);
        st16(dst + (size_t)(i + 32) * 16, v1);
        st16(dst + (size_t)(i + 64) * 16, v2);
        st16(dst + (size_t)(i + 96) * 16, v3);
      }
      for (; i < packs; i += 32) st16(dst + (size_t)i * 16, ldLocal16(src + (size_t)i * 16));
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    sIsLast = 0;
    if (sendPhase) {
      __threadfence_system();
      sIsLast = atomicAdd(&st[5], 1u) == gridDim.x - 1;
    }
  }
  __syncthreads();
  if (sIsLast && threadIdx.x < n && !(mask && mask[threadIdx.x])) {
    __threadfence();
    stReleaseSys64(a.combFlag[threadIdx.x] + rank, (unsigned long long)epoch);
  }
  if (!recvPhase) return;

  // ---------------------------------------------------------------- wait for everybody's rows, then weighted sum
  if (threadIdx.x == 0) sOk = 1;
  __syncthreads();
  if (threadIdx.x < n && !(mask && mask[threadIdx.x])) {
    const unsigned long long* f = a.combFlag[rank] + threadIdx.x;
    const bool quiet = a.enableMask && mask;
    bool got = boundedWait(w, WAIT_TILE, threadIdx.x, epoch, [&] { return (int32_t)((uint32_t)ldRelaxedSys64((const uint64_t*)f) - epoch) >= 0; }, !quiet);
    fenceSys();
    if (!got) {
      if (quiet && !(a.sync.abortFlag && ldRelaxedSys(a.sync.abortFlag))) mask[threadIdx.x] = 1;   // its experts' rows are left out of the sums below
      else sOk = 0;
    }
  }
  __syncthreads();
  if (sOk) {
    const int T = a.numTokens[rank];
    __nv_bfloat16* out = (__nv_bfloat16*)a.outTokens[rank];
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
      for (int c = threadIdx.x; c < H / 8; c += kEpThreads) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        // the rows of up to eight selected experts are fetched together, then accumulated in slot order
        for (int k0 = 0; k0 < K; k0 += 8) {
          uint4 v[8];
          float wk[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int k = k0 + u;
            wk[u] = 0.0f;
            v[u] = make_uint4(0, 0, 0, 0);
            if (k < K) {
              const long long e = a.topkIdx[rank][(size_t)t * K + k];
              if (e >= 0 && e < a.numExperts && !(mask && mask[e / El])) {
                wk[u] = a.topkW[rank][(size_t)t * K + k];
                v[u] = ldLocal16(a.combBuf[rank] + combOff + ((size_t)(t * K + k) * H + (size_t)c * 8) * 2);
              }
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const __nv_bfloat162* p = (const __nv_bfloat162*)&v[u];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              acc[2 * i] += wk[u] * __bfloat162float(p[i].x);
              acc[2 * i + 1] += wk[u] * __bfloat162float(p[i].y);
            }
          }
        }
        uint4 o;
        __nv_bfloat162* q = (__nv_bfloat162*)&o;
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        *(uint4*)(out + (size_t)t * H + (size_t)c * 8) = o;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&st[6], 1u) == gridDim.x - 1) {
      st[5] = 0;
      st[6] = 0;
      st[4] = epoch;
    }
  }
}

const void* epDispatchKernelFn() { return (const void*)epDispatchKernel; }
const void* epCombineKernelFn() { return (const void*)epCombineKernel; }

}  // namespace b200
