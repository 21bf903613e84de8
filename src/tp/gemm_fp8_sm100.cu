// Block-scaled fp8 (e4m3) tensor-parallel GEMM for sm_100a: C[M,N] = A[M,K] * W[N,K]^T where
// A carries one fp32 scale per row and 128 columns (scaleA[K/128][M]) and W one per 128 x 128
// block (scaleW[K/128][N/128]); accumulation is fp32.
//
// The tensor cores cannot apply fp32 block scales themselves, so accumulation has two levels:
//   level 1  tcgen05.mma kind::f8f6f4 (128x256x32) sums one 128-wide K block into a TMEM
//            accumulator; two 256-column accumulators alternate block by block;
//   level 2  the epilogue warps read each finished block from TMEM (tcgen05.ld), multiply by
//            scaleA[row] * scaleW[block] and add into fp32 registers, while the tensor cores
//            already work on the next K block in the other accumulator.
// Persistent CTAs of 320 threads: warp 0 TMA producer (128x128-byte A tiles, 256x128-byte W tiles,
// 128-byte swizzle, 4-stage ring), warp 1 MMA issuer, warps 2-9 epilogue (each warp owns 32 TMEM
// lanes and one 128-column half of the tile: 128 fp32 accumulators per thread).
// The fused modes work as in the bf16 kernel (gemm_sm100.cu): REDUCE stores the scaled tile as bf16
// into this rank's slot of the owning rank's staging buffer over NVLink (summed afterwards);
// GATHER has comm CTAs pull remote row blocks with bulk copies and their scales with plain peer
// loads. No load uses cluster multicast; tensor-map TMA loads read local memory only.
// Quantisation kernels for both operand kinds are at the end of the file.
// Every wait is bounded; on expiry the kernel records a status, drains its TMA copies, frees its
// tensor memory and returns.
#include <cuda_fp8.h>

#include "gemm_sm100.cuh"

#include "../kernels/common.cuh"
#include "tp.h"

namespace b200 {

using namespace sm100;

namespace {
constexpr int BM = kTpBM, BN = kTpBN, BK = 128, STAGES = 4, UMMA_K = 32;
constexpr int kThreads = 320, kEpiWarps = 8;
constexpr uint32_t kStageABytes = BM * BK, kStageBBytes = BN * BK;
constexpr uint32_t kStageBytes = kStageABytes + kStageBBytes;
constexpr uint32_t kTmemCols = 512;
constexpr size_t kEpiBufBytes = kEpiWarps * 4096;   // one 32 x 128-byte transpose buffer per epilogue warp
constexpr size_t kSmemBytes = 1024 + (size_t)STAGES * kStageBytes + 256 + kEpiBufBytes;
constexpr int kPrefetch = 4;   // K blocks of scale look-ahead
}  // namespace

__global__ void __launch_bounds__(kThreads, 1)
tpGemmFp8Kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ TpGemmArgs a) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
  uint8_t* ctrl = smem + (size_t)STAGES * kStageBytes;
  uint64_t* fullBar = (uint64_t*)ctrl;
  uint64_t* emptyBar = fullBar + STAGES;
  uint64_t* accFull = emptyBar + STAGES;
  uint64_t* accEmpty = accFull + 2;
  uint32_t* tmemSlot = (uint32_t*)(accEmpty + 2);
  volatile uint32_t* abortFlag = tmemSlot + 1;
  uint8_t* epiBuf = ctrl + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = a.rank, n = a.nRanks;
  const bool multi = n > 1 && a.mode != TP_MODE_STORE;
  const bool commCta = a.mode == TP_MODE_GATHER && n > 1 && (int)blockIdx.x >= a.gemmCtas;
  const int kBlocks = a.K / BK;

  CtaBarrier bar;
  bool ok = true;
  if (multi) {
    bar.init(a.sync, rank, n, blockIdx.x);
    ok = bar.sync(false, false);
  }

  if (commCta) {
    // ---- all-gather role: rows (fp8) and their scales, block by block in consumption order
    const int blocksPerRank = a.M / n / BM;
    const size_t blockBytes = (size_t)BM * a.K;
    const int commIdx = blockIdx.x - a.gemmCtas, commN = gridDim.x - a.gemmCtas;
    constexpr int kPipeStages = 6;
    constexpr uint32_t kPipeChunk = 32768;
    static_assert((size_t)kPipeStages * kPipeChunk <= (size_t)STAGES * kStageBytes, "copy ring must fit the operand ring");
    uint64_t* pipeBars = fullBar;
    if (threadIdx.x == 0) {
      for (int s = 0; s < kPipeStages; ++s) mbarInit(smemAddr(&pipeBars[s]), 1);
      mbarInitFence();
    }
    __syncthreads();
    uint32_t phaseBits = 0;
    // remote blocks in the order the GEMM consumes them (rank+1 first), dealt round-robin to the comm CTAs
    for (int idx = commIdx; idx < (n - 1) * blocksPerRank && ok; idx += commN) {
      const int src = (rank + 1 + idx / blocksPerRank) % n;
      {
        const int b = idx % blocksPerRank;
        const int mb = src * blocksPerRank + b;
        // scales of these 128 rows: one 512-byte run per K block, plain peer loads by all threads
        const float* sFrom = (const float*)((const char*)a.peerA[src] + a.scaleOffset);
        float* sTo = (float*)((char*)a.peerA[rank] + a.scaleOffset);
        for (int e = threadIdx.x; e < kBlocks * (BM / 4); e += kThreads) {
          const size_t off = (size_t)(e / (BM / 4)) * a.M + (size_t)mb * BM + (size_t)(e % (BM / 4)) * 4;
          st16(sTo + off, ldStream16(sFrom + off));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
          // the rows: bulk copies peer -> shared memory -> local, driven by this one thread
          const char* from = (const char*)a.peerA[src] + (size_t)mb * blockBytes;
          char* to = (char*)a.peerA[rank] + (size_t)mb * blockBytes;
          ok = bulkPipe<kPipeStages, kPipeChunk>(to, from, blockBytes, smemAddr(smem), pipeBars, phaseBits);
          if (ok) {
            fenceProxyAsync();
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a.blockFlags + mb), "r"(a.flagEpoch) : "memory");
          } else if (a.sync.status[rank] && ldRelaxedSys(a.sync.status[rank]) == DEV_OK) {
            a.sync.status[rank][1] = WAIT_TILE;
            a.sync.status[rank][2] = 5000 + mb;
            a.sync.status[rank][3] = blockIdx.x;
            __threadfence_system();
            stRelaxedSys(a.sync.status[rank], DEV_TIMEOUT);
          }
        }
        ok = __syncthreads_and(ok);
      }
    }
    bar.sync(true, false);
    bar.finish();
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbarInit(smemAddr(&fullBar[s]), 1); mbarInit(smemAddr(&emptyBar[s]), 1); }
    for (int b = 0; b < 2; ++b) { mbarInit(smemAddr(&accFull[b]), 1); mbarInit(smemAddr(&accEmpty[b]), kEpiWarps); }
    *abortFlag = ok ? 0u : 1u;
    mbarInitFence();
    prefetchTensorMap(&tmA);
    prefetchTensorMap(&tmB);
  }
  if (warp == 1) {
    tmemAlloc(smemAddr(tmemSlot), kTmemCols);
    tmemRelinquish();
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;

  const int tilesN = a.N / BN;
  const int nTiles = (a.M / BM) * tilesN;
  const int gemmCtas = (a.mode == TP_MODE_GATHER && n > 1) ? a.gemmCtas : gridDim.x;
  const uint32_t smemA0 = smemAddr(smem), smemB0 = smemA0 + STAGES * kStageABytes;
  auto fail = [&](uint32_t kind, uint32_t what) {
    *abortFlag = 1;
    if (a.sync.status[rank] && ldRelaxedSys(a.sync.status[rank]) == DEV_OK) {
      a.sync.status[rank][1] = kind;
      a.sync.status[rank][2] = what;
      a.sync.status[rank][3] = blockIdx.x;
      __threadfence_system();
      stRelaxedSys(a.sync.status[rank], DEV_TIMEOUT);
    }
  };

  if (warp == 0) {
    if (electOne()) {
      uint32_t kc = 0;
      int armedStage[STAGES];
      for (int s = 0; s < STAGES; ++s) armedStage[s] = -1;
      for (int t = blockIdx.x; t < nTiles && !*abortFlag; t += gemmCtas) {
        const TileCoord tc = tileOf(a, t);
        if (a.mode == TP_MODE_GATHER && n > 1 && tc.owner != rank) {
          const uint32_t* f = a.blockFlags + tc.mBlk;
          bool got = false;
          for (uint32_t spin = 0; spin < (1u << 26); ++spin) {
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if ((int32_t)(v - a.flagEpoch) >= 0) { got = true; break; }
            if (*abortFlag) break;
          }
          if (!got) { fail(WAIT_TILE, (uint32_t)tc.mBlk); break; }
          fenceProxyAsync();
        }
        for (int kb = 0; kb < kBlocks; ++kb, ++kc) {
          const int s = kc % STAGES;
          const uint32_t ph = (kc / STAGES) & 1;
          if (!mbarWait(smemAddr(&emptyBar[s]), ph ^ 1)) { fail(WAIT_TILE, 1000 + s); break; }
          const uint32_t fb = smemAddr(&fullBar[s]);
          mbarExpectTx(fb, kStageBytes);
          tmaLoad2d(smemA0 + s * kStageABytes, &tmA, kb * BK, tc.mBlk * BM, fb);
          tmaLoad2d(smemB0 + s * kStageBBytes, &tmB, kb * BK, tc.nBlk * BN, fb);
          armedStage[s] = (int)ph;
        }
      }
      if (*abortFlag) {
        for (int s = 0; s < STAGES; ++s)
          if (armedStage[s] >= 0) mbarWait(smemAddr(&fullBar[s]), (uint32_t)armedStage[s], 1u << 20);
      }
    }
  } else if (warp == 1) {
    if (electOne()) {
      const uint32_t idesc = umInstrE4m3(BM, BN);
      uint32_t kc = 0;
      for (int t = blockIdx.x; t < nTiles && !*abortFlag; t += gemmCtas) {
        bool bad = false;
        for (int kb = 0; kb < kBlocks; ++kb, ++kc) {
          const int buf = kc & 1;
          const uint32_t aph = (kc >> 1) & 1;
          if (!mbarWait(smemAddr(&accEmpty[buf]), aph ^ 1)) { fail(WAIT_TILE, 2000 + buf); bad = true; break; }
          const int s = kc % STAGES;
          const uint32_t ph = (kc / STAGES) & 1;
          if (!mbarWait(smemAddr(&fullBar[s]), ph)) { fail(WAIT_TILE, 3000 + s); bad = true; break; }
          tcFenceAfter();
          const uint32_t dT = tmemBase + buf * BN;
          const uint32_t aAddr = smemA0 + s * kStageABytes, bAddr = smemB0 + s * kStageBBytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            ummaF8(dT, umDescK128(aAddr + k * UMMA_K), umDescK128(bAddr + k * UMMA_K), idesc, k != 0);
          ummaCommit(smemAddr(&emptyBar[s]));   // the stage is free once these MMAs have read it
          ummaCommit(smemAddr(&accFull[buf]));  // this K block's partial sums are complete
        }
        if (bad) break;
      }
    }
  } else {
    // ---- epilogue warps: TMEM lanes [32q, 32q+32), columns [128h, 128h+128)
    const int q = warp & 3;
    const int h = (warp - 2) >> 2;
    const float* scaleA = a.mode == TP_MODE_GATHER && n > 1 ? (const float*)((const char*)a.peerA[rank] + a.scaleOffset) : a.scaleA;
    const int wBlocksN = a.N / 128;
    uint32_t kc = 0;
    for (int t = blockIdx.x; t < nTiles && !*abortFlag; t += gemmCtas) {
      const TileCoord tc = tileOf(a, t);
      const int row = tc.mBlk * BM + q * 32 + lane;
      const int wCol = tc.nBlk * 2 + h;
      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.0f;
      // Scales of the next kPrefetch K blocks travel ahead of the accumulators that need them.
      // In GATHER mode the scales of remote rows land together with the rows: the flag the TMA
      // producer waited for covers them, and accFull orders this warp after the producer.
      float sc[kPrefetch];
#pragma unroll
      for (int u = 0; u < kPrefetch; ++u) sc[u] = 0.0f;
      bool bad = false;
      // Rows gathered from a peer arrive during this kernel: their scales may be read only after
      // the tile's first accumulator is published (the producer saw the block's flag before it
      // issued the TMA loads that fed it), and never through the read-only cache path.
      const bool gathered = a.mode == TP_MODE_GATHER && n > 1;
      const bool remoteRows = gathered && tc.owner != rank;
      auto scaleOf = [&](int kb) -> float {
        const float* pa = scaleA + (size_t)kb * a.M + row;
        const float sa = gathered ? *(const volatile float*)pa : __ldg(pa);
        return sa * __ldg(a.scaleW + (size_t)kb * wBlocksN + wCol);
      };
      bool primed = false;
      if (!remoteRows) {
#pragma unroll
        for (int u = 0; u < kPrefetch; ++u)
          if (u < kBlocks) sc[u] = scaleOf(u);
        primed = true;
      }
      for (int kb0 = 0; kb0 < kBlocks && !bad; kb0 += kPrefetch) {
#pragma unroll
        for (int u = 0; u < kPrefetch; ++u) {
          const int kb = kb0 + u;
          if (kb >= kBlocks || bad) continue;
          const int buf = kc & 1;
          const uint32_t aph = (kc >> 1) & 1;
          if (!mbarWait(smemAddr(&accFull[buf]), aph)) { if (lane == 0) fail(WAIT_TILE, 4000 + buf); bad = true; continue; }
          tcFenceAfter();
          if (!primed) {
#pragma unroll
            for (int v = 0; v < kPrefetch; ++v)
              if (v < kBlocks) sc[v] = scaleOf(v);
            primed = true;
          }
          const float s = sc[u];
          if (kb + kPrefetch < kBlocks) sc[u] = scaleOf(kb + kPrefetch);
          const uint32_t tBase = tmemBase + ((uint32_t)(q * 32) << 16) + buf * BN + h * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmemLd32(tBase + c * 32, r);
            tmemLdWait();
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(__uint_as_float(r[j]), s, acc[c * 32 + j]);
          }
          tcFenceBefore();
          __syncwarp();
          if (lane == 0) mbarArrive(smemAddr(&accEmpty[buf]));
          ++kc;
        }
      }
      if (bad) break;
      // final tile: bf16, transposed through shared memory so that every store instruction writes
      // whole 128-byte row segments (see the bf16 kernel); REDUCE targets the owner's staging slot
      {
        const int row0 = tc.mBlk * BM + q * 32;
        __nv_bfloat16* dstBase;
        size_t ld;
        if (a.mode == TP_MODE_REDUCE && n > 1) {
          const int rowsPerRank = a.M / n;
          dstBase = (__nv_bfloat16*)a.partial[tc.owner] + ((size_t)rank * rowsPerRank + (row0 - tc.owner * rowsPerRank)) * a.N + (size_t)tc.nBlk * BN + h * 128;
          ld = (size_t)a.N;
        } else {
          dstBase = (__nv_bfloat16*)a.C + (size_t)row0 * a.ldc + (size_t)tc.nBlk * BN + h * 128;
          ld = (size_t)a.ldc;
        }
        uint8_t* wbuf = epiBuf + (size_t)(warp - 2) * 4096;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 o;
            const int b0 = cc * 64 + j * 8;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(acc[b0], acc[b0 + 1]);
            __nv_bfloat162 p1 = __floats2bfloat162_rn(acc[b0 + 2], acc[b0 + 3]);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[b0 + 4], acc[b0 + 5]);
            __nv_bfloat162 p3 = __floats2bfloat162_rn(acc[b0 + 6], acc[b0 + 7]);
            o.x = *(uint32_t*)&p0; o.y = *(uint32_t*)&p1; o.z = *(uint32_t*)&p2; o.w = *(uint32_t*)&p3;
            *(uint4*)(wbuf + lane * 128 + ((j ^ (lane & 7)) * 16)) = o;
          }
          __syncwarp();
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int rr = k * 4 + (lane >> 3), j = lane & 7;
            const uint4 o = *(const uint4*)(wbuf + rr * 128 + ((j ^ (rr & 7)) * 16));
            *(uint4*)((char*)(dstBase + (size_t)rr * ld) + cc * 128 + j * 16) = o;
          }
          __syncwarp();
        }
      }
    }
  }

  tcFenceBefore();
  __syncthreads();
  if (warp == 1) {
    tcFenceAfter();
    tmemDealloc(tmemBase, kTmemCols);
  }
  if (multi) {
    bar.sync(true, false);
    bar.finish();
  }
}

// ------------------------------------------------------------------------------------ quantisation
__device__ __forceinline__ uint32_t packE4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

// Activations: one scale per row and 128 columns. One warp per (row, K block); scales[kb][row].
__global__ void __launch_bounds__(256) tpQuantRowsKernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scales,
                                                          int rows, int K) {
  const int kBlocks = K / 128;
  const size_t warpId = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const size_t nWarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (size_t w = warpId; w < (size_t)rows * kBlocks; w += nWarps) {
    const int row = (int)(w / kBlocks), kb = (int)(w % kBlocks);
    const size_t off = (size_t)row * K + (size_t)kb * 128 + lane * 4;
    const uint2 raw = *(const uint2*)(x + off);
    const __nv_bfloat162* p = (const __nv_bfloat162*)&raw;
    float v0 = __bfloat162float(p[0].x), v1 = __bfloat162float(p[0].y), v2 = __bfloat162float(p[1].x), v3 = __bfloat162float(p[1].y);
    float m = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float s = fmaxf(m, 1e-10f) / 448.0f;
    const float inv = 1.0f / s;
    *(uint32_t*)(q + off) = packE4m3x4(v0 * inv, v1 * inv, v2 * inv, v3 * inv);
    if (lane == 0) scales[(size_t)kb * rows + row] = s;
  }
}

// Weights: one scale per 128 x 128 block. One CTA of 256 threads per block; scales[kb][rows/128].
__global__ void __launch_bounds__(256) tpQuantBlocksKernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scales,
                                                            int rows, int K) {
  __shared__ float red[8];
  const int kBlocks = K / 128, rBlocks = rows / 128;
  for (int blk = blockIdx.x; blk < kBlocks * rBlocks; blk += gridDim.x) {
    const int rb = blk / kBlocks, kb = blk % kBlocks;
    // thread t: rows (t / 32) + 8 i, columns 4 (t % 32) .. +3
    float v[16][4];
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const size_t off = (size_t)(rb * 128 + (threadIdx.x >> 5) + 8 * i) * K + (size_t)kb * 128 + (threadIdx.x & 31) * 4;
      const uint2 raw = *(const uint2*)(x + off);
      const __nv_bfloat162* p = (const __nv_bfloat162*)&raw;
      v[i][0] = __bfloat162float(p[0].x); v[i][1] = __bfloat162float(p[0].y); v[i][2] = __bfloat162float(p[1].x); v[i][3] = __bfloat162float(p[1].y);
      m = fmaxf(m, fmaxf(fmaxf(fabsf(v[i][0]), fabsf(v[i][1])), fmaxf(fabsf(v[i][2]), fabsf(v[i][3]))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    const float s = fmaxf(m, 1e-10f) / 448.0f;
    const float inv = 1.0f / s;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const size_t off = (size_t)(rb * 128 + (threadIdx.x >> 5) + 8 * i) * K + (size_t)kb * 128 + (threadIdx.x & 31) * 4;
      *(uint32_t*)(q + off) = packE4m3x4(v[i][0] * inv, v[i][1] * inv, v[i][2] * inv, v[i][3] * inv);
    }
    if (threadIdx.x == 0) scales[(size_t)kb * rBlocks + rb] = s;
  }
}

const void* tpGemmFp8KernelFn() { return (const void*)tpGemmFp8Kernel; }
const void* tpQuantRowsKernelFn() { return (const void*)tpQuantRowsKernel; }
const void* tpQuantBlocksKernelFn() { return (const void*)tpQuantBlocksKernel; }
size_t tpGemmFp8SmemBytes() { return kSmemBytes; }
int tpGemmFp8Threads() { return kThreads; }

}  // namespace b200
