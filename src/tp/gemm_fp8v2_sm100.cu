// Block-scaled fp8 GEMM, second kernel: the same two-level accumulation as gemm_fp8_sm100.cu (one
// 128-wide K block per tcgen05.mma pass into one of two TMEM accumulators, then a scaled add into
// fp32 registers), rearranged so that a CTA has exactly 8 warps and every thread may use 255
// registers: 128 accumulators plus two 32-column staging buffers, which lets the tcgen05.ld of the
// next column chunk fly while the current one is being accumulated.
//   warps 0-7   all are epilogue warps: warp w owns TMEM lanes [32 (w & 3), +32) and columns
//               [128 (w >> 2), +128) of the 128 x 256 tile;
//   control     thread 0 (lane 0 of warp 0) additionally drives the pipeline between its epilogue
//               steps: it issues the TMA loads of stages that became free and the MMAs of the K
//               block after the one being accumulated, with non-blocking mbarrier tests for work
//               that lies ahead and bounded waits for work the epilogue is about to need.
// Operands, scales, tile walk and fused modes are those of gemm_fp8_sm100.cu. Every wait is bounded.
#include <cuda_fp8.h>

#include "gemm_sm100.cuh"

#include "../kernels/common.cuh"
#include "tp.h"

namespace b200 {

using namespace sm100;

namespace {
constexpr int BM = kTpBM, BN = kTpBN, BK = 128, STAGES = 4, UMMA_K = 32;
constexpr int kThreads = 256, kEpiWarps = 8;
constexpr uint32_t kStageABytes = BM * BK, kStageBBytes = BN * BK;
constexpr uint32_t kStageBytes = kStageABytes + kStageBBytes;
constexpr uint32_t kTmemCols = 512;
constexpr size_t kEpiBufBytes = kEpiWarps * 4096;
constexpr size_t kSmemBytes = 1024 + (size_t)STAGES * kStageBytes + 256 + kEpiBufBytes;
constexpr int kPrefetch = 4;

__device__ __forceinline__ bool mbarTest(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

// Pipeline state of the control thread.
struct Ctl {
  uint32_t loadKc = 0, mmaKc = 0;     // K blocks (counted over all tiles of this CTA) loaded / issued so far
  int armedStage[STAGES];
};
}  // namespace

__global__ void __launch_bounds__(kThreads, 1)
tpGemmFp8KernelV2(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ TpGemmArgs a) {
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
    // ---- all-gather role, as in gemm_fp8_sm100.cu: scales with plain peer loads, rows with bulk copies
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
    for (int idx = commIdx; idx < (n - 1) * blocksPerRank && ok; idx += commN) {
      const int src = (rank + 1 + idx / blocksPerRank) % n;
      const int mb = src * blocksPerRank + idx % blocksPerRank;
      const float* sFrom = (const float*)((const char*)a.peerA[src] + a.scaleOffset);
      float* sTo = (float*)((char*)a.peerA[rank] + a.scaleOffset);
      for (int e = threadIdx.x; e < kBlocks * (BM / 4); e += kThreads) {
        const size_t off = (size_t)(e / (BM / 4)) * a.M + (size_t)mb * BM + (size_t)(e % (BM / 4)) * 4;
        st16(sTo + off, ldStream16(sFrom + off));
      }
      __syncthreads();
      if (threadIdx.x == 0) {
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
  const int myTiles = (int)blockIdx.x < nTiles ? (nTiles - 1 - (int)blockIdx.x) / gemmCtas + 1 : 0;
  const uint32_t totalKc = (uint32_t)myTiles * (uint32_t)kBlocks;
  const uint32_t smemA0 = smemAddr(smem), smemB0 = smemA0 + STAGES * kStageABytes;
  const uint32_t idesc = umInstrE4m3(BM, BN);
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

  const bool isCtl = threadIdx.x == 0;
  Ctl ctl;
  for (int s = 0; s < STAGES; ++s) ctl.armedStage[s] = -1;

  // Issues the loads of K block `kc` (counted over this CTA's tiles). must: wait (bounded) for the stage; else only test.
  auto tryLoad = [&](bool must) -> bool {
    const uint32_t kc = ctl.loadKc;
    const int s = kc % STAGES;
    const uint32_t ph = (kc / STAGES) & 1;
    const uint32_t eb = smemAddr(&emptyBar[s]);
    if (!(must ? mbarWait(eb, ph ^ 1) : mbarTest(eb, ph ^ 1))) {
      if (must) fail(WAIT_TILE, 1000 + s);
      return false;
    }
    const int t = blockIdx.x + (int)(kc / kBlocks) * gemmCtas, kb = (int)(kc % kBlocks);
    const TileCoord tc = tileOf(a, t);
    if (kb == 0 && a.mode == TP_MODE_GATHER && n > 1 && tc.owner != rank) {
      // the comm CTAs must have landed this block of rows (and its scales)
      const uint32_t* f = a.blockFlags + tc.mBlk;
      bool got = false;
      const uint32_t limit = must ? (1u << 26) : 1u;
      for (uint32_t spin = 0; spin < limit; ++spin) {
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if ((int32_t)(v - a.flagEpoch) >= 0) { got = true; break; }
        if (*abortFlag) break;
      }
      if (!got) {
        if (must) fail(WAIT_TILE, (uint32_t)tc.mBlk);
        return false;
      }
      fenceProxyAsync();
    }
    const uint32_t fb = smemAddr(&fullBar[s]);
    mbarExpectTx(fb, kStageBytes);
    tmaLoad2d(smemA0 + s * kStageABytes, &tmA, kb * BK, tc.mBlk * BM, fb);
    tmaLoad2d(smemB0 + s * kStageBBytes, &tmB, kb * BK, tc.nBlk * BN, fb);
    ctl.armedStage[s] = (int)ph;
    ++ctl.loadKc;
    return true;
  };
  // Issues the MMAs of K block ctl.mmaKc into accumulator (mmaKc & 1).
  auto tryMma = [&](bool must) -> bool {
    const uint32_t kc = ctl.mmaKc;
    const int buf = kc & 1;
    const uint32_t aph = (kc >> 1) & 1;
    const uint32_t ab = smemAddr(&accEmpty[buf]);
    if (!(must ? mbarWait(ab, aph ^ 1) : mbarTest(ab, aph ^ 1))) {
      if (must) fail(WAIT_TILE, 2000 + buf);
      return false;
    }
    const int s = kc % STAGES;
    const uint32_t ph = (kc / STAGES) & 1;
    const uint32_t fb = smemAddr(&fullBar[s]);
    if (!(must ? mbarWait(fb, ph) : mbarTest(fb, ph))) {
      if (must) fail(WAIT_TILE, 3000 + s);
      return false;
    }
    tcFenceAfter();
    const uint32_t dT = tmemBase + buf * BN;
    const uint32_t aAddr = smemA0 + s * kStageABytes, bAddr = smemB0 + s * kStageBBytes;
#pragma unroll
    for (int k = 0; k < BK / UMMA_K; ++k) ummaF8(dT, umDescK128(aAddr + k * UMMA_K), umDescK128(bAddr + k * UMMA_K), idesc, k != 0);
    ummaCommit(smemAddr(&emptyBar[s]));
    ummaCommit(smemAddr(&accFull[buf]));
    ++ctl.mmaKc;
    return true;
  };
  // Keeps the pipeline ahead of the epilogue, which is about to accumulate K block `kc`.
  auto pump = [&](uint32_t kc) {
    // loads: as many stages as are free, never further than STAGES ahead of the MMAs
    while (ctl.loadKc < totalKc && ctl.loadKc < ctl.mmaKc + STAGES && !*abortFlag) {
      const bool must = ctl.loadKc <= kc;   // the block the epilogue waits for next has to be on its way
      if (!tryLoad(must)) break;
    }
    // MMAs: block kc must be issued now, and block kc+1 right behind it so that the tensor cores work
    // on it while block kc is being accumulated. Its accumulator is free once every warp has finished
    // block kc-1, which they do within a few hundred cycles of this warp: a (bounded) wait, not a test.
    while (ctl.mmaKc < totalKc && ctl.mmaKc <= kc + 1 && !*abortFlag) {
      if (ctl.loadKc <= ctl.mmaKc) { if (!tryLoad(true)) break; }
      if (!tryMma(true)) break;
    }
    while (ctl.loadKc < totalKc && ctl.loadKc < ctl.mmaKc + STAGES && !*abortFlag) {
      if (!tryLoad(false)) break;
    }
  };

  // ---- every warp: epilogue over this CTA's K blocks
  const int q = warp & 3;
  const int h = warp >> 2;
  const float* scaleA = a.mode == TP_MODE_GATHER && n > 1 ? (const float*)((const char*)a.peerA[rank] + a.scaleOffset) : a.scaleA;
  const int wBlocksN = a.N / 128;
  const bool gathered = a.mode == TP_MODE_GATHER && n > 1;
  uint32_t kc = 0;
  bool bad = false;
  for (int t = blockIdx.x; t < nTiles && !bad && !*abortFlag; t += gemmCtas) {
    const TileCoord tc = tileOf(a, t);
    const int row = tc.mBlk * BM + q * 32 + lane;
    const int wCol = tc.nBlk * 2 + h;
    float acc[128];
#pragma unroll
    for (int j = 0; j < 128; ++j) acc[j] = 0.0f;
    float sc[kPrefetch];
#pragma unroll
    for (int u = 0; u < kPrefetch; ++u) sc[u] = 0.0f;
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
        if (isCtl) pump(kc);
        __syncwarp();   // lane 0 of warp 0 rejoins its warp before the warp-wide tensor-memory instructions
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
        // two staging buffers: the load of the next 32 columns is in flight while these are accumulated
        uint32_t r0[32], r1[32];
        tmemLd32(tBase, r0);
        tmemLdWait();
        tmemLd32(tBase + 32, r1);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = fmaf(__uint_as_float(r0[j]), s, acc[j]);
        tmemLdWait();
        tmemLd32(tBase + 64, r0);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[32 + j] = fmaf(__uint_as_float(r1[j]), s, acc[32 + j]);
        tmemLdWait();
        tmemLd32(tBase + 96, r1);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[64 + j] = fmaf(__uint_as_float(r0[j]), s, acc[64 + j]);
        tmemLdWait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[96 + j] = fmaf(__uint_as_float(r1[j]), s, acc[96 + j]);
        tcFenceBefore();
        __syncwarp();
        if (lane == 0) mbarArrive(smemAddr(&accEmpty[buf]));
        ++kc;
      }
    }
    if (bad) break;
    // keep the tensor cores fed while this warp writes the tile out
    if (isCtl && kc < totalKc) pump(kc);
    __syncwarp();
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
      uint8_t* wbuf = epiBuf + (size_t)warp * 4096;
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
  if (isCtl && *abortFlag) {
    // copies already issued still write into this CTA's shared memory: wait for them (bounded)
    for (int s = 0; s < STAGES; ++s)
      if (ctl.armedStage[s] >= 0) mbarWait(smemAddr(&fullBar[s]), (uint32_t)ctl.armedStage[s], 1u << 20);
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

const void* tpGemmFp8V2KernelFn() { return (const void*)tpGemmFp8KernelV2; }
size_t tpGemmFp8V2SmemBytes() { return kSmemBytes; }
int tpGemmFp8V2Threads() { return kThreads; }

}  // namespace b200
