// Tensor-parallel GEMM kernels for sm_100a: C[M,N] = A[M,K] * W[N,K]^T in bf16 with fp32
// accumulation in tensor memory, fused with the collective that follows or precedes it.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      TMA producer: streams 128x64 A tiles and 256x64 W tiles (128-byte swizzle) through
//               a 4-stage shared-memory ring, one elected thread, mbarrier transaction counts.
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (128x256x16, cta_group::1) into
//               one of two 256-column TMEM accumulators; tcgen05.commit releases ring stages and
//               publishes finished accumulators.
//   warps 2-5   epilogue: tcgen05.ld the accumulator (each warp owns 32 TMEM lanes = 32 rows),
//               then, depending on the mode,
//                 STORE      convert to bf16 and store C;
//                 REDUCE     GEMM -> reduce-scatter: store the tile, rounded to bf16 (what a separate
//                            GEMM would hand to a reduce-scatter), straight into this rank's slot of
//                            the staging buffer of the rank that owns those rows, over NVLink; tiles
//                            are visited owner by owner, starting with the next rank, so every step
//                            each GPU receives from exactly one peer. A small kernel sums the slots.
//   GATHER mode all-gather -> GEMM: extra "comm" CTAs pull the other ranks' A rows from their
//               windows into the local A buffer, 128-row block by block, with bulk copies
//               (cp.async.bulk peer -> shared memory -> local, one issuing thread, several copies
//               in flight) and publish a flag per block; the TMA producer waits for the flag of
//               the block it needs. Blocks are fetched in the order the GEMM consumes them.
// No load uses cluster multicast; tensor-map (tiled) TMA loads read local memory only.
// Every wait (mbarrier, flag, cross-GPU barrier) is bounded; on expiry the kernel records a status,
// drains its outstanding TMA copies, frees its tensor memory and returns.
// gemm_pair_sm100.cu is the variant on CTA pairs (256 x 256 tiles, tcgen05 cta_group::2), which the host
// prefers when every rank's rows split into 256-row tiles; this kernel covers the remaining shapes.
// The reference has no GEMM kernels; the comparison point is its reduce-scatter / all-gather plus a
// separate GEMM.
#include "gemm_roles.cuh"

namespace b200 {

using namespace sm100;

constexpr int BM = kTpBM, BN = kTpBN, BK = kTpBK, STAGES = 4, UMMA_K = 16;
constexpr int kTpThreads = 192;
constexpr uint32_t kStageABytes = BM * BK * 2, kStageBBytes = BN * BK * 2;
constexpr uint32_t kStageBytes = kStageABytes + kStageBBytes;
constexpr uint32_t kTmemCols = 512;
constexpr size_t kEpiBufBytes = 4 * 4096;   // one 32 x 128-byte transpose buffer per epilogue warp
constexpr size_t kTpSmemBytes = 1024 + (size_t)STAGES * kStageBytes + 256 + kEpiBufBytes;

__global__ void __launch_bounds__(kTpThreads, 1)
tpGemmKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ TpGemmArgs a) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
  uint8_t* ctrl = smem + (size_t)STAGES * kStageBytes;
  uint64_t* fullBar = (uint64_t*)ctrl;            // [STAGES]
  uint64_t* emptyBar = fullBar + STAGES;          // [STAGES]
  uint64_t* accFull = emptyBar + STAGES;          // [2]
  uint64_t* accEmpty = accFull + 2;               // [2]
  uint32_t* tmemSlot = (uint32_t*)(accEmpty + 2);
  volatile uint32_t* abortFlag = tmemSlot + 1;
  uint8_t* epiBuf = ctrl + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = a.rank, n = a.nRanks;
  const bool multi = n > 1 && a.mode != TP_MODE_STORE;
  const bool commCta = a.mode == TP_MODE_GATHER && n > 1 && (int)blockIdx.x >= a.gemmCtas;

  CtaBarrier bar;
  bool ok = true;
  if (multi) {
    bar.init(a.sync, rank, n, blockIdx.x);
    ok = bar.sync(false, false);   // REDUCE: every accumulation buffer is zeroed; GATHER: every rank's rows are in place
  }

  if (commCta) {
    // ---- all-gather role: pull the other ranks' row blocks in consumption order
    static_assert(kTpPipeBytes <= (size_t)STAGES * kStageBytes, "copy ring must fit the operand ring");
    static_assert(kTpPipeStages <= 2 * STAGES, "not enough barriers");   // the operand barriers are unused by a comm CTA
    tpCommRole(a, blockIdx.x - a.gemmCtas, gridDim.x - a.gemmCtas, smem, fullBar, ok);
    bar.sync(true, false);   // nobody reads my rows any more
    bar.finish();
    return;
  }

  // ---- GEMM CTA set-up
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbarInit(smemAddr(&fullBar[s]), 1); mbarInit(smemAddr(&emptyBar[s]), 1); }
    for (int b = 0; b < 2; ++b) { mbarInit(smemAddr(&accFull[b]), 1); mbarInit(smemAddr(&accEmpty[b]), 4); }
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
  const int kBlocks = a.K / BK;
  const int gemmCtas = (a.mode == TP_MODE_GATHER && n > 1) ? a.gemmCtas : gridDim.x;
  const uint32_t smemA0 = smemAddr(smem), smemB0 = smemA0 + STAGES * kStageABytes;
  auto fail = [&](uint32_t kind, uint32_t what) {
    *abortFlag = 1;
    tpReportTimeout(a, kind, what);
  };

  if (warp == 0) {
    if (electOne()) {
      uint32_t kc = 0;
      int armedStage[STAGES];
      for (int s = 0; s < STAGES; ++s) armedStage[s] = -1;
      for (int t = blockIdx.x; t < nTiles && !*abortFlag; t += gemmCtas) {
        const TileCoord tc = tileOf(a, t);
        if (a.mode == TP_MODE_GATHER && n > 1 && tc.owner != rank) {
          // wait until the comm CTAs have landed this block of rows
          if (!tpWaitBlock(a, tc.mBlk, abortFlag)) { fail(WAIT_TILE, (uint32_t)tc.mBlk); break; }
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
        // copies already issued still write into this CTA's shared memory: wait for them (bounded)
        for (int s = 0; s < STAGES; ++s)
          if (armedStage[s] >= 0) mbarWait(smemAddr(&fullBar[s]), (uint32_t)armedStage[s], 1u << 20);
      }
    }
  } else if (warp == 1) {
    if (electOne()) {
      const uint32_t idesc = umInstrBf16(BM, BN);
      uint32_t kc = 0;
      int it = 0;
      for (int t = blockIdx.x; t < nTiles && !*abortFlag; t += gemmCtas, ++it) {
        const int buf = it & 1;
        const uint32_t aph = (it >> 1) & 1;
        if (!mbarWait(smemAddr(&accEmpty[buf]), aph ^ 1)) { fail(WAIT_TILE, 2000 + buf); break; }
        tcFenceAfter();
        const uint32_t dT = tmemBase + buf * BN;
        bool bad = false;
        for (int kb = 0; kb < kBlocks; ++kb, ++kc) {
          const int s = kc % STAGES;
          const uint32_t ph = (kc / STAGES) & 1;
          if (!mbarWait(smemAddr(&fullBar[s]), ph)) { fail(WAIT_TILE, 3000 + s); bad = true; break; }
          tcFenceAfter();
          const uint32_t aAddr = smemA0 + s * kStageABytes, bAddr = smemB0 + s * kStageBBytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            ummaBf16(dT, umDescK128(aAddr + k * UMMA_K * 2), umDescK128(bAddr + k * UMMA_K * 2), idesc, (kb | k) != 0);
          ummaCommit(smemAddr(&emptyBar[s]));   // the stage is free once these MMAs have read it
        }
        if (bad) break;
        ummaCommit(smemAddr(&accFull[buf]));    // accumulator complete
      }
    }
  } else {
    // ---- epilogue warps: TMEM lanes [32q, 32q+32) belong to the warp with warp % 4 == q
    const int q = warp & 3;
    int it = 0;
    for (int t = blockIdx.x; t < nTiles && !*abortFlag; t += gemmCtas, ++it) {
      const TileCoord tc = tileOf(a, t);
      const int buf = it & 1;
      const uint32_t aph = (it >> 1) & 1;
      if (!mbarWait(smemAddr(&accFull[buf]), aph)) { if (lane == 0) fail(WAIT_TILE, 4000 + buf); break; }
      tcFenceAfter();
      const int row0 = tc.mBlk * BM + q * 32;   // first of this warp's 32 rows
      const uint32_t tBase = tmemBase + ((uint32_t)(q * 32) << 16) + buf * BN;
      tpStoreAccum(a, tBase, row0, tc.nBlk, tc.owner, epiBuf + (size_t)(warp - 2) * 4096, lane);
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArrive(smemAddr(&accEmpty[buf]));
    }
  }

  // ---- teardown: everybody meets, tensor memory goes back, then the cross-GPU barrier
  tcFenceBefore();
  __syncthreads();
  if (warp == 1) {
    tcFenceAfter();
    tmemDealloc(tmemBase, kTmemCols);
  }
  if (multi) {
    bar.sync(true, false);   // REDUCE: every partial sum has landed in its owner's buffer
    bar.finish();
  }
}

// out[i] = sum over sources of staged[src][i]: the partial products of GEMM -> reduce-scatter become the
// output; bf16 inputs, fp32 accumulation in source order, bf16 result. count is a multiple of 8.
__global__ void tpReduceKernel(const __nv_bfloat16* __restrict__ staged, __nv_bfloat16* __restrict__ out, size_t count, int nSources) {
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  const size_t stride = (size_t)gridDim.x * blockDim.x * 8;
  for (; i + 7 < count; i += stride) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < nSources; ++s) {
      const uint4 v = *(const uint4*)(staged + (size_t)s * count + i);
      const __nv_bfloat162* p = (const __nv_bfloat162*)&v;
#pragma unroll
      for (int k = 0; k < 4; ++k) { acc[2 * k] += __bfloat162float(p[k].x); acc[2 * k + 1] += __bfloat162float(p[k].y); }
    }
    uint4 o;
    __nv_bfloat162* q = (__nv_bfloat162*)&o;
#pragma unroll
    for (int k = 0; k < 4; ++k) q[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
    *(uint4*)(out + i) = o;
  }
}

const void* tpGemmKernelFn() { return (const void*)tpGemmKernel; }
const void* tpReduceKernelFn() { return (const void*)tpReduceKernel; }
size_t tpGemmSmemBytes() { return kTpSmemBytes; }
int tpGemmThreads() { return kTpThreads; }

}  // namespace b200
