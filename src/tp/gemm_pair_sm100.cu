// CTA-pair variant of the tensor-parallel bf16 GEMM for sm_100a: two CTAs on neighbouring SMs (a
// cluster of two) work on one 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
// Each CTA streams only its half of the operands per 64-wide K step: 128 rows of A (its half of the
// tile's rows) and 128 rows of W (its half of the tile's columns), 32 KiB instead of the 48 KiB a
// single CTA needs for a 128 x 256 tile, through a 6-stage ring. One thread of the even ("leader")
// CTA issues 256 x 256 x 16 MMAs that read both CTAs' shared memory and write both CTAs' tensor
// memory: each CTA ends up with its 128 rows x 256 columns of the accumulator and runs the same
// epilogue as the one-CTA kernel.
//
// Synchronisation inside the pair:
//   fullBar[s]   (leader's copy only) counts the TMA bytes of BOTH CTAs for ring stage s: the peer's
//                loads name the leader's barrier (cp.async.bulk.tensor ... cta_group::2, no multicast);
//   emptyBar[s]  in each CTA: tcgen05.commit with an mbarrier multicast to both CTAs frees stage s;
//   accFull[b]   in each CTA: the same multicast commit publishes accumulator b to both epilogues;
//   accEmpty[b]  (leader's copy only) collects the arrivals of the eight epilogue warps of both CTAs.
// Tensor memory is allocated and freed by one warp in each CTA (cta_group::2 allocation is collective
// over the pair). A cluster barrier after set-up and one before the tensor memory is freed keep either
// CTA's shared and tensor memory alive while its partner may still touch it.
// Modes, the all-gather role of the comm CTAs, flags, bounded waits and status reporting are those of
// the one-CTA kernel (gemm_sm100.cu); rows per rank must be a multiple of 256 in the fused modes.
#include "gemm_roles.cuh"

namespace b200 {

using namespace sm100;

namespace {
constexpr int PM = 256;                         // rows of a pair tile
constexpr int BN = kTpBN, BK = kTpBK, UMMA_K = 16;
constexpr int P_STAGES = 6;
constexpr int kThreads = 192;
constexpr uint32_t kHalfBytes = 128 * BK * 2;   // 128 rows x 64 bf16: A half and W half are the same size
constexpr uint32_t kStageBytes = 2 * kHalfBytes;
constexpr int kAccBufs = 2;                     // accumulators of 256 columns in tensor memory: the epilogue of one tile overlaps the MMAs of the next
constexpr uint32_t kTmemCols = kAccBufs * 256;
constexpr size_t kEpiBufBytes = 4 * 4096;
constexpr size_t kSmemBytes = 1024 + (size_t)P_STAGES * kStageBytes + 256 + kEpiBufBytes;
static_assert(kTpPipeBytes <= (size_t)P_STAGES * kStageBytes, "copy ring must fit the operand ring");
static_assert(kTpPipeStages <= 2 * P_STAGES, "not enough barriers for the copy ring");
static_assert((2 * P_STAGES + 4) * 8 + 8 <= 256, "control block too small");
}  // namespace

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
tpGemmPairKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ TpGemmArgs a) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
  uint8_t* ctrl = smem + (size_t)P_STAGES * kStageBytes;
  uint64_t* fullBar = (uint64_t*)ctrl;            // [P_STAGES]
  uint64_t* emptyBar = fullBar + P_STAGES;        // [P_STAGES]
  uint64_t* accFull = emptyBar + P_STAGES;        // [2]
  uint64_t* accEmpty = accFull + 2;               // [2]
  uint32_t* tmemSlot = (uint32_t*)(accEmpty + 2);
  volatile uint32_t* abortFlag = tmemSlot + 1;
  uint8_t* epiBuf = ctrl + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = a.rank, n = a.nRanks;
  const bool multi = n > 1 && a.mode != TP_MODE_STORE;
  const bool gather = a.mode == TP_MODE_GATHER && n > 1;
  const bool commCta = gather && (int)blockIdx.x >= a.gemmCtas;   // gemmCtas is even: both CTAs of a pair have the same role

  CtaBarrier bar;
  bool ok = true;
  if (multi) {
    bar.init(a.sync, rank, n, blockIdx.x);
    ok = bar.sync(false, false);
  }

  if (commCta) {
    tpCommRole(a, blockIdx.x - a.gemmCtas, gridDim.x - a.gemmCtas, smem, fullBar, ok);
    bar.sync(true, false);   // nobody reads my rows any more
    bar.finish();
    return;
  }

  // ---- pair set-up
  const uint32_t cr = clusterCtaRank();   // 0: leader (issues the MMAs, owns fullBar / accEmpty), 1: peer
  const bool leader = cr == 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) { mbarInit(smemAddr(&fullBar[s]), 1); mbarInit(smemAddr(&emptyBar[s]), 1); }
    for (int b = 0; b < kAccBufs; ++b) { mbarInit(smemAddr(&accFull[b]), 1); mbarInit(smemAddr(&accEmpty[b]), 8); }
    *abortFlag = ok ? 0u : 1u;
    mbarInitFence();
    prefetchTensorMap(&tmA);
    prefetchTensorMap(&tmB);
  }
  if (warp == 1) {
    tmemAllocPair(smemAddr(tmemSlot), kTmemCols);
    tmemRelinquishPair();
  }
  tcFenceBefore();
  __syncthreads();
  __syncwarp();
  clusterSync();   // both CTAs' barriers are initialised before either signals the other's
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;
  if (!ok && threadIdx.x == 0) stSharedCluster(mapaShared(smemAddr((const void*)abortFlag), cr ^ 1), 1u);

  const int tilesN = a.N / BN;
  const int nTiles = (a.M / PM) * tilesN;
  const int kBlocks = a.K / BK;
  const int pairIdx = blockIdx.x >> 1;
  const int nPairs = (gather ? a.gemmCtas : (int)gridDim.x) >> 1;
  const uint32_t smemA0 = smemAddr(smem), smemB0 = smemA0 + P_STAGES * kHalfBytes;
  auto fail = [&](uint32_t kind, uint32_t what) {
    *abortFlag = 1;
    stSharedCluster(mapaShared(smemAddr((const void*)abortFlag), cr ^ 1), 1u);   // the partner gives up too
    tpReportTimeout(a, kind, what);
  };

  if (warp == 0) {
    if (electOne()) {
      uint32_t kc = 0;
      int armedStage[P_STAGES];
      for (int s = 0; s < P_STAGES; ++s) armedStage[s] = -1;
      for (int t = pairIdx; t < nTiles && !*abortFlag; t += nPairs) {
        const TileCoord tc = tileOf(a, t, PM);
        const int myBlk = tc.mBlk * 2 + (int)cr;   // this CTA's 128-row block of A
        if (gather && tc.owner != rank && !tpWaitBlock(a, myBlk, abortFlag)) { fail(WAIT_TILE, (uint32_t)myBlk); break; }
        for (int kb = 0; kb < kBlocks; ++kb, ++kc) {
          const int s = kc % P_STAGES;
          const uint32_t ph = (kc / P_STAGES) & 1;
          if (!mbarWait(smemAddr(&emptyBar[s]), ph ^ 1)) { fail(WAIT_TILE, 1000 + s); break; }
          if (*abortFlag) break;
          if (leader) mbarExpectTx(smemAddr(&fullBar[s]), 2 * kStageBytes);   // the bytes of both CTAs
          const uint32_t fb = mapaShared(smemAddr(&fullBar[s]), 0);
          tmaLoad2dPair(smemA0 + s * kHalfBytes, &tmA, kb * BK, myBlk * 128, fb);
          tmaLoad2dPair(smemB0 + s * kHalfBytes, &tmB, kb * BK, tc.nBlk * BN + (int)cr * 128, fb);
          armedStage[s] = (int)ph;
        }
      }
      if (*abortFlag && leader) {
        // copies already issued (by either CTA) still write into shared memory: wait for them (bounded)
        for (int s = 0; s < P_STAGES; ++s)
          if (armedStage[s] >= 0) mbarWait(smemAddr(&fullBar[s]), (uint32_t)armedStage[s], 1u << 20);
      }
    }
  } else if (warp == 1) {
    if (leader && electOne()) {
      const uint32_t idesc = umInstrBf16(PM, BN);
      uint32_t kc = 0;
      int it = 0;
      for (int t = pairIdx; t < nTiles && !*abortFlag; t += nPairs, ++it) {
        const int buf = it % kAccBufs;
        const uint32_t aph = (it / kAccBufs) & 1;
        if (!mbarWait(smemAddr(&accEmpty[buf]), aph ^ 1)) { fail(WAIT_TILE, 2000 + buf); break; }
        tcFenceAfter();
        const uint32_t dT = tmemBase + buf * BN;
        bool bad = false;
        for (int kb = 0; kb < kBlocks; ++kb, ++kc) {
          const int s = kc % P_STAGES;
          const uint32_t ph = (kc / P_STAGES) & 1;
          if (!mbarWait(smemAddr(&fullBar[s]), ph)) { fail(WAIT_TILE, 3000 + s); bad = true; break; }
          tcFenceAfter();
          const uint32_t aAddr = smemA0 + s * kHalfBytes, bAddr = smemB0 + s * kHalfBytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            ummaBf16Pair(dT, umDescK128(aAddr + k * UMMA_K * 2), umDescK128(bAddr + k * UMMA_K * 2), idesc, (kb | k) != 0);
          ummaCommitPair(smemAddr(&emptyBar[s]), 3);   // stage s is free in both CTAs once these MMAs have read it
        }
        if (bad) break;
        ummaCommitPair(smemAddr(&accFull[buf]), 3);    // accumulator complete, in both CTAs
      }
    }
  } else {
    // ---- epilogue warps: TMEM lanes [32q, 32q+32) belong to the warp with warp % 4 == q
    const int q = warp & 3;
    uint8_t* wbuf = epiBuf + (size_t)(warp - 2) * 4096;
    int it = 0;
    for (int t = pairIdx; t < nTiles && !*abortFlag; t += nPairs, ++it) {
      const TileCoord tc = tileOf(a, t, PM);
      const int buf = it % kAccBufs;
      const uint32_t aph = (it / kAccBufs) & 1;
      if (!mbarWait(smemAddr(&accFull[buf]), aph)) { if (lane == 0) fail(WAIT_TILE, 4000 + buf); break; }
      tcFenceAfter();
      const int row0 = tc.mBlk * PM + (int)cr * 128 + q * 32;
      const uint32_t tBase = tmemBase + ((uint32_t)(q * 32) << 16) + buf * BN;
      tpStoreAccum(a, tBase, row0, tc.nBlk, tc.owner, wbuf, lane);
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArriveCluster(mapaShared(smemAddr(&accEmpty[buf]), 0));
    }
  }

  // ---- teardown: the pair meets (nobody touches the partner's shared or tensor memory afterwards),
  // tensor memory goes back, then the cross-GPU barrier
  tcFenceBefore();
  __syncthreads();
  __syncwarp();
  clusterSync();
  if (warp == 1) {
    tcFenceAfter();
    tmemDeallocPair(tmemBase, kTmemCols);
  }
  if (multi) {
    bar.sync(true, false);
    bar.finish();
  }
}

const void* tpGemmPairKernelFn() { return (const void*)tpGemmPairKernel; }
size_t tpGemmPairSmemBytes() { return kSmemBytes; }
int tpGemmPairThreads() { return kThreads; }

}  // namespace b200
