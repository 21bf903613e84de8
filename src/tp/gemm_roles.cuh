// Roles shared by the one-CTA and the CTA-pair tensor-parallel GEMM kernels: the all-gather role
// of the extra "comm" CTAs and the epilogue that moves one accumulator tile from tensor memory to
// global memory (this GPU's or a peer's).
#pragma once
#include "gemm_sm100.cuh"

#include "../kernels/common.cuh"
#include "tp.h"

namespace b200 {

constexpr int kTpBK = 64;
constexpr int kTpPipeStages = 6;
constexpr uint32_t kTpPipeChunk = 32768;
constexpr size_t kTpPipeBytes = (size_t)kTpPipeStages * kTpPipeChunk;

__device__ __forceinline__ void tpReportTimeout(const TpGemmArgs& a, uint32_t kind, uint32_t what) {
  uint32_t* st = a.sync.status[a.rank];
  if (st && ldRelaxedSys(st) == DEV_OK) {
    st[1] = kind;
    st[2] = what;
    st[3] = blockIdx.x;
    __threadfence_system();
    stRelaxedSys(st, DEV_TIMEOUT);
  }
}

// All-gather role of comm CTA `commIdx` of `commN`: pulls the other ranks' 128-row blocks of A from
// their windows into the local buffer in the order the GEMM consumes them (rank+1 first), blocks
// dealt round-robin to the comm CTAs, and publishes a flag per block. One thread drives bulk copies
// peer -> shared memory -> local rows through `smemRing` (kTpPipeBytes, 128-byte aligned);
// `pipeBars` are kTpPipeStages uninitialised mbarriers. Returns false after a wait ran out.
__device__ __forceinline__ bool tpCommRole(const TpGemmArgs& a, int commIdx, int commN, uint8_t* smemRing, uint64_t* pipeBars, bool ok) {
  using namespace sm100;
  const int rank = a.rank, n = a.nRanks;
  const int blocksPerRank = a.M / n / kTpBM;
  const size_t blockBytes = (size_t)kTpBM * a.K * 2;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kTpPipeStages; ++s) mbarInit(smemAddr(&pipeBars[s]), 1);
    mbarInitFence();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t phaseBits = 0;
    for (int idx = commIdx; idx < (n - 1) * blocksPerRank && ok; idx += commN) {
      const int src = (rank + 1 + idx / blocksPerRank) % n;
      const int mb = src * blocksPerRank + idx % blocksPerRank;
      const char* from = (const char*)a.peerA[src] + (size_t)mb * blockBytes;
      char* to = (char*)a.peerA[rank] + (size_t)mb * blockBytes;
      ok = bulkPipe<kTpPipeStages, kTpPipeChunk>(to, from, blockBytes, smemAddr(smemRing), pipeBars, phaseBits);
      if (!ok) { tpReportTimeout(a, WAIT_TILE, 5000 + mb); break; }
      // the rows were written through the async proxy and will be read by TMA loads of other CTAs
      fenceProxyAsync();
      __threadfence();
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a.blockFlags + mb), "r"(a.flagEpoch) : "memory");
    }
  }
  __syncthreads();
  return ok;
}

// Waits (bounded) until the comm CTAs have landed 128-row block `mb`; `abortFlag` ends the wait early.
__device__ __forceinline__ bool tpWaitBlock(const TpGemmArgs& a, int mb, volatile uint32_t* abortFlag) {
  const uint32_t* f = a.blockFlags + mb;
  for (uint32_t spin = 0; spin < (1u << 26); ++spin) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if ((int32_t)(v - a.flagEpoch) >= 0) { sm100::fenceProxyAsync(); return true; }
    if (*abortFlag) break;
  }
  return false;
}

// Epilogue of one warp for its 32 rows x 256 columns of an accumulator: tBase is the tensor-memory
// address of the warp's first lane and the tile's first column, row0 the global row of that lane.
// STORE / GATHER write C; REDUCE writes slot `rank` of the staging buffer of the rank that owns the rows
// (over NVLink when that is a peer). Each lane owns one row of the accumulator, so storing straight
// from registers would write 16 scattered bytes per lane and instruction. The warp instead
// transposes 64 columns at a time through 4 KiB of shared memory (16-byte chunks XOR-swizzled by
// row against bank conflicts) and writes 128 contiguous bytes per row, four rows per instruction:
// whole lines for HBM and NVLink.
__device__ __forceinline__ void tpStoreAccum(const TpGemmArgs& a, uint32_t tBase, int row0, int nBlk, int owner, uint8_t* wbuf, int lane) {
  using namespace sm100;
  __nv_bfloat16* dstBase;
  size_t ld;
  if (a.mode == TP_MODE_REDUCE && a.nRanks > 1) {
    const int rowsPerRank = a.M / a.nRanks;
    dstBase = (__nv_bfloat16*)a.partial[owner] + ((size_t)a.rank * rowsPerRank + (row0 - owner * rowsPerRank)) * a.N + (size_t)nBlk * kTpBN;
    ld = (size_t)a.N;
  } else {
    dstBase = (__nv_bfloat16*)a.C + (size_t)row0 * a.ldc + (size_t)nBlk * kTpBN;
    ld = (size_t)a.ldc;
  }
  for (int cc = 0; cc < kTpBN / 64; ++cc) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t r[32];
      tmemLd32(tBase + (cc * 2 + half) * 32, r);
      tmemLdWait();
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        uint4 o;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[8 * v]), __uint_as_float(r[8 * v + 1]));
        __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
        __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
        __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
        o.x = *(uint32_t*)&p0; o.y = *(uint32_t*)&p1; o.z = *(uint32_t*)&p2; o.w = *(uint32_t*)&p3;
        const int j = half * 4 + v;   // 16-byte chunk of the 128-byte row segment
        *(uint4*)(wbuf + lane * 128 + ((j ^ (lane & 7)) * 16)) = o;
      }
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

}  // namespace b200
