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
#include "../tp/gemm_sm100.cuh"

namespace b200 {

constexpr int kEpThreads = 512;
constexpr int kStCounters = 8;   // first per-expert counter inside state[]

__device__ __forceinline__ void stReleaseSys64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__global__ void __launch_bounds__(kEpThreads, 1) epDispatchKernel(const __grid_constant__ EpArgs a) {
  extern __shared__ uint8_t epSmem[];   // one packed token: payload (+ scales)
  __shared__ int sCnt[kMaxRanks], sOff[kMaxRanks + 1];
  __shared__ int sCell[kEpMaxCells], sExpOff[kEpMaxLocalExperts + 1];   // expert-major receive: per (expert, source) and per expert
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
  // With bulkStages > 0 the packed token is written into one stage of a shared-memory ring and leaves through the bulk-copy
  // engine (cp.async.bulk shared -> peer memory): lanes of warp 0 claim the slots, store the headers and issue one bulk store
  // per destination; the warps go on to quantise the next token while earlier ones drain. A stage is reused once the bulk
  // groups that read it have finished reading.
  const int nStages = a.bulkStages > 0 ? a.bulkStages : 1;
  const size_t stageBytes = a.bulkStages > 0 ? epStageBytes(H, a.fp8) : 0;
  uint8_t* const smBase = (uint8_t*)(((uintptr_t)epSmem + 127) & ~(uintptr_t)127);
  int iter = 0;
  for (int t = blockIdx.x; sendPhase && t < T; t += gridDim.x, ++iter) {
    uint8_t* const stage = smBase + (size_t)(iter % nStages) * stageBytes;
    if (a.bulkStages > 0 && iter >= nStages) {
      if (warp == 0) sm100::bulkWaitRead<kEpBulkStages - 1>();   // the groups of the token that used this stage have read it
      __syncthreads();
    }
    const __nv_bfloat16* row = x + (size_t)t * H;
    if (a.fp8) {
      float* scales = (float*)(stage + H);
      // four groups of 128 channels per warp and round: the loads of a round are issued together, so a token costs one
      // trip to memory per round instead of one per group
      for (int g0 = warp; g0 < H / 128; g0 += 4 * nWarps) {
        uint2 raws[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int g = g0 + u * nWarps;
          raws[u] = g < H / 128 ? *(const uint2*)(row + g * 128 + lane * 4) : make_uint2(0, 0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int g = g0 + u * nWarps;
          if (g >= H / 128) break;
          const uint2 raw = raws[u];
          __nv_bfloat162 p0 = *(const __nv_bfloat162*)&raw.x, p1 = *(const __nv_bfloat162*)&raw.y;
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
          *(uint32_t*)(stage + g * 128 + lane * 4) = packed;
          if (lane == 0) scales[g] = scale;
        }
      }
    } else {
      for (int i = threadIdx.x; i < H / 8; i += kEpThreads) ((uint4*)stage)[i] = ((const uint4*)row)[i];
    }
    if (a.bulkStages > 0) sm100::fenceProxyAsync();   // the bulk-copy engine reads what the threads just wrote
    __syncthreads();
    if (a.layout != EP_EXPERT_MAJOR && a.bulkStages > 0) {
      // one copy per destination rank; lane d of warp 0 serves destination d
      if (warp == 0) {
        const size_t slotR = slotBytes + epMetaBytes(K);
        const size_t zoneR = (size_t)(epoch & 1) * ((size_t)n * a.maxTokens * slotR);
        if (lane < n && !(mask && mask[lane])) {
          const int dst = lane;
          bool any = false;
          for (int k = 0; k < K; ++k) {
            const long long e = a.topkIdx[rank][(size_t)t * K + k];
            any = any || (e >= 0 && e < E && (int)(e / El) == dst);
          }
          int s = t;
          if (any && a.layout == EP_FLAT) s = (int)atomicAdd(&st[kStCounters + dst], 1u);
          if (any && s < a.maxTokens) {
            char* slot = a.recvBuf[dst] + zoneR + ((size_t)rank * a.maxTokens + s) * slotR;
            *(int4*)slot = make_int4(t, (int)epoch, 0, 0);
            sm100::bulkStore(slot + 16, sm100::smemAddr(stage), (uint32_t)payload);
            for (int k = 0; k < K; ++k) {
              const long long e = a.topkIdx[rank][(size_t)t * K + k];
              const bool local = e >= 0 && e < E && (int)(e / El) == dst;
              const float wk = a.topkW[rank] ? a.topkW[rank][(size_t)t * K + k] : 0.0f;
              *(int2*)(slot + slotBytes + (size_t)k * 8) = make_int2(local ? (int)e : -1, __float_as_int(wk));
            }
          }
        }
        sm100::bulkCommit();   // every lane, every token: the number of groups counts the tokens, which is what the stage reuse relies on
      }
      continue;
    }
    if (a.layout != EP_EXPERT_MAJOR) {
      // one copy per destination rank: a warp per rank looks whether any of the token's experts lives there
      const size_t slotR = slotBytes + epMetaBytes(K);
      const size_t zoneR = (size_t)(epoch & 1) * ((size_t)n * a.maxTokens * slotR);
      long long eK = -1;
      float wK = 0.0f;
      if (lane < K) {
        eK = a.topkIdx[rank][(size_t)t * K + lane];
        if (eK < 0 || eK >= E) eK = -1;
        if (a.topkW[rank]) wK = a.topkW[rank][(size_t)t * K + lane];
      }
      for (int dst = warp; dst < n; dst += nWarps) {
        const bool local = eK >= 0 && (int)(eK / El) == dst;
        if (__ballot_sync(0xffffffffu, local) == 0u) continue;
        if (mask && mask[dst]) continue;
        int s = t;   // rank-major: the row is the token's index
        if (a.layout == EP_FLAT) {
          if (lane == 0) s = (int)atomicAdd(&st[kStCounters + dst], 1u);
          s = __shfl_sync(0xffffffffu, s, 0);
        }
        if (s >= a.maxTokens) continue;
        char* slot = a.recvBuf[dst] + zoneR + ((size_t)rank * a.maxTokens + s) * slotR;
        if (lane == 0) *(int4*)slot = make_int4(t, (int)epoch, 0, 0);
        for (size_t i = lane; i < payload / 16; i += 32) st16(slot + 16 + i * 16, ((const uint4*)stage)[i]);
        if (lane < K) *(int2*)(slot + slotBytes + (size_t)lane * 8) = make_int2(local ? (int)eK : -1, __float_as_int(wK));
      }
      __syncthreads();
      continue;
    }
    if (a.bulkStages > 0) {
      // warp 0: lane k serves the token's k-th expert (slot claim, header, one bulk store)
      if (warp == 0) {
        const long long e = lane < K ? a.topkIdx[rank][(size_t)t * K + lane] : -1;
        if (e >= 0 && e < E) {
          const int dst = (int)(e / El), el = (int)(e % El);
          if (!(mask && mask[dst])) {
            const int s = (int)atomicAdd(&st[kStCounters + e], 1u);
            if (s < a.maxTokens) {
              char* slot = a.recvBuf[dst] + zoneOff + ((size_t)(el * n + rank) * a.maxTokens + s) * slotBytes;
              *(int4*)slot = make_int4(t * K + lane, 0, 0, 0);
              sm100::bulkStore(slot + 16, sm100::smemAddr(stage), (uint32_t)payload);
            }
          }
        }
        sm100::bulkCommit();   // every lane, every token (empty groups included): groups count tokens
      }
      continue;   // no barrier: the next token goes into another stage
    }
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
      for (size_t i = lane; i < payload / 16; i += 32) st16(slot + 16 + i * 16, ((const uint4*)stage)[i]);
    }
    __syncthreads();
  }
  // everything this CTA handed to the bulk-copy engine has been written before the counts go out
  if (a.bulkStages > 0 && sendPhase) sm100::bulkWaitAll();
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
  if (sIsLast && a.layout != EP_EXPERT_MAJOR) {
    __threadfence();
    if (threadIdx.x < n) {
      const int dst = threadIdx.x;
      const uint32_t c = a.layout == EP_FLAT ? st[kStCounters + dst] : (uint32_t)T;   // rank-major: rows [0, T) may be in use
      st[kStCounters + dst] = 0;
      if (!(mask && mask[dst])) stReleaseSys64(a.recvCount[dst] + cntOff + rank, ((unsigned long long)epoch << 32) | c);
    }
  } else if (sIsLast) {
    // The count of a destination's LAST local expert is the word its receivers poll: it goes out after the counts of the
    // other experts (one word to watch per source instead of one per expert and source).
    __threadfence();
    for (int e = threadIdx.x; e < E; e += kEpThreads) {
      const int dst = e / El, el = e % El;
      if (el == El - 1) continue;
      const uint32_t c = st[kStCounters + e];
      st[kStCounters + e] = 0;
      if (mask && mask[dst]) continue;
      stReleaseSys64(a.recvCount[dst] + cntOff + (size_t)el * n + rank, ((unsigned long long)epoch << 32) | c);
    }
    __threadfence_system();
    __syncthreads();   // sIsLast is the same for the whole CTA
    if (threadIdx.x < n) {
      const int dst = threadIdx.x, e = dst * El + El - 1;
      const uint32_t c = st[kStCounters + e];
      st[kStCounters + e] = 0;
      if (!(mask && mask[dst])) stReleaseSys64(a.recvCount[dst] + cntOff + (size_t)(El - 1) * n + rank, ((unsigned long long)epoch << 32) | c);
    }
  }
  if (!recvPhase) return;   // split-phase call: ncclEpComplete runs the receiving half

  // ---------------------------------------------------------------- receive and pack
  const int cap = n * a.maxTokens;
  const size_t rowBytes = a.fp8 ? (size_t)H : (size_t)H * 2;
  bool ok = true;
  if (a.layout != EP_EXPERT_MAJOR) {
    // every CTA waits for the n count words (they are local), then the CTAs share the rows
    const size_t slotR = slotBytes + epMetaBytes(K);
    const size_t zoneR = (size_t)(epoch & 1) * ((size_t)n * a.maxTokens * slotR);
    if (threadIdx.x < n) {
      const unsigned long long* c = a.recvCount[rank] + cntOff + threadIdx.x;
      unsigned long long v = 0;
      int cnt = 0;
      if (!(mask && mask[threadIdx.x])) {
        const bool quiet = a.enableMask && mask;
        bool got = boundedWait(w, WAIT_TILE, threadIdx.x, epoch, [&] {
          v = ldRelaxedSys64((const uint64_t*)c);
          if ((uint32_t)(v >> 32) == epoch) return true;
          __nanosleep(200);
          return false;
        }, !quiet);
        fenceSys();
        if (got) cnt = (int)(uint32_t)v;
        else if (quiet && !(a.sync.abortFlag && ldRelaxedSys(a.sync.abortFlag))) { mask[threadIdx.x] = 1; cnt = 0; }
        else cnt = -1;
      }
      sCnt[threadIdx.x] = cnt;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int off = 0;
      for (int s = 0; s < n; ++s) { sOff[s] = off; off += sCnt[s] > 0 ? sCnt[s] : 0; if (sCnt[s] < 0) off = -1 << 30; }
      sOff[n] = off;
    }
    __syncthreads();
    ok = sOff[n] >= 0;
    if (ok) {
      const bool flat = a.layout == EP_FLAT;
      const int total = sOff[n];
      const int rows = flat ? (a.outSlots < cap ? a.outSlots : cap) : cap;
      if (flat && blockIdx.x == 0 && threadIdx.x == 0 && a.recvTotal[rank]) *a.recvTotal[rank] = total;
      for (int pos = blockIdx.x * nWarps + warp; pos < rows; pos += gridDim.x * nWarps) {
        int s, j;
        bool valid;
        if (flat) {
          s = 0;
          while (s + 1 < n && pos >= sOff[s + 1]) ++s;
          j = pos - sOff[s];
          valid = pos < total;
        } else {
          s = pos / a.maxTokens;
          j = pos - s * a.maxTokens;
          valid = j < sCnt[s];
        }
        const char* slot = a.recvBuf[rank] + zoneR + ((size_t)s * a.maxTokens + j) * slotR;
        int4 hdr = make_int4(0, 0, 0, 0);
        if (valid) hdr = *(const int4*)slot;
        valid = valid && (uint32_t)hdr.y == epoch;   // rank-major: a row that was not written in this call keeps an older epoch
        if (lane == 0) a.srcInfo[rank][pos] = valid ? make_int2(s, hdr.x) : make_int2(-1, 0);
        if (lane < K) {
          int2 meta = valid ? *(const int2*)(slot + slotBytes + (size_t)lane * 8) : make_int2(-1, 0);
          if (a.outTopkIdx[rank]) a.outTopkIdx[rank][(size_t)pos * K + lane] = meta.x;
          if (a.outTopkW[rank]) a.outTopkW[rank][(size_t)pos * K + lane] = __int_as_float(meta.y);
          if (meta.x >= 0 && a.expertCount[rank]) atomicAdd(&a.expertCount[rank][meta.x - rank * El], 1);
        }
        if (!valid) continue;
        char* dstTok = (char*)a.outTokens[rank] + (size_t)pos * rowBytes;
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
        if (a.fp8) {
          const float* sc = (const float*)(slot + 16 + H);
          float* dsc = a.outScales[rank] + (size_t)pos * (H / 128);
          for (int q = lane; q < H / 128; q += 32) dsc[q] = sc[q];
        }
      }
    }
  }
  if (a.layout == EP_EXPERT_MAJOR) {
    // Every CTA waits for the counts of all (local expert, source) cells (the words are local), then the warps of ALL CTAs
    // share the rows of all experts: the packing is spread over the whole grid, not over one CTA per expert.
    const int cells = El * n;
    // One thread per source watches the count of the last local expert (the sender writes it after all others), with a pause
    // between polls: thousands of threads spinning on these words would compete with the rows that are still arriving.
    if (threadIdx.x < n) {
      const int s = threadIdx.x;
      const unsigned long long* cw = a.recvCount[rank] + cntOff + (size_t)(El - 1) * n + s;
      int state = 0;   // 1: counts are there, 0: source is left out, -1: the wait failed
      if (!(mask && mask[s])) {
        const bool quiet = a.enableMask && mask;
        unsigned long long v = 0;
        bool got = boundedWait(w, WAIT_TILE, (uint32_t)s, epoch, [&] {
          v = ldRelaxedSys64((const uint64_t*)cw);
          if ((uint32_t)(v >> 32) == epoch) return true;
          __nanosleep(200);
          return false;
        }, !quiet);
        if (got) state = 1;
        else if (quiet && !(a.sync.abortFlag && ldRelaxedSys(a.sync.abortFlag))) { mask[s] = 1; state = 0; }   // left out from now on; the call goes on without it
        else state = -1;
      }
      sCnt[s] = state;
    }
    fenceSys();
    __syncthreads();
    for (int c = threadIdx.x; c < cells; c += kEpThreads) {
      const int s = c % n;
      int cnt = sCnt[s] > 0 ? 0 : sCnt[s];
      if (sCnt[s] > 0) {
        const unsigned long long v = ldRelaxedSys64((const uint64_t*)(a.recvCount[rank] + cntOff + c));
        cnt = (uint32_t)(v >> 32) == epoch ? (int)(uint32_t)v : -1;   // written before the word that was polled: anything else is a protocol error
      }
      sCell[c] = cnt;
    }
    fenceSys();   // acquire: the rows behind the counts
    __syncthreads();
    if (threadIdx.x == 0) {
      int off = 0;
      bool bad = false;
      for (int el = 0; el < El; ++el) {
        sExpOff[el] = off;
        int inExp = 0;
        for (int s = 0; s < n; ++s) {
          const int c = sCell[el * n + s];
          if (c < 0) bad = true;
          sCell[el * n + s] = inExp;            // from now on: first row of this source inside the expert
          inExp += c > 0 ? c : 0;
        }
        if (blockIdx.x == 0 && !bad) a.expertCount[rank][el] = inExp;
        off += inExp;
      }
      sExpOff[El] = bad ? -1 : off;
    }
    __syncthreads();
    ok = sExpOff[El] >= 0;
    if (ok) {
      const int total = sExpOff[El];
      for (int g = blockIdx.x * nWarps + warp; g < total; g += gridDim.x * nWarps) {
        // which expert: the last one whose first row is <= g
        int lo = 0, hi = El - 1;
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (sExpOff[mid] <= g) lo = mid; else hi = mid - 1;
        }
        const int el = lo, pos = g - sExpOff[el];
        int s = 0;
        while (s + 1 < n && pos >= sCell[el * n + s + 1]) ++s;
        const int j = pos - sCell[el * n + s];
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

constexpr int kCombStaged = 64;   // tokens of one CTA whose routing is staged in shared memory
constexpr int kCombMaxK = 16;

__global__ void __launch_bounds__(kEpThreads, 1) epCombineKernel(const __grid_constant__ EpArgs a) {
  __shared__ int sIsLast, sOk;
  __shared__ int sExpOffC[kEpMaxLocalExperts + 1];
  __shared__ float sCombW[kCombStaged * kCombMaxK];
  __shared__ unsigned char sCombUse[kCombStaged * kCombMaxK];
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
  if (sendPhase && a.layout != EP_EXPERT_MAJOR) {
    // one pre-reduced row per received token goes to row (token, this rank) of its source rank
    const size_t combOffR = (size_t)(epoch & 1) * ((size_t)a.maxTokens * n * H * 2);
    const int rows = a.layout == EP_FLAT ? (a.outSlots < cap ? a.outSlots : cap) : cap;
    for (int pos = blockIdx.x * nWarps + warp; pos < rows; pos += gridDim.x * nWarps) {
      const int2 info = a.srcInfo[rank][pos];
      if (info.x < 0 || (mask && mask[info.x])) continue;
      const char* src = (const char*)(y + (size_t)pos * H);
      char* dst = a.combBuf[info.x] + combOffR + ((size_t)info.y * n + rank) * H * 2;
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
  if (sendPhase && a.layout == EP_EXPERT_MAJOR) {
    // the rows of all local experts form one list that the warps of all CTAs share (an expert with few rows costs no round of its own)
    if (threadIdx.x == 0) {
      int off = 0;
      for (int el = 0; el < El; ++el) { sExpOffC[el] = off; off += a.expertCount[rank][el]; }
      sExpOffC[El] = off;
    }
    __syncthreads();
    const int total = sExpOffC[El];
    for (int g = blockIdx.x * nWarps + warp; g < total; g += gridDim.x * nWarps) {
      int lo = 0, hi = El - 1;   // the last expert whose first row is <= g
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (sExpOffC[mid] <= g) lo = mid; else hi = mid - 1;
      }
      const size_t o = (size_t)lo * cap + (g - sExpOffC[lo]);
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
    bool got = boundedWait(w, WAIT_TILE, threadIdx.x, epoch, [&] {
      if ((int32_t)((uint32_t)ldRelaxedSys64((const uint64_t*)f) - epoch) >= 0) return true;
      __nanosleep(200);   // a pause between polls: every CTA of the rank watches these words while rows are still arriving
      return false;
    }, !quiet);
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
    for (int t = blockIdx.x; a.layout != EP_EXPERT_MAJOR && t < T; t += gridDim.x) {
      // which ranks hold an expert of this token: one row each, already weighted by the caller
      const size_t combOffR = (size_t)(epoch & 1) * ((size_t)a.maxTokens * n * H * 2);
      unsigned hit = 0;
      for (int k = 0; k < K; ++k) {
        const long long e = a.topkIdx[rank][(size_t)t * K + k];
        if (e >= 0 && e < a.numExperts && !(mask && mask[e / El])) hit |= 1u << (int)(e / El);
      }
      for (int c = threadIdx.x; c < H / 8; c += kEpThreads) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        uint4 v[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
          v[r] = make_uint4(0, 0, 0, 0);
          if (r < n && ((hit >> r) & 1u)) v[r] = ldLocal16(a.combBuf[rank] + combOffR + (((size_t)t * n + r) * H + (size_t)c * 8) * 2);
        }
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
          const __nv_bfloat162* p = (const __nv_bfloat162*)&v[r];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[2 * i] += __bfloat162float(p[i].x);
            acc[2 * i + 1] += __bfloat162float(p[i].y);
          }
        }
        uint4 o;
        __nv_bfloat162* q = (__nv_bfloat162*)&o;
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        *(uint4*)(out + (size_t)t * H + (size_t)c * 8) = o;
      }
    }
    // The routing (which of a token's experts count, and their weights) of the first kCombStaged tokens of this CTA goes to shared
    // memory first: the loop below then waits for one trip to memory per token (the rows) instead of two (routing, then rows).
    int staged = 0;
    if (a.layout == EP_EXPERT_MAJOR && K <= kCombMaxK) {
      const int mine = T > (int)blockIdx.x ? (T - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
      staged = mine < kCombStaged ? mine : kCombStaged;
      for (int i = threadIdx.x; i < staged * K; i += kEpThreads) {
        const int t = (int)blockIdx.x + (i / K) * (int)gridDim.x, k = i % K;
        const long long e = a.topkIdx[rank][(size_t)t * K + k];
        const bool use = e >= 0 && e < a.numExperts && !(mask && mask[e / El]);
        sCombUse[i] = use ? 1 : 0;
        sCombW[i] = use ? a.topkW[rank][(size_t)t * K + k] : 0.0f;
      }
      __syncthreads();
    }
    int j = 0;
    for (int t = blockIdx.x; a.layout == EP_EXPERT_MAJOR && t < T; t += gridDim.x, ++j) {
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
              bool use;
              float wgt;
              if (j < staged) {
                use = sCombUse[j * K + k] != 0;
                wgt = sCombW[j * K + k];
              } else {
                const long long e = a.topkIdx[rank][(size_t)t * K + k];
                use = e >= 0 && e < a.numExperts && !(mask && mask[e / El]);
                wgt = use ? a.topkW[rank][(size_t)t * K + k] : 0.0f;
              }
              if (use) {
                wk[u] = wgt;
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
