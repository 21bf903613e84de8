// Neighbour-ring and double-binary-tree schedules over peer-mapped work buffers.
// These are the classic bandwidth-optimal (ring) and latency-optimal (tree) schedules of the
// reference's channel kernels, kept for parity (NCCL_ALGO=Ring / Tree) and for fabrics where not
// every pair of ranks is directly connected. Instead of FIFO staging with proxy threads, a step
// reads the neighbour's work buffer directly and publishes a step counter to the next rank.
//   ringKernel   all-reduce (reduce-scatter steps then all-gather steps), reduce-scatter, all-gather,
//                in place on a symmetric work buffer W; each CTA owns a contiguous range of W and
//                runs its own ring over that range.
//   treeKernel   all-reduce: partial sums flow up two complementary binary trees (each tree owns
//                half of a CTA's range), totals flow back down.
// Reference parity: src/device/all_reduce.h:14-83 (runRing), :86-225 (trees), all_gather.h:14-89,
// reduce_scatter.h:14-56, src/graph/rings.cc, src/graph/trees.cc (tree shapes).
#include "common.cuh"
#include "launch.h"
#include "../comm/comm.h"

namespace b200 {

// dst[i] = op(dst[i], src[i]) or dst[i] = src[i] over `cnt` elements starting at element `off`.
template <typename T, int OP, bool REDUCE>
__device__ __forceinline__ void rangeOp(char* dstBase, const char* srcBase, size_t off, size_t cnt, bool vec16) {
  constexpr int N = 16 / sizeof(T);
  T* dst = (T*)dstBase + off;
  const T* src = (const T*)srcBase + off;
  size_t nPacks = vec16 ? cnt / N : 0;
  for (size_t i = threadIdx.x; i < nPacks; i += blockDim.x) {
    uint4 s = ldStream16((const char*)src + i * 16);
    if (REDUCE) {
      PackAcc<T, OP> acc;
      acc.set(ldLocal16((const char*)dst + i * 16));
      acc.add(s);
      s = acc.get(SCALE_NONE, 1.f, 1.0, 1);
    }
    st16((char*)dst + i * 16, s);
  }
  for (size_t e = nPacks * N + threadIdx.x; e < cnt; e += blockDim.x) {
    if (REDUCE) dst[e] = Elem<T>::st(redApply<OP>(Elem<T>::ld(dst[e]), Elem<T>::ld(src[e])));
    else dst[e] = src[e];
  }
}

template <typename T, int OP>
__device__ __forceinline__ void rangeScale(char* base, size_t off, size_t cnt, const CollArgs& a) {
  T* p = (T*)base + off;
  for (size_t e = threadIdx.x; e < cnt; e += blockDim.x) p[e] = scalarPost<T, OP>(Elem<T>::ld(p[e]), a);
}

struct StepFlags {
  WaitCtx w;
  uint32_t* mine;          // my flag words for this slot: [src]
  uint32_t base;
  __device__ __forceinline__ void post(uint32_t* peerWords, int me, uint32_t value) {
    __syncthreads();
    if (threadIdx.x == 0) {
      fenceSys();
      stRelaxedSys(peerWords + me, value);
    }
  }
  __device__ __forceinline__ bool wait(int src, uint32_t value) {
    bool ok = true;
    if (threadIdx.x == 0) {
      const uint32_t* p = mine + src;
      ok = boundedWait(w, WAIT_TILE, (uint32_t)src, value, [&] { return (int32_t)(ldRelaxedSys(p) - value) >= 0; });
      fenceSys();
    }
    return __syncthreads_and(ok);
  }
};

// Contiguous element range of CTA `c` out of `nc`, cut at multiples of `unit` elements.
__device__ __forceinline__ void ctaRange(size_t count, size_t unit, int c, int nc, size_t* b, size_t* e) {
  size_t units = (count + unit - 1) / unit;
  size_t per = (units + nc - 1) / nc;
  size_t ub = (size_t)c * per, ue = ub + per;
  *b = ub * unit < count ? ub * unit : count;
  *e = ue * unit < count ? ue * unit : count;
}

template <typename T, int OP>
__global__ void __launch_bounds__(kCtaThreads, 1) ringKernel(const __grid_constant__ CollArgs a) {
  const int rank = ctaRank(a.emu, a.rank);
  const int n = a.nRanks;
  const int slot = blockIdx.x;
  const int next = (rank + 1) % n, prev = (rank + n - 1) % n;
  constexpr size_t unit = 16 / sizeof(T);
  pdlEnter();
  KernelStamp stamp(a.sync.stamps);
  CtaBarrier bar;
  bar.init(a.sync, rank, n, slot);
  uint32_t* basePtr = a.sync.epoch[rank] + kPrivRingBase + slot;
  StepFlags f;
  f.w = bar.w;
  f.mine = (uint32_t*)((char*)a.sync.inbox[rank] + kOffRingFlags) + (size_t)slot * kMaxRanks;
  f.base = *basePtr;
  uint32_t* nextWords = (uint32_t*)((char*)a.sync.inbox[next] + kOffRingFlags) + (size_t)slot * kMaxRanks;
  char* W = (char*)a.recv[rank];
  const char* Wprev = (const char*)a.recv[prev];
  bool ok = bar.sync(false, false);   // every rank's work buffer holds its input (copied in by an earlier stream operation)
  // this CTA's range, cut in n chunks
  size_t rb, re;
  const bool gatherOnly = a.func == FUNC_ALLGATHER;
  // all-gather and reduce-scatter move whole per-rank blocks of a.count elements: chunk c = block c
  const bool blocks = a.func != FUNC_ALLREDUCE;
  const size_t total = blocks ? a.count : a.count;
  ctaRange(total, unit, slot, gridDim.x, &rb, &re);
  auto chunkOf = [&](int c, size_t* off, size_t* cnt) {
    if (blocks) { *off = (size_t)c * a.count + rb; *cnt = re - rb; return; }
    size_t len = re - rb;
    size_t per = ((len + n - 1) / n + unit - 1) / unit * unit;
    size_t b = (size_t)c * per < len ? (size_t)c * per : len;
    size_t e = b + per < len ? b + per : len;
    *off = rb + b;
    *cnt = e - b;
  };
  uint32_t step = 0;
  const int rsShift = a.func == FUNC_REDUCESCATTER ? -1 : 0;   // reduce-scatter leaves chunk r on rank r
  if (!gatherOnly) {
    for (int s = 0; s < n - 1 && ok; ++s, ++step) {
      if (step > 0) ok = f.wait(prev, f.base + step);
      if (!ok) break;
      int c = ((rank - s - 1 + rsShift) % n + 2 * n) % n;
      size_t off, cnt;
      chunkOf(c, &off, &cnt);
      rangeOp<T, OP, true>(W, Wprev, off, cnt, a.vec16);
      f.post(nextWords, rank, f.base + step + 1);
    }
  }
  if (a.func == FUNC_ALLREDUCE && ok) {
    // the chunk this rank completed gets its post-scale (average) before it travels on
    if (a.scaleMode != SCALE_NONE) {
      size_t off, cnt;
      chunkOf((rank + 1) % n, &off, &cnt);
      __syncthreads();
      rangeScale<T, OP>(W, off, cnt, a);
    }
  }
  if (a.func == FUNC_REDUCESCATTER && ok && a.scaleMode != SCALE_NONE) {
    size_t off, cnt;
    chunkOf(rank, &off, &cnt);
    __syncthreads();
    rangeScale<T, OP>(W, off, cnt, a);
  }
  if (a.func != FUNC_REDUCESCATTER) {
    const int own = a.func == FUNC_ALLREDUCE ? 1 : 0;   // chunk (rank + own) is complete here
    for (int s = 0; s < n - 1 && ok; ++s, ++step) {
      // the neighbour must have finished the step that completed the chunk I am about to copy
      if (step > 0) ok = f.wait(prev, f.base + step);
      if (!ok) break;
      int c = ((rank + own - s - 1) % n + 2 * n) % n;
      size_t off, cnt;
      chunkOf(c, &off, &cnt);
      rangeOp<T, OP, false>(W, Wprev, off, cnt, a.vec16);
      f.post(nextWords, rank, f.base + step + 1);
    }
  }
  // steps that were not run (failed wait) still advance the base identically on every rank
  const uint32_t planned = (gatherOnly ? 0 : n - 1) + (a.func != FUNC_REDUCESCATTER ? n - 1 : 0);
  bar.sync(true, false);  // nobody still reads my work buffer
  if (threadIdx.x == 0) *basePtr = f.base + planned;
  bar.finish();
}

// Binary tree in heap order over "virtual" ranks; tree 1 mirrors the ranks so that interior nodes
// of one tree are leaves of the other.
__device__ __forceinline__ int treeReal(int v, int tree, int n) { return tree == 0 ? v : n - 1 - v; }

template <typename T, int OP>
__global__ void __launch_bounds__(kCtaThreads, 1) treeKernel(const __grid_constant__ CollArgs a) {
  const int rank = ctaRank(a.emu, a.rank);
  const int n = a.nRanks;
  const int slot = blockIdx.x;
  constexpr size_t unit = 16 / sizeof(T);
  pdlEnter();
  KernelStamp stamp(a.sync.stamps);
  CtaBarrier bar;
  bar.init(a.sync, rank, n, slot);
  uint32_t* basePtr = a.sync.epoch[rank] + kPrivTreeBase + slot;
  const uint32_t base = *basePtr;
  char* W = (char*)a.recv[rank];
  bool ok = bar.sync(false, false);
  size_t rb, re;
  ctaRange(a.count, unit, slot, gridDim.x, &rb, &re);
  const size_t half = ((re - rb) / 2 + unit - 1) / unit * unit;
  for (int tree = 0; tree < 2 && ok; ++tree) {
    const size_t off = tree == 0 ? rb : (rb + half < re ? rb + half : re);
    const size_t cnt = tree == 0 ? (half < re - rb ? half : re - rb) : re - off;
    const int v = tree == 0 ? rank : n - 1 - rank;
    const int parentV = v == 0 ? -1 : (v - 1) / 2;
    StepFlags f;
    f.w = bar.w;
    f.mine = (uint32_t*)((char*)a.sync.inbox[rank] + kOffTreeFlags) + ((size_t)slot * 2 + tree) * kMaxRanks;
    f.base = base;
    auto words = [&](int r) { return (uint32_t*)((char*)a.sync.inbox[r] + kOffTreeFlags) + ((size_t)slot * 2 + tree) * kMaxRanks; };
    // up: fold the children's partial sums into mine, then tell the parent
    for (int k = 1; k <= 2 && ok; ++k) {
      int cv = 2 * v + k;
      if (cv >= n) break;
      int c = treeReal(cv, tree, n);
      ok = f.wait(c, base + 1);
      if (ok) rangeOp<T, OP, true>(W, (const char*)a.recv[c], off, cnt, a.vec16);
    }
    if (!ok) break;
    if (parentV >= 0) {
      int p = treeReal(parentV, tree, n);
      f.post(words(p), rank, base + 1);
      // down: wait for the total in the parent's buffer and take it
      ok = f.wait(p, base + 2);
      if (ok) rangeOp<T, OP, false>(W, (const char*)a.recv[p], off, cnt, a.vec16);
    } else if (a.scaleMode != SCALE_NONE) {
      __syncthreads();
      rangeScale<T, OP>(W, off, cnt, a);
    }
    if (!ok) break;
    for (int k = 1; k <= 2; ++k) {
      int cv = 2 * v + k;
      if (cv >= n) break;
      f.post(words(treeReal(cv, tree, n)), rank, base + 2);
    }
  }
  bar.sync(true, false);
  if (threadIdx.x == 0) *basePtr = base + 2;
  bar.finish();
}

template <typename T, int OP> static const void* ringFn() { return (const void*)ringKernel<T, OP>; }
template <typename T, int OP> static const void* treeFn() { return (const void*)treeKernel<T, OP>; }
#define RT_BY_OP(FN, T, op) \
  ((op) == RED_SUM ? FN<T, RED_SUM>() : (op) == RED_PROD ? FN<T, RED_PROD>() : (op) == RED_MAX ? FN<T, RED_MAX>() : FN<T, RED_MIN>())
#define RT_BY_TYPE(FN, type, op)                                 \
  switch (type) {                                                \
    case ncclInt8: return RT_BY_OP(FN, int8_t, op);              \
    case ncclUint8: return RT_BY_OP(FN, uint8_t, op);            \
    case ncclInt32: return RT_BY_OP(FN, int32_t, op);            \
    case ncclUint32: return RT_BY_OP(FN, uint32_t, op);          \
    case ncclInt64: return RT_BY_OP(FN, int64_t, op);            \
    case ncclUint64: return RT_BY_OP(FN, uint64_t, op);          \
    case ncclFloat16: return RT_BY_OP(FN, __half, op);           \
    case ncclFloat32: return RT_BY_OP(FN, float, op);            \
    case ncclFloat64: return RT_BY_OP(FN, double, op);           \
    case ncclBfloat16: return RT_BY_OP(FN, __nv_bfloat16, op);   \
    case ncclFloat8e4m3: return RT_BY_OP(FN, F8E4, op);          \
    case ncclFloat8e5m2: return RT_BY_OP(FN, F8E5, op);          \
    default: return nullptr;                                     \
  }
const void* ringKernelFn(ncclDataType_t type, int op) { RT_BY_TYPE(ringFn, type, op) }
const void* treeKernelFn(ncclDataType_t type, int op) { RT_BY_TYPE(treeFn, type, op) }

}  // namespace b200
