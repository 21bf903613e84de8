// Flagged-line ("LL") kernels for small messages: one NVLink crossing, no barrier.
// A 16-byte line carries 8 payload bytes and the call's epoch twice: {data, epoch, data, epoch}.
// Senders store lines straight into the receiver's LL region (one region per source rank and
// epoch parity); receivers poll a line until both flags show the epoch, which also proves the
// payload is whole because a 16-byte store is never torn. Two parities make a region safe to
// reuse: a rank can only be two calls ahead of a peer once that peer has consumed the call
// before.
//   llReduceKernel  all-reduce (everyone sends everything to everyone), reduce-scatter (rank p
//                   gets slice p from everyone) and reduce (everyone sends to the root); the
//                   receiver reduces in rank order with fp32 accumulation for narrow floats.
//   llCopyKernel    all-gather, all-to-all, broadcast, gather and scatter.
// Reference parity: src/device/symmetric/all_reduce.cuh:506-584 (AGxLL_R), all_gather.cuh:310-424
// (LL), reduce_scatter.cuh:471-548 (LL), nccl_device/impl/ll_a2a__funcs.h (line format).
#include "common.cuh"
#include "launch.h"
#include "../comm/comm.h"

namespace b200 {

__device__ __forceinline__ uint64_t llLoad8(const char* p, size_t valid) {
  if (valid >= 8 && ((uintptr_t)p & 7) == 0) return *(const uint64_t*)p;
  uint64_t v = 0;
  for (size_t b = 0; b < 8 && b < valid; ++b) v |= (uint64_t)(uint8_t)p[b] << (8 * b);
  return v;
}
__device__ __forceinline__ void llStore8(char* p, uint64_t v, size_t valid) {
  if (valid >= 8 && ((uintptr_t)p & 7) == 0) { *(uint64_t*)p = v; return; }
  for (size_t b = 0; b < 8 && b < valid; ++b) p[b] = (char)(v >> (8 * b));
}

struct LLCtx {
  uint32_t* ep;
  uint32_t epoch;
  int parity;
  __device__ __forceinline__ void begin(const CollArgs& a, int rank) {
    ep = a.llEpoch[rank];
    epoch = ep[0] + 1;
    if (epoch == 0) epoch = 1;
    parity = epoch & 1;
  }
  __device__ __forceinline__ char* region(const CollArgs& a, int owner, int src) const {
    return (char*)a.ll[owner] + ((size_t)(parity * kMaxRanks + src) * kLLLines) * 16;
  }
  // The last CTA of the grid to finish publishes the epoch for the next call. Rooted collectives
  // move data one way only, so nothing would stop the sending side from running two calls ahead
  // and overwriting lines that were not consumed yet: there the consumers acknowledge (last line
  // of their region at the producer) and the producers wait for the acknowledgements here.
  __device__ __forceinline__ void end(const CollArgs& a, const WaitCtx& w, int rank, unsigned ackTo, unsigned ackFrom) {
    __syncthreads();
    if (threadIdx.x == 0) {
      // a grid of one CTA (the smallest messages) has nobody to count
      uint32_t done = 0;
      if (gridDim.x > 1) {
        __threadfence();
        done = atomicAdd(&ep[1], 1u);
      }
      if (done == gridDim.x - 1) {
        const uint32_t e = epoch;
        for (int p = 0; p < a.nRanks; ++p)
          if (ackTo & (1u << p)) stVolatile16(region(a, p, rank) + (kLLLines - 1) * 16, make_uint4(e, e, e, e));
        for (int p = 0; p < a.nRanks; ++p)
          if (ackFrom & (1u << p)) {
            const char* slot = region(a, rank, p) + (kLLLines - 1) * 16;
            boundedWait(w, WAIT_LL, (uint32_t)p, e, [&] { uint4 v = ldVolatile16(slot); return v.y == e && v.w == e; });
          }
        ep[1] = 0;
        ep[0] = epoch;
      }
    }
  }
  // Lines of all sources for one position, loaded together: the loads are independent, so a
  // receiver pays one trip to memory instead of one per source; only lines that have not landed
  // yet are polled again.
  template <typename F>
  __device__ __forceinline__ bool recvLines(const CollArgs& a, const WaitCtx& w, int rank, size_t l, uint64_t own, F&& consume) const {
    const uint32_t e = epoch;
    uint4 v[kMaxRanks];
#pragma unroll
    for (int s = 0; s < kMaxRanks; ++s)
      if (s < a.nRanks && s != rank) v[s] = ldVolatile16(region(a, rank, s) + l * 16);
    bool ok = true;
#pragma unroll
    for (int s = 0; s < kMaxRanks; ++s) {
      if (s >= a.nRanks) break;
      uint64_t d = own;
      if (s != rank) {
        if (v[s].y != e || v[s].w != e) {
          const char* slot = region(a, rank, s) + l * 16;
          uint4 r = v[s];
          ok = ok && boundedWait(w, WAIT_LL, (uint32_t)s, e, [&] { r = ldVolatile16(slot); return r.y == e && r.w == e; });
          v[s] = r;
        }
        d = (uint64_t)v[s].x | ((uint64_t)v[s].z << 32);
      }
      if (ok) consume(s, d);
    }
    return ok;
  }
  __device__ __forceinline__ bool recvLine(const WaitCtx& w, const char* slot, int src, uint64_t* d) const {
    uint4 v = ldVolatile16(slot);
    const uint32_t e = epoch;
    if (v.y != e || v.w != e) {
      if (!boundedWait(w, WAIT_LL, (uint32_t)src, e, [&] { v = ldVolatile16(slot); return v.y == e && v.w == e; })) return false;
    }
    *d = (uint64_t)v.x | ((uint64_t)v.z << 32);
    return true;
  }
};

template <typename T, int OP>
__global__ void __launch_bounds__(kCtaThreads, 1) llReduceKernel(const __grid_constant__ CollArgs a) {
  const int rank = ctaRank(a.emu, a.rank);
  const int n = a.nRanks;
  constexpr int N = 8 / sizeof(T);
  pdlEnter();
  KernelStamp stamp(a.sync.stamps);
  LLCtx ll;
  ll.begin(a, rank);
  WaitCtx w{&a.sync, a.sync.status[rank]};
  const size_t bytes = a.count * sizeof(T);            // bytes every receiver ends up with
  const size_t nLines = (bytes + 7) / 8;
  const bool scatter = a.func == FUNC_REDUCESCATTER;   // destination p gets my slice p
  const bool rooted = a.func == FUNC_REDUCE;           // only the root receives
  const char* in = (const char*)a.lsend[rank];
  char* out = (char*)a.lrecv[rank];
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  // phase 1: publish
  // all-reduce sends the same line to every peer: with a multicast alias of the region one
  // multimem.st does it (the switch replicates; the copy that lands in this rank's own region is unused)
  const bool mcast = a.llMc != nullptr && !scatter && !rooted;
  for (size_t l = tid; l < nLines; l += stride) {
    const size_t valid = bytes - l * 8;
    uint64_t d = scatter ? 0 : llLoad8(in + l * 8, valid);
    if (mcast) {
      char* slot = a.llMc + ((size_t)(ll.parity * kMaxRanks + rank) * kLLLines) * 16 + l * 16;
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(slot), "r"((uint32_t)d), "r"(ll.epoch), "r"((uint32_t)(d >> 32)),
                   "r"(ll.epoch) : "memory");
      continue;
    }
    for (int j = 1; j < n; ++j) {
      const int p = (rank + j) % n;
      if (rooted && p != a.root) continue;
      if (scatter) d = llLoad8(in + (size_t)p * bytes + l * 8, valid);
      stVolatile16(ll.region(a, p, rank) + l * 16, make_uint4((uint32_t)d, ll.epoch, (uint32_t)(d >> 32), ll.epoch));
    }
  }
  // phase 2: collect, reduce in rank order, write
  if (!rooted || rank == a.root) {
    const char* own = in + (scatter ? (size_t)rank * bytes : 0);
    bool ok = true;
    for (size_t l = tid; l < nLines && ok; l += stride) {
      const size_t valid = bytes - l * 8;
      typename Elem<T>::Acc acc[N];
      // sources are folded in rank order whatever order their lines arrived in
      ok = ll.recvLines(a, w, rank, l, llLoad8(own + l * 8, valid), [&](int s, uint64_t d) {
        union { uint64_t u; T e[N]; } cv;
        cv.u = d;
#pragma unroll
        for (int k = 0; k < N; ++k) {
          typename Elem<T>::Acc x = Elem<T>::ld(cv.e[k]);
          acc[k] = s == 0 ? x : redApply<OP>(acc[k], x);
        }
      });
      if (!ok) break;
      union { uint64_t u; T e[N]; } res;
#pragma unroll
      for (int k = 0; k < N; ++k) res.e[k] = scalarPost<T, OP>(acc[k], a);
      llStore8(out + l * 8, res.u, valid);
    }
  }
  unsigned ackTo = 0, ackFrom = 0;
  if (rooted) {
    const unsigned others = ((1u << n) - 1) & ~(1u << a.root);
    if (rank == a.root) ackTo = others; else ackFrom = 1u << a.root;
  }
  ll.end(a, w, rank, ackTo, ackFrom);
}

// One launch for a whole group of small all-reduces of one type and operator: the CTAs share the
// flattened line space of all items, one epoch and one closing step serve them all.
// Reference parity: the role of src/scheduler/symmetric_sched.cc:227-364 (several tasks per launch).
template <typename T, int OP>
__global__ void __launch_bounds__(kCtaThreads, 1) llReduceBatchKernel(const __grid_constant__ LLBatchArgs b) {
  const CollArgs& a = b.c;
  const int rank = ctaRank(a.emu, a.rank);
  const int n = a.nRanks;
  constexpr int N = 8 / sizeof(T);
  __shared__ LLItem items[kMaxLLItems];
  for (int i = threadIdx.x; i < b.nItems; i += blockDim.x) items[i] = b.items[i];
  pdlEnter();
  KernelStamp stamp(a.sync.stamps);
  LLCtx ll;
  ll.begin(a, rank);
  WaitCtx w{&a.sync, a.sync.status[rank]};
  __syncthreads();
  const char* inBase = (const char*)a.lsend[rank];
  char* outBase = (char*)a.lrecv[rank];
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool mcast = a.llMc != nullptr;
  auto itemOf = [&](uint32_t L) {
    int lo = 0, hi = b.nItems - 1;   // last item whose lineOff <= L
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (items[mid].lineOff <= L) lo = mid; else hi = mid - 1;
    }
    return lo;
  };
  for (size_t L = tid; L < b.totalLines; L += stride) {
    const LLItem it = items[itemOf((uint32_t)L)];
    const size_t l = L - it.lineOff;
    const size_t bytes = (size_t)it.count * sizeof(T);
    const uint64_t d = llLoad8(inBase + it.sendOff + l * 8, bytes - l * 8);
    if (mcast) {
      char* slot = a.llMc + ((size_t)(ll.parity * kMaxRanks + rank) * kLLLines) * 16 + L * 16;
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(slot), "r"((uint32_t)d), "r"(ll.epoch), "r"((uint32_t)(d >> 32)),
                   "r"(ll.epoch) : "memory");
      continue;
    }
    for (int j = 1; j < n; ++j) {
      const int p = (rank + j) % n;
      stVolatile16(ll.region(a, p, rank) + L * 16, make_uint4((uint32_t)d, ll.epoch, (uint32_t)(d >> 32), ll.epoch));
    }
  }
  bool ok = true;
  for (size_t L = tid; L < b.totalLines && ok; L += stride) {
    const LLItem it = items[itemOf((uint32_t)L)];
    const size_t l = L - it.lineOff;
    const size_t bytes = (size_t)it.count * sizeof(T);
    const size_t valid = bytes - l * 8;
    typename Elem<T>::Acc acc[N];
    ok = ll.recvLines(a, w, rank, L, llLoad8(inBase + it.sendOff + l * 8, valid), [&](int s, uint64_t d) {
      union { uint64_t u; T e[N]; } cv;
      cv.u = d;
#pragma unroll
      for (int k = 0; k < N; ++k) {
        typename Elem<T>::Acc x = Elem<T>::ld(cv.e[k]);
        acc[k] = s == 0 ? x : redApply<OP>(acc[k], x);
      }
    });
    if (!ok) break;
    union { uint64_t u; T e[N]; } res;
#pragma unroll
    for (int k = 0; k < N; ++k) res.e[k] = scalarPost<T, OP>(acc[k], a);
    llStore8(outBase + it.recvOff + l * 8, res.u, valid);
  }
  ll.end(a, w, rank, 0, 0);
}

// a.count = bytes of one block; a.sendStride / a.recvStride = pitch of blocks in the user buffers.
__global__ void __launch_bounds__(kCtaThreads, 1) llCopyKernel(const __grid_constant__ CollArgs a) {
  const int rank = ctaRank(a.emu, a.rank);
  const int n = a.nRanks;
  pdlEnter();
  KernelStamp stamp(a.sync.stamps);
  LLCtx ll;
  ll.begin(a, rank);
  WaitCtx w{&a.sync, a.sync.status[rank]};
  const size_t B = a.count;
  const size_t nLines = (B + 7) / 8;
  const char* in = (const char*)a.lsend[rank];
  char* out = (char*)a.lrecv[rank];
  const size_t SS = a.sendStride, RS = a.recvStride;
  const int func = a.func, root = a.root;
  // who I send to / receive from, and where the block sits in my buffers
  auto sendsTo = [&](int p) {
    if (func == FUNC_BROADCAST || func == FUNC_SCATTER) return rank == root;
    if (func == FUNC_GATHER) return p == root;
    return true;
  };
  auto recvsFrom = [&](int s) {
    if (func == FUNC_BROADCAST || func == FUNC_SCATTER) return s == root;
    if (func == FUNC_GATHER) return rank == root;
    return true;
  };
  auto srcOff = [&](int p) -> size_t { return (func == FUNC_ALLTOALL || func == FUNC_SCATTER) ? (size_t)p * SS : 0; };
  auto dstOff = [&](int s) -> size_t { return (func == FUNC_BROADCAST || func == FUNC_SCATTER) ? 0 : (size_t)s * RS; };
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t items = nLines * (size_t)(n - 1);
  // phase 1: publish (item = (peer offset j, line))
  for (size_t it = tid; it < items; it += stride) {
    const int j = (int)(it / nLines) + 1;
    const size_t l = it % nLines;
    const int p = (rank + j) % n;
    if (!sendsTo(p)) continue;
    uint64_t d = llLoad8(in + srcOff(p) + l * 8, B - l * 8);
    stVolatile16(ll.region(a, p, rank) + l * 16, make_uint4((uint32_t)d, ll.epoch, (uint32_t)(d >> 32), ll.epoch));
  }
  // my own block moves locally
  if (recvsFrom(rank) && sendsTo(rank)) {
    const char* s = in + srcOff(rank);
    char* d = out + dstOff(rank);
    if (s != d)
      for (size_t l = tid; l < nLines; l += stride) llStore8(d + l * 8, llLoad8(s + l * 8, B - l * 8), B - l * 8);
  }
  // phase 2: collect
  bool ok = true;
  for (size_t it = tid; it < items && ok; it += stride) {
    const int j = (int)(it / nLines) + 1;
    const size_t l = it % nLines;
    const int s = (rank + n - j) % n;
    if (!recvsFrom(s)) continue;
    uint64_t d;
    ok = ll.recvLine(w, ll.region(a, rank, s) + l * 16, s, &d);
    if (ok) llStore8(out + dstOff(s) + l * 8, d, B - l * 8);
  }
  unsigned ackTo = 0, ackFrom = 0;
  const unsigned others = ((1u << n) - 1) & ~(1u << root);
  if (func == FUNC_BROADCAST || func == FUNC_SCATTER) {
    if (rank == root) ackFrom = others; else ackTo = 1u << root;      // consumers tell the root
  } else if (func == FUNC_GATHER) {
    if (rank == root) ackTo = others; else ackFrom = 1u << root;      // the root tells the producers
  }
  ll.end(a, w, rank, ackTo, ackFrom);
}

template <typename T, int OP> static const void* llFn(bool batch) {
  return batch ? (const void*)llReduceBatchKernel<T, OP> : (const void*)llReduceKernel<T, OP>;
}
#define LL_BY_OP(T, op) \
  ((op) == RED_SUM ? llFn<T, RED_SUM>(batch) : (op) == RED_PROD ? llFn<T, RED_PROD>(batch) : (op) == RED_MAX ? llFn<T, RED_MAX>(batch) : llFn<T, RED_MIN>(batch))

static const void* llAnyFn(ncclDataType_t type, int op, bool batch) {
  switch (type) {
    case ncclInt8: return LL_BY_OP(int8_t, op);
    case ncclUint8: return LL_BY_OP(uint8_t, op);
    case ncclInt32: return LL_BY_OP(int32_t, op);
    case ncclUint32: return LL_BY_OP(uint32_t, op);
    case ncclInt64: return LL_BY_OP(int64_t, op);
    case ncclUint64: return LL_BY_OP(uint64_t, op);
    case ncclFloat16: return LL_BY_OP(__half, op);
    case ncclFloat32: return LL_BY_OP(float, op);
    case ncclFloat64: return LL_BY_OP(double, op);
    case ncclBfloat16: return LL_BY_OP(__nv_bfloat16, op);
    case ncclFloat8e4m3: return LL_BY_OP(F8E4, op);
    case ncclFloat8e5m2: return LL_BY_OP(F8E5, op);
    default: return nullptr;
  }
}
const void* llReduceKernelFn(ncclDataType_t type, int op) { return llAnyFn(type, op, false); }
const void* llReduceBatchKernelFn(ncclDataType_t type, int op) { return llAnyFn(type, op, true); }
const void* llCopyKernelFn() { return (const void*)llCopyKernel; }

}  // namespace b200
