// Device building blocks of every data-movement kernel: memory-ordering wrappers, bounded
// waits, the cross-GPU CTA barrier, multimem wrappers and typed 16-byte pack arithmetic.
// Reference parity: src/device/op128.h (ld/st/fence wrappers), nccl_device/impl/lsa_barrier__funcs.h
// (epoch barrier with time-outs), src/device/reduce_kernel.h (typed reductions, multimem forms).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "args.h"

namespace b200 {

// ------------------------------------------------------------------ memory ordering
__device__ __forceinline__ uint32_t ldAcquireSys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t ldAcquireSys64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ldRelaxedSys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t ldRelaxedSys64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// A system-scope fence costs microseconds on this part, and st.release / ld.acquire each carry
// one. Flags are therefore published as "one fence, then a relaxed store" and awaited as
// "relaxed polls, then one fence": the same ordering with one fence per hand-off side.
__device__ __forceinline__ void stReleaseSys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void stRelaxedSys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void redReleaseSysAdd64(uint64_t* p, uint64_t v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void fenceSys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ unsigned long long globalTimerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint4 ldVolatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void stVolatile16(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// Streaming 16-byte accesses: data crosses NVLink once and is not worth keeping in L1.
__device__ __forceinline__ uint4 ldStream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ldLocal16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

// ------------------------------------------------------------------ multimem (NVLS)
__device__ __forceinline__ void mcSt16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void mcRedAdd32(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
__device__ __forceinline__ void mcRedAdd32Relaxed(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

// ------------------------------------------------------------------ programmatic dependent launch
// Collective kernels are launched with programmatic stream serialisation: the grid may be scheduled
// while the previous kernel of the stream is still draining, which hides the launch latency between
// back-to-back collectives. pdlWait() returns once every earlier grid of the stream has completed
// and its writes are visible; nothing that an earlier kernel may have written (epoch words, user
// buffers) is read before it. pdlLaunchDependents() lets the next grid be scheduled from then on
// (it still waits for this grid's completion in its own pdlWait()). Both are no-ops for a grid
// launched without the attribute.
// Reference parity: cudaGridDependencySynchronize at the top of every symmetric kernel
// (src/device/symmetric/generate.py:171-222), launch attribute in src/enqueue.cc:1753-1851.
__device__ __forceinline__ void pdlWait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdlLaunchDependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdlEnter() { pdlWait(); pdlLaunchDependents(); }

// Start and stop times of a CTA for profiler plugins, taken on the device: constructed right after pdlEnter() (so the
// wait for the previous grid is not counted), the stop is written when the kernel body is left, on every path. A
// task that takes several launches keeps the first start and the last stop.
// Reference parity: work-counter time stamps of src/device/common.h:323-353 (KernelCh events of the profiler).
struct KernelStamp {
  unsigned long long* const& base;   // refers to the launch arguments (constant bank): nothing is kept in registers across the kernel
  __device__ __forceinline__ bool mine() const { return base != nullptr && threadIdx.x == 0 && blockIdx.y == 0 && blockIdx.x < kStampCtas; }
  __device__ __forceinline__ explicit KernelStamp(unsigned long long* const& b) : base(b) {
    if (mine()) {
      volatile unsigned long long* p = base + 2 * blockIdx.x;
      if (p[0] == 0) p[0] = globalTimerNs();
    }
  }
  __device__ __forceinline__ ~KernelStamp() {
    if (mine()) ((volatile unsigned long long*)base)[2 * blockIdx.x + 1] = globalTimerNs();
  }
};

// ------------------------------------------------------------------ bounded waits
// A wait polls until `done()` holds, the host raises the abort flag, or the time budget runs
// out. On failure it records what it was waiting for in the rank's status words and returns
// false; callers then skip the rest of their protocol so that the kernel always terminates.
struct WaitCtx {
  const SyncArgs* sync;
  uint32_t* status;
  __device__ __forceinline__ bool failed() const { return ldRelaxedSys(status) != DEV_OK; }
};

// `record = false`: the caller handles a wait that ran out itself (e.g. leaves the peer out from
// then on) and nothing is written to the status words.
template <typename Pred>
__device__ __forceinline__ bool boundedWait(const WaitCtx& w, uint32_t kind, uint32_t peer, uint32_t expected, Pred done, bool record = true) {
  if (done()) return true;
  unsigned long long start = globalTimerNs();
  uint32_t spins = 0;
  for (;;) {
    if (done()) return true;
    if ((++spins & 0xff) == 0) {
      uint32_t code = DEV_OK;
      if (w.sync->abortFlag && ldRelaxedSys(w.sync->abortFlag)) code = DEV_ABORTED;
      else if (globalTimerNs() - start > w.sync->timeoutNs) code = DEV_TIMEOUT;
      else if (ldRelaxedSys(w.status) != DEV_OK) return false;  // another wait of this rank already failed
      if (code != DEV_OK && !(record || code == DEV_ABORTED)) return false;
      if (code != DEV_OK) {
        // Status words may live in host-mapped memory: plain stores only; concurrent failing
        // waits write equivalent records, so the race between them is harmless.
        if (ldRelaxedSys(w.status) == DEV_OK) {
          w.status[1] = kind;
          w.status[2] = peer;
          w.status[3] = expected;
          __threadfence_system();
          stRelaxedSys(w.status, code);
        }
        return false;
      }
    }
  }
}

// ------------------------------------------------------------------ cross-GPU CTA barrier
// CTA `slot` of every rank meets CTA `slot` of every other rank. Two forms:
//   unicast    thread t (< nRanks) of the CTA signals peer t with a store of the new epoch into
//              the peer's inbox and then polls its own inbox for that peer's epoch;
//   multicast  (when the sync page has a multicast alias) one thread adds 1 to the slot's arrival
//              counter on every rank with a single multimem.red and polls its own copy until it
//              shows nRanks arrivals per barrier so far (reference:
//              nccl_device/impl/lsa_barrier__funcs.h:58-66, 100-115).
// Epoch counters are private per rank, per slot and per form and persist across launches, so a
// CUDA-graph replay needs no host-side state.
struct CtaBarrier {
  WaitCtx w;
  uint32_t* const* inbox;
  uint32_t* epochPtr;
  uint32_t* mcArrive;     // multicast address of this slot's arrival counter, or null
  const uint32_t* mcMine; // this rank's copy of that counter
  int rank, nRanks, slot;
  uint32_t epoch;

  __device__ __forceinline__ void init(const SyncArgs& s, int rank_, int nRanks_, int slot_) {
    w.sync = &s;
    w.status = s.status[rank_];
    inbox = s.inbox;
    rank = rank_;
    nRanks = nRanks_;
    slot = slot_;
    mcArrive = s.mcArrive ? s.mcArrive + slot_ : nullptr;
    mcMine = s.mcArrive ? (const uint32_t*)((const char*)s.inbox[rank_] + kOffMcBarrier) + slot_ : nullptr;
    epochPtr = s.epoch[rank_] + (s.mcArrive ? kPrivMcEpoch : 0) + slot_;
    epoch = *epochPtr;  // every thread reads the same value; written back by finish()
  }
  // All threads of the CTA must call.
  //   release: data written before the call by any thread of the CTA is visible to every peer CTA
  //            after its matching call returns (one system-scope fence by the signalling thread,
  //            cumulative over the CTA through the __syncthreads before it);
  //   acquire: data the peers released before their call may be read after this call returns.
  // A barrier that only says "my kernel has started" (inputs were written by earlier kernels, which
  // a kernel boundary already made visible) needs neither, and a closing barrier after which this
  // kernel reads nothing needs no acquire: system-scope fences cost microseconds each, so callers
  // ask only for what they need. Polling uses relaxed loads; the acquire fence comes once, after.
  __device__ __forceinline__ bool sync(bool release = true, bool acquire = true) {
    ++epoch;
    __syncthreads();
    bool ok = true;
    int t = threadIdx.x;
    if (mcArrive) {
      if (t == 0) {
        if (release) mcRedAdd32(mcArrive, 1u); else mcRedAdd32Relaxed(mcArrive, 1u);
        const uint32_t want = epoch * (uint32_t)nRanks;   // arrivals of all barriers so far on this slot, modulo 2^32
        const uint32_t* mine = mcMine;
        ok = boundedWait(w, WAIT_BARRIER, (uint32_t)rank, want, [&] { return (int32_t)(ldRelaxedSys(mine) - want) >= 0; });
        if (acquire) fenceSys();
      }
    } else if (t < nRanks && t != rank) {
      if (release) fenceSys();
      stRelaxedSys(inbox[t] + (size_t)slot * kMaxRanks + rank, epoch);
      const uint32_t* mine = inbox[rank] + (size_t)slot * kMaxRanks + t;
      uint32_t want = epoch;
      ok = boundedWait(w, WAIT_BARRIER, (uint32_t)t, want, [&] { return (int32_t)(ldRelaxedSys(mine) - want) >= 0; });
      if (acquire) fenceSys();
    }
    ok = __syncthreads_and(ok);
    return ok;
  }
  __device__ __forceinline__ void finish() {
    if (threadIdx.x == 0) *epochPtr = epoch;
  }
};

// ------------------------------------------------------------------ typed element access
struct F8E4 { uint8_t v; };
struct F8E5 { uint8_t v; };

template <typename T> struct Elem;
#define B200_NATIVE_ELEM(T, A)                                              \
  template <> struct Elem<T> {                                              \
    using Acc = A;                                                          \
    static __device__ __forceinline__ Acc ld(T x) { return (Acc)x; }        \
    static __device__ __forceinline__ T st(Acc a) { return (T)a; }          \
  };
B200_NATIVE_ELEM(int8_t, int)
B200_NATIVE_ELEM(uint8_t, unsigned)
B200_NATIVE_ELEM(int32_t, int32_t)
B200_NATIVE_ELEM(uint32_t, uint32_t)
B200_NATIVE_ELEM(int64_t, long long)
B200_NATIVE_ELEM(uint64_t, unsigned long long)
B200_NATIVE_ELEM(float, float)
B200_NATIVE_ELEM(double, double)
template <> struct Elem<__half> {
  using Acc = float;
  static __device__ __forceinline__ float ld(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half st(float a) { return __float2half_rn(a); }
};
template <> struct Elem<__nv_bfloat16> {
  using Acc = float;
  static __device__ __forceinline__ float ld(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 st(float a) { return __float2bfloat16_rn(a); }
};
template <> struct Elem<F8E4> {
  using Acc = float;
  static __device__ __forceinline__ float ld(F8E4 x) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(x.v, __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
  }
  static __device__ __forceinline__ F8E4 st(float a) { return F8E4{(uint8_t)__nv_cvt_float_to_fp8(a, __NV_SATFINITE, __NV_E4M3)}; }
};
template <> struct Elem<F8E5> {
  using Acc = float;
  static __device__ __forceinline__ float ld(F8E5 x) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(x.v, __NV_E5M2);
    return __half2float(*reinterpret_cast<__half*>(&h));
  }
  static __device__ __forceinline__ F8E5 st(float a) { return F8E5{(uint8_t)__nv_cvt_float_to_fp8(a, __NV_SATFINITE, __NV_E5M2)}; }
};

template <int OP, typename A> __device__ __forceinline__ A redApply(A a, A b) {
  if (OP == RED_SUM) return a + b;
  if (OP == RED_PROD) return a * b;
  if (OP == RED_MAX) return a > b ? a : b;
  return a < b ? a : b;
}

template <typename T> struct Pack16 {
  static constexpr int N = 16 / sizeof(T);
  union { uint4 v; T e[N]; };
};

// acc (op)= elements of v
template <typename T, int OP> struct PackAcc {
  using A = typename Elem<T>::Acc;
  static constexpr int N = 16 / sizeof(T);
  A a[N];
  __device__ __forceinline__ void set(uint4 v) {
    Pack16<T> p; p.v = v;
#pragma unroll
    for (int i = 0; i < N; ++i) a[i] = Elem<T>::ld(p.e[i]);
  }
  __device__ __forceinline__ void add(uint4 v) {
    Pack16<T> p; p.v = v;
#pragma unroll
    for (int i = 0; i < N; ++i) a[i] = redApply<OP, A>(a[i], Elem<T>::ld(p.e[i]));
  }
  __device__ __forceinline__ uint4 get(int scaleMode, float scaleF, double scaleD, long long intDiv) {
    Pack16<T> p;
#pragma unroll
    for (int i = 0; i < N; ++i) p.e[i] = Elem<T>::st(postScale(a[i], scaleMode, scaleF, scaleD, intDiv));
    return p.v;
  }
  static __device__ __forceinline__ float postScale(float x, int m, float f, double, long long) { return m == SCALE_MUL ? x * f : x; }
  static __device__ __forceinline__ double postScale(double x, int m, float, double d, long long) { return m == SCALE_MUL ? x * d : x; }
  template <typename I> static __device__ __forceinline__ I postScale(I x, int m, float, double, long long div) {
    return m == SCALE_INTDIV ? (I)(x / (I)div) : x;
  }
};

template <typename T, int OP>
__device__ __forceinline__ T scalarPost(typename Elem<T>::Acc a, const CollArgs& c) {
  return Elem<T>::st(PackAcc<T, OP>::postScale(a, c.scaleMode, c.scaleF, c.scaleD, c.intDiv));
}

// Rank played by this CTA and the index of the CTA within that rank's grid.
__device__ __forceinline__ int ctaRank(int emu, int rank) { return emu ? (int)blockIdx.y : rank; }

}  // namespace b200
