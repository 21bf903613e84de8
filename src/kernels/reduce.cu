// Reduction kernels over peer-mapped buffers.
//   reduceP2pKernel    every rank loads its slice from all ranks, reduces in registers (fp32
//                      accumulation for 8/16-bit floats, fixed rank order) and stores the result
//                      locally (reduce-scatter, reduce) or to every rank (two-shot all-reduce).
//   (the flagged-line kernels for small payloads are in ll.cu)
//   reduceNvlsKernel   the same three collectives with multimem.ld_reduce (the NVSwitch reduces)
//                      and multimem.st (the switch replicates).
// Reference parity: src/device/symmetric/all_reduce.cuh:14-262 (RSxLD_AGxST), :431-504
// (RSxLDMC_AGxSTMC), :506-584 (AGxLL_R), reduce_scatter.cuh:13-242,396-469.
#include "common.cuh"
#include "launch.h"

namespace b200 {

// ------------------------------------------------------------------------- P2P
template <typename T, int OP>
__global__ void __launch_bounds__(kCtaThreads, 1) reduceP2pKernel(const __grid_constant__ CollArgs a) {
  const int rank = ctaRank(a.emu, a.rank);
  const int n = a.nRanks;
  pdlEnter();
  KernelStamp stamp(a.sync.stamps);
  CtaBarrier bar;
  bar.init(a.sync, rank, n, blockIdx.x);
  bool ok = bar.sync(false, false);  // inputs of every rank are final (written by earlier kernels); outputs may be overwritten
  const size_t begin = a.sliceBegin[rank], cnt = a.sliceCount[rank];
  if (ok && cnt) {
    constexpr int N = 16 / sizeof(T);
    // Peer pointers stay in the kernel-parameter bank (a.send / a.recv) and are re-read per access:
    // keeping sixteen 64-bit pointers in registers next to 2 * nRanks 16-byte packs spilled.
    const size_t inOff = begin * sizeof(T), outOff = a.dstOff[rank] * sizeof(T);
    const int nDst = a.dstAll ? n : 1;
    auto srcOf = [&](int p) { return (const char*)a.send[p] + inOff; };
    auto dstOf = [&](int q) { return (a.dstAll ? (char*)a.recv[q] : (char*)a.lrecv[rank]) + outOff; };
    const size_t nPacks = a.vec16 ? cnt / N : 0;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    // two packs per iteration: 2 * nRanks independent 16-byte loads in flight per thread
    for (; i + stride < nPacks; i += 2 * stride) {
      uint4 v0[kMaxRanks], v1[kMaxRanks];
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p) {
        if (p < n) {
          const char* s = srcOf(p);
          v0[p] = ldStream16(s + i * 16);
          v1[p] = ldStream16(s + (i + stride) * 16);
        }
      }
      PackAcc<T, OP> a0, a1;
      a0.set(v0[0]);
      a1.set(v1[0]);
#pragma unroll
      for (int p = 1; p < kMaxRanks; ++p) {
        if (p < n) { a0.add(v0[p]); a1.add(v1[p]); }
      }
      uint4 r0 = a0.get(a.scaleMode, a.scaleF, a.scaleD, a.intDiv);
      uint4 r1 = a1.get(a.scaleMode, a.scaleF, a.scaleD, a.intDiv);
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q) {
        if (q < nDst) { char* d = dstOf(q); st16(d + i * 16, r0); st16(d + (i + stride) * 16, r1); }
      }
    }
    for (; i < nPacks; i += stride) {
      PackAcc<T, OP> acc;
      acc.set(ldStream16(srcOf(0) + i * 16));
#pragma unroll
      for (int p = 1; p < kMaxRanks; ++p) if (p < n) acc.add(ldStream16(srcOf(p) + i * 16));
      uint4 r = acc.get(a.scaleMode, a.scaleF, a.scaleD, a.intDiv);
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q) if (q < nDst) st16(dstOf(q) + i * 16, r);
    }
    // ragged tail (and the whole slice when a pointer is not 16-byte aligned): one element at a time
    for (size_t e = nPacks * N + (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < cnt; e += stride) {
      typename Elem<T>::Acc acc = Elem<T>::ld(((const T*)srcOf(0))[e]);
      for (int p = 1; p < n; ++p) acc = redApply<OP>(acc, Elem<T>::ld(((const T*)srcOf(p))[e]));
      T r = scalarPost<T, OP>(acc, a);
      for (int q = 0; q < nDst; ++q) ((T*)dstOf(q))[e] = r;
    }
  }
  bar.sync(a.dstAll != 0, false);  // results have landed everywhere (release only when peers were written); nobody reads this rank's input any more
  bar.finish();
}

// ------------------------------------------------------------------------- NVLS
template <typename T, int OP> struct McRed { static constexpr bool kSupported = false; };

#define MC_V4(T, OP, INSTR)                                                                                  \
  template <> struct McRed<T, OP> {                                                                          \
    static constexpr bool kSupported = true;                                                                 \
    static __device__ __forceinline__ uint4 ld(const void* mc) {                                             \
      uint4 v;                                                                                               \
      asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " {%0,%1,%2,%3}, [%4];"                    \
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");                       \
      return v;                                                                                              \
    }                                                                                                        \
  };
#define MC_S32(T, OP, INSTR)                                                                                 \
  template <> struct McRed<T, OP> {                                                                          \
    static constexpr bool kSupported = true;                                                                 \
    static __device__ __forceinline__ uint4 ld(const void* mc) {                                             \
      uint4 v;                                                                                               \
      const char* p = (const char*)mc;                                                                       \
      asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : "=r"(v.x) : "l"(p) : "memory");      \
      asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : "=r"(v.y) : "l"(p + 4) : "memory");  \
      asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : "=r"(v.z) : "l"(p + 8) : "memory");  \
      asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : "=r"(v.w) : "l"(p + 12) : "memory"); \
      return v;                                                                                              \
    }                                                                                                        \
  };
#define MC_S64(T, OP, INSTR, CONSTRAINT)                                                                     \
  template <> struct McRed<T, OP> {                                                                          \
    static constexpr bool kSupported = true;                                                                 \
    static __device__ __forceinline__ uint4 ld(const void* mc) {                                             \
      union { uint4 v; unsigned long long q[2]; double d[2]; } u;                                            \
      const char* p = (const char*)mc;                                                                       \
      asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : CONSTRAINT(u.q[0]) : "l"(p) : "memory");     \
      asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : CONSTRAINT(u.q[1]) : "l"(p + 8) : "memory"); \
      return u.v;                                                                                            \
    }                                                                                                        \
  };
MC_V4(float, RED_SUM, "add.v4.f32")
MC_V4(__half, RED_SUM, "add.acc::f32.v4.f16x2")
MC_V4(__half, RED_MAX, "max.v4.f16x2")
MC_V4(__half, RED_MIN, "min.v4.f16x2")
MC_V4(__nv_bfloat16, RED_SUM, "add.acc::f32.v4.bf16x2")
MC_V4(__nv_bfloat16, RED_MAX, "max.v4.bf16x2")
MC_V4(__nv_bfloat16, RED_MIN, "min.v4.bf16x2")
MC_V4(F8E4, RED_SUM, "add.acc::f16.v4.e4m3x4")
MC_V4(F8E5, RED_SUM, "add.acc::f16.v4.e5m2x4")
MC_S32(int32_t, RED_SUM, "add.s32")
MC_S32(int32_t, RED_MAX, "max.s32")
MC_S32(int32_t, RED_MIN, "min.s32")
MC_S32(uint32_t, RED_SUM, "add.u32")
MC_S32(uint32_t, RED_MAX, "max.u32")
MC_S32(uint32_t, RED_MIN, "min.u32")
MC_S64(int64_t, RED_SUM, "add.u64", "=l")
MC_S64(int64_t, RED_MAX, "max.s64", "=l")
MC_S64(int64_t, RED_MIN, "min.s64", "=l")
MC_S64(uint64_t, RED_SUM, "add.u64", "=l")
MC_S64(uint64_t, RED_MAX, "max.u64", "=l")
MC_S64(uint64_t, RED_MIN, "min.u64", "=l")
MC_S64(double, RED_SUM, "add.f64", "=l")

// Slices, offsets and counts must be multiples of 16 bytes (the host falls back to P2P otherwise).
template <typename T, int OP>
__global__ void __launch_bounds__(kCtaThreads, 1) reduceNvlsKernel(const __grid_constant__ CollArgs a) {
  const int rank = a.rank;
  pdlEnter();
  KernelStamp stamp(a.sync.stamps);
  CtaBarrier bar;
  bar.init(a.sync, rank, a.nRanks, blockIdx.x);
  bool ok = bar.sync(false, false);
  if constexpr (McRed<T, OP>::kSupported) {
    const size_t cnt = a.sliceCount[rank];
    if (ok && cnt) {
      constexpr int N = 16 / sizeof(T);
      const char* src = (const char*)a.sendMc + a.sliceBegin[rank] * sizeof(T);
      char* dst = (a.dstAll ? (char*)a.recvMc : (char*)a.lrecv[rank]) + a.dstOff[rank] * sizeof(T);
      const size_t nPacks = cnt / N;
      const size_t stride = (size_t)gridDim.x * blockDim.x;
      const bool scale = a.scaleMode != SCALE_NONE;
      // Eight independent multimem loads per thread and round (tails predicated, not peeled): the
      // switch round trip is long, and a few CTAs with deep queues keep the links as busy as many
      // CTAs with shallow ones while their barriers cost less.
      constexpr int U = 8;
      for (size_t base = (size_t)blockIdx.x * blockDim.x + threadIdx.x; base < nPacks; base += (size_t)U * stride) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t i = base + (size_t)u * stride;
          if (i < nPacks) v[u] = McRed<T, OP>::ld(src + i * 16);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t i = base + (size_t)u * stride;
          if (i < nPacks) {
            if (scale) { PackAcc<T, OP> acc; acc.set(v[u]); v[u] = acc.get(a.scaleMode, a.scaleF, a.scaleD, a.intDiv); }
            if (a.dstAll) mcSt16(dst + i * 16, v[u]); else st16(dst + i * 16, v[u]);
          }
        }
      }
    }
  }
  bar.sync(a.dstAll != 0, false);   // only results stored to peers need a release; otherwise: "I have read your input"
  bar.finish();
}

// ------------------------------------------------------------------------- dispatch
template <template <typename, int> class K> struct KernelOf;

template <typename T, int OP> static const void* p2pFn() { return (const void*)reduceP2pKernel<T, OP>; }
template <typename T, int OP> static const void* nvlsFn() {
  if constexpr (McRed<T, OP>::kSupported) return (const void*)reduceNvlsKernel<T, OP>;
  else return nullptr;
}

#define BY_OP(FN, T, op)                                   \
  ((op) == RED_SUM ? FN<T, RED_SUM>() : (op) == RED_PROD ? FN<T, RED_PROD>() : (op) == RED_MAX ? FN<T, RED_MAX>() : FN<T, RED_MIN>())
#define BY_TYPE(FN, type, op)                                               \
  switch (type) {                                                           \
    case ncclInt8: return BY_OP(FN, int8_t, op);                            \
    case ncclUint8: return BY_OP(FN, uint8_t, op);                          \
    case ncclInt32: return BY_OP(FN, int32_t, op);                          \
    case ncclUint32: return BY_OP(FN, uint32_t, op);                        \
    case ncclInt64: return BY_OP(FN, int64_t, op);                          \
    case ncclUint64: return BY_OP(FN, uint64_t, op);                        \
    case ncclFloat16: return BY_OP(FN, __half, op);                         \
    case ncclFloat32: return BY_OP(FN, float, op);                          \
    case ncclFloat64: return BY_OP(FN, double, op);                         \
    case ncclBfloat16: return BY_OP(FN, __nv_bfloat16, op);                 \
    case ncclFloat8e4m3: return BY_OP(FN, F8E4, op);                        \
    case ncclFloat8e5m2: return BY_OP(FN, F8E5, op);                        \
    default: return nullptr;                                                \
  }

const void* reduceKernelFn(int algo, ncclDataType_t type, int op) {
  if (algo == KERNEL_REDUCE_P2P) { BY_TYPE(p2pFn, type, op) }
  if (algo == KERNEL_ALLREDUCE_LL) return llReduceKernelFn(type, op);
  if (algo == KERNEL_REDUCE_NVLS) { BY_TYPE(nvlsFn, type, op) }
  return nullptr;
}

bool nvlsReduceSupported(ncclDataType_t type, int op) { return reduceKernelFn(KERNEL_REDUCE_NVLS, type, op) != nullptr; }

}  // namespace b200
