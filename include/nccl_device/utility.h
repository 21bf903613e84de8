/*
 * Small device helpers: memory-ordering wrappers, abort test, rolling comparisons, division by a
 * kernel-constant divisor, pointer and alignment arithmetic, lane identifiers.
 * Reference parity: src/include/nccl_device/utility.h (testAbort, rolling compares, fast division, pointer math).
 */
#ifndef NCCL_DEVICE_UTILITY_H_
#define NCCL_DEVICE_UTILITY_H_
#include "core.h"
#if defined(__CUDACC__)
namespace nccl_device {
__device__ __forceinline__ uint32_t ldAcquireSys(const uint32_t* p) { uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ uint32_t ldRelaxedSys(const uint32_t* p) { uint32_t v; asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void stReleaseSys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void stRelaxedSys(uint32_t* p, uint32_t v) { asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void fenceAcqRelSys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ uint4 ldVolatile16(const void* p) { uint4 v; asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void stVolatile16(void* p, uint4 v) { asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory"); }
/* a - b in modular arithmetic: >= 0 when a is at or past b */
__device__ __forceinline__ int rollingDiff(uint32_t a, uint32_t b) { return (int)(a - b); }
/* Rolling (wrap-around) comparisons of counters that only ever increase: valid while the two values are less
 * than half the counter's range apart. */
__device__ __forceinline__ bool rollingLessEq(uint32_t a, uint32_t b) { return (int32_t)(b - a) >= 0; }
__device__ __forceinline__ bool rollingLessEq(uint64_t a, uint64_t b) { return (int64_t)(b - a) >= 0; }
__device__ __forceinline__ uint32_t rollingMin(uint32_t a, uint32_t b) { return rollingLessEq(a, b) ? a : b; }
__device__ __forceinline__ uint32_t rollingMax(uint32_t a, uint32_t b) { return rollingLessEq(a, b) ? b : a; }

/* Division by a divisor that is fixed for a whole kernel (a rank count, a tile count): the reciprocal is computed
 * once, on the host or at kernel start, and every division becomes a multiply-high plus one correction step.
 *   ncclFastDiv32 d = ncclFastDiv32::make(nRanks);   q = d.div(x);   r = d.mod(x);
 * Exact for every 32-bit x and every d >= 1. */
struct ncclFastDiv32 {
  uint32_t d, rcp;   /* rcp = floor(2^32 / d) (0 stands for d == 1) */
  __host__ __device__ static ncclFastDiv32 make(uint32_t d) {
    ncclFastDiv32 f;
    f.d = d;
    f.rcp = d <= 1 ? 0u : (uint32_t)(0x100000000ull / d);
    return f;
  }
  __device__ __forceinline__ uint32_t div(uint32_t x) const {
    if (d <= 1) return x;
    uint32_t q = __umulhi(x, rcp);          /* q <= x / d, short by at most 1 */
    if (x - q * d >= d) ++q;
    return q;
  }
  __device__ __forceinline__ uint32_t mod(uint32_t x) const { return x - div(x) * d; }
  __device__ __forceinline__ void divmod(uint32_t x, uint32_t* q, uint32_t* r) const { *q = div(x); *r = x - *q * d; }
};

/* Pointer arithmetic in bytes, and alignment helpers for packs of 2^k bytes. */
template <typename T> __host__ __device__ __forceinline__ T* ncclPtrAddBytes(T* p, size_t bytes) { return (T*)((char*)p + bytes); }
template <typename T> __host__ __device__ __forceinline__ size_t ncclPtrDiffBytes(const T* a, const T* b) { return (size_t)((const char*)a - (const char*)b); }
__host__ __device__ __forceinline__ bool ncclIsAligned(const void* p, size_t bytes) { return ((size_t)p & (bytes - 1)) == 0; }
__host__ __device__ __forceinline__ size_t ncclAlignUp(size_t x, size_t a) { return (x + a - 1) / a * a; }
__host__ __device__ __forceinline__ size_t ncclAlignDown(size_t x, size_t a) { return x / a * a; }
__host__ __device__ __forceinline__ size_t ncclDivUp(size_t x, size_t y) { return (x + y - 1) / y; }

/* Lane helpers used by the cooperative loops. */
__device__ __forceinline__ unsigned ncclLaneId() { unsigned l; asm("mov.u32 %0, %%laneid;" : "=r"(l)); return l; }
__device__ __forceinline__ unsigned ncclLaneMaskLt() { unsigned m; asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m)); return m; }
__device__ __forceinline__ unsigned long long ncclGlobalTimerNs() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
}  // namespace nccl_device

/* True once the host has aborted the communicator; kernels poll this inside long waits. */
__device__ inline bool ncclTestAbort(const ncclDevComm_t& c) { return c.abortFlag && nccl_device::ldRelaxedSys(c.abortFlag) != 0; }
#endif
#endif
