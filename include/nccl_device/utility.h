/*
 * Small device helpers: memory-ordering wrappers, abort test, bounded polling.
 * Reference parity: src/include/nccl_device/utility.h (testAbort, rolling compares).
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
}  // namespace nccl_device

/* True once the host has aborted the communicator; kernels poll this inside long waits. */
__device__ inline bool ncclTestAbort(const ncclDevComm_t& c) { return c.abortFlag && nccl_device::ldRelaxedSys(c.abortFlag) != 0; }
#endif
#endif
