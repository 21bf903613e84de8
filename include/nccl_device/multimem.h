/*
 * Typed wrappers of the NVLink-SHARP instructions on multicast addresses: multimem.ld_reduce (the
 * switch reduces the copies of all ranks), multimem.st (the switch stores to all ranks) and
 * multimem.red. 16-byte forms for fp32 / fp16x2 / bf16x2 / e4m3x4 / e5m2x4.
 * Reference parity: src/include/nccl_device/impl/multimem__funcs.h.
 */
#ifndef NCCL_DEVICE_MULTIMEM_H_
#define NCCL_DEVICE_MULTIMEM_H_
#if defined(__CUDACC__)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#define NCCL_MULTIMEM_LD(NAME, INSTR)                                                                       \
  __device__ __forceinline__ uint4 NAME(const void* mc) {                                                   \
    uint4 v;                                                                                                \
    asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " {%0,%1,%2,%3}, [%4];"                     \
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");                        \
    return v;                                                                                               \
  }
NCCL_MULTIMEM_LD(ncclMultimemLoadSumF32x4, "add.v4.f32")
NCCL_MULTIMEM_LD(ncclMultimemLoadSumF16x8, "add.acc::f32.v4.f16x2")
NCCL_MULTIMEM_LD(ncclMultimemLoadSumBf16x8, "add.acc::f32.v4.bf16x2")
NCCL_MULTIMEM_LD(ncclMultimemLoadSumE4m3x16, "add.acc::f16.v4.e4m3x4")
NCCL_MULTIMEM_LD(ncclMultimemLoadSumE5m2x16, "add.acc::f16.v4.e5m2x4")
NCCL_MULTIMEM_LD(ncclMultimemLoadMaxBf16x8, "max.v4.bf16x2")
NCCL_MULTIMEM_LD(ncclMultimemLoadMinBf16x8, "min.v4.bf16x2")
NCCL_MULTIMEM_LD(ncclMultimemLoadMaxF16x8, "max.v4.f16x2")
NCCL_MULTIMEM_LD(ncclMultimemLoadMinF16x8, "min.v4.f16x2")
#undef NCCL_MULTIMEM_LD
__device__ __forceinline__ void ncclMultimemStore16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void ncclMultimemRedAddU32(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
__device__ __forceinline__ void ncclMultimemRedAddF32(float* mc, float v) {
  asm volatile("multimem.red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(mc), "f"(v) : "memory");
}
#endif
#endif
