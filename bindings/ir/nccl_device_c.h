/*
 * The device API as plain C functions, for compilers of kernel languages that cannot include C++ templates.
 * The functions are built into a device library that carries link-time-optimisation IR (NVVM IR, produced with
 * `nvcc -dc -dlto`; `make ir` -> nccl_b200/lib/libnccl_device_c.a): a DSL compiler emits calls to these symbols
 * and links the library with nvJitLink or `nvcc -dlto`, after which the calls inline like the C++ originals.
 * Opaque objects (barrier sessions, cooperative groups) live in caller-provided storage whose size the
 * *_C_size() functions report.
 * Reference parity: bindings/ir/nccl_device_wrapper.h (the same idea, delivered there as LLVM bitcode built with clang).
 */
#ifndef NCCL_DEVICE_C_H_
#define NCCL_DEVICE_C_H_
#include "nccl_device.h"

#ifdef __cplusplus
#define NCCL_IR_EXTERN_C extern "C"
#else
#define NCCL_IR_EXTERN_C
#endif

/* cooperative group chosen at run time: kind 0 thread, 1 warp, 2 CTA, 3 span of warps */
typedef struct { int kind, warp0, nWarps, barrierId; } ncclCoopAny;

NCCL_IR_EXTERN_C __device__ size_t ncclLsaBarrierSession_C_size();
NCCL_IR_EXTERN_C __device__ size_t ncclLLA2ASession_C_size();

/* communicator fields */
NCCL_IR_EXTERN_C __device__ int ncclDevComm_Rank(const ncclDevComm_t* comm);
NCCL_IR_EXTERN_C __device__ int ncclDevComm_NRanks(const ncclDevComm_t* comm);
NCCL_IR_EXTERN_C __device__ int ncclDevComm_LsaRank(const ncclDevComm_t* comm);
NCCL_IR_EXTERN_C __device__ int ncclDevComm_LsaSize(const ncclDevComm_t* comm);
NCCL_IR_EXTERN_C __device__ int ncclDevComm_TestAbort(const ncclDevComm_t* comm);

/* window pointers */
NCCL_IR_EXTERN_C __device__ void* ncclGetLocalPointer_C(ncclWindow_t w, size_t offset);
NCCL_IR_EXTERN_C __device__ void* ncclGetLsaPointer_C(ncclWindow_t w, size_t offset, int lsaPeer);
NCCL_IR_EXTERN_C __device__ void* ncclGetPeerPointer_C(ncclWindow_t w, size_t offset, int worldPeer);
NCCL_IR_EXTERN_C __device__ void* ncclGetMultimemPointer_C(ncclWindow_t w, size_t offset);

/* cooperative groups */
NCCL_IR_EXTERN_C __device__ void ncclCoopAnyInitThread(ncclCoopAny* coop);
NCCL_IR_EXTERN_C __device__ void ncclCoopAnyInitWarp(ncclCoopAny* coop);
NCCL_IR_EXTERN_C __device__ void ncclCoopAnyInitCta(ncclCoopAny* coop);
NCCL_IR_EXTERN_C __device__ void ncclCoopAnyInitWarpSpan(ncclCoopAny* coop, int warp0, int nWarps, int id);
NCCL_IR_EXTERN_C __device__ int ncclCoopThreadRank(const ncclCoopAny* coop);
NCCL_IR_EXTERN_C __device__ int ncclCoopSize(const ncclCoopAny* coop);
NCCL_IR_EXTERN_C __device__ void ncclCoopSync(const ncclCoopAny* coop);

/* barrier over the load/store domain: the whole CTA takes part (storage: ncclLsaBarrierSession_C_size() bytes, 8-byte aligned) */
NCCL_IR_EXTERN_C __device__ void ncclLsaBarrierSessionInit(void* session, const ncclDevComm_t* comm, int barrierIndex);
NCCL_IR_EXTERN_C __device__ void ncclLsaBarrierSessionArrive(void* session, int release);
NCCL_IR_EXTERN_C __device__ int ncclLsaBarrierSessionWait(void* session, int acquire, unsigned long long timeoutCycles);   /* ncclResult_t */
NCCL_IR_EXTERN_C __device__ int ncclLsaBarrierSessionSync(void* session, int release, int acquire, unsigned long long timeoutCycles);
NCCL_IR_EXTERN_C __device__ void ncclLsaBarrierSessionFinish(void* session);

/* multimem */
NCCL_IR_EXTERN_C __device__ void ncclMultimemStore16_C(void* mc, unsigned x, unsigned y, unsigned z, unsigned w);
NCCL_IR_EXTERN_C __device__ void ncclMultimemRedAddU32_C(unsigned* mc, unsigned v);
NCCL_IR_EXTERN_C __device__ void ncclMultimemLdReduceSumF32x4_C(const void* mc, float* out4);
NCCL_IR_EXTERN_C __device__ void ncclMultimemLdReduceSumBf16x8_C(const void* mc, unsigned* out4);

#endif
