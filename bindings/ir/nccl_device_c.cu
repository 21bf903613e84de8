// Definitions of the C-callable device API (see nccl_device_c.h): each function forwards to the C++ header of the
// same name, so a kernel language that can only call C symbols gets the same code after link-time optimisation.
#include "nccl_device_c.h"

#include <new>

using CtaBarrierSession = ncclLsaBarrierSession<ncclCoopCta>;

extern "C" {

__device__ size_t ncclLsaBarrierSession_C_size() { return sizeof(CtaBarrierSession); }
__device__ size_t ncclLLA2ASession_C_size() { return sizeof(ncclLLA2ASession<ncclCoopCta>); }

__device__ int ncclDevComm_Rank(const ncclDevComm_t* c) { return c->rank; }
__device__ int ncclDevComm_NRanks(const ncclDevComm_t* c) { return c->nRanks; }
__device__ int ncclDevComm_LsaRank(const ncclDevComm_t* c) { return c->lsaRank; }
__device__ int ncclDevComm_LsaSize(const ncclDevComm_t* c) { return c->lsaSize; }
__device__ int ncclDevComm_TestAbort(const ncclDevComm_t* c) { return ncclTestAbort(*c) ? 1 : 0; }

__device__ void* ncclGetLocalPointer_C(ncclWindow_t w, size_t offset) { return ncclGetLocalPointer(w, offset); }
__device__ void* ncclGetLsaPointer_C(ncclWindow_t w, size_t offset, int lsaPeer) { return ncclGetLsaPointer(w, offset, lsaPeer); }
__device__ void* ncclGetPeerPointer_C(ncclWindow_t w, size_t offset, int worldPeer) { return ncclGetPeerPointer(w, offset, worldPeer); }
__device__ void* ncclGetMultimemPointer_C(ncclWindow_t w, size_t offset) { return ncclGetMultimemPointer(w, offset); }

__device__ void ncclCoopAnyInitThread(ncclCoopAny* c) { *c = ncclCoopAny{0, 0, 0, 0}; }
__device__ void ncclCoopAnyInitWarp(ncclCoopAny* c) { *c = ncclCoopAny{1, 0, 1, 0}; }
__device__ void ncclCoopAnyInitCta(ncclCoopAny* c) { *c = ncclCoopAny{2, 0, 0, 0}; }
__device__ void ncclCoopAnyInitWarpSpan(ncclCoopAny* c, int warp0, int nWarps, int id) { *c = ncclCoopAny{3, warp0, nWarps, id}; }
__device__ int ncclCoopThreadRank(const ncclCoopAny* c) {
  switch (c->kind) {
    case 0: return 0;
    case 1: return threadIdx.x % 32;
    case 2: return ncclCoopCta().thread_rank();
    default: return ncclCoopWarpSpan(c->warp0, c->nWarps, c->barrierId).thread_rank();
  }
}
__device__ int ncclCoopSize(const ncclCoopAny* c) {
  switch (c->kind) {
    case 0: return 1;
    case 1: return 32;
    case 2: return ncclCoopCta().size();
    default: return 32 * c->nWarps;
  }
}
__device__ void ncclCoopSync(const ncclCoopAny* c) {
  switch (c->kind) {
    case 0: break;
    case 1: __syncwarp(); break;
    case 2: __syncthreads(); break;
    default: ncclCoopWarpSpan(c->warp0, c->nWarps, c->barrierId).sync(); break;
  }
}

__device__ void ncclLsaBarrierSessionInit(void* s, const ncclDevComm_t* comm, int barrierIndex) {
  new (s) CtaBarrierSession(ncclCoopCta(), *comm, ncclTeamLsa(*comm), barrierIndex);
}
__device__ void ncclLsaBarrierSessionArrive(void* s, int release) { ((CtaBarrierSession*)s)->arrive(release != 0); }
__device__ int ncclLsaBarrierSessionWait(void* s, int acquire, unsigned long long timeoutCycles) { return (int)((CtaBarrierSession*)s)->wait(timeoutCycles, acquire != 0); }
__device__ int ncclLsaBarrierSessionSync(void* s, int release, int acquire, unsigned long long timeoutCycles) {
  return (int)((CtaBarrierSession*)s)->sync(timeoutCycles, release != 0, acquire != 0);
}
__device__ void ncclLsaBarrierSessionFinish(void* s) { ((CtaBarrierSession*)s)->finish(); }

__device__ void ncclMultimemStore16_C(void* mc, unsigned x, unsigned y, unsigned z, unsigned w) { ncclMultimemStore16(mc, make_uint4(x, y, z, w)); }
__device__ void ncclMultimemRedAddU32_C(unsigned* mc, unsigned v) { ncclMultimemRedAddU32(mc, v); }
__device__ void ncclMultimemLdReduceSumF32x4_C(const void* mc, float* out4) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  out4[0] = __uint_as_float(v.x); out4[1] = __uint_as_float(v.y); out4[2] = __uint_as_float(v.z); out4[3] = __uint_as_float(v.w);
}
__device__ void ncclMultimemLdReduceSumBf16x8_C(const void* mc, unsigned* out4) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  out4[0] = v.x; out4[1] = v.y; out4[2] = v.z; out4[3] = v.w;
}

}  // extern "C"
