// Compile-only check: kernels written with the reference's spellings of the device API (team tags, scoped
// barrier sessions with memory orders, typed put / signal actions, team arithmetic) build against this
// library's headers. Used by tests/test_device_api_compile.py.
#include "nccl_device.h"

__global__ void lsaAllReduce(ncclDevComm devComm, ncclWindow_t win, size_t count) {
  ncclLsaBarrierSession<ncclCoopCta> bar{ncclCoopCta(), devComm, ncclTeamTagLsa(), blockIdx.x};
  bar.sync(ncclCoopCta(), cuda::memory_order_relaxed);
  ncclTeam lsa = ncclTeamLsa(devComm);
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
    float v = 0;
    for (int p = 0; p < lsa.nRanks; ++p) v += ((float*)ncclGetLsaPointer(win, 0, p))[i];
    for (int p = 0; p < lsa.nRanks; ++p) ((float*)ncclGetLsaPointer(win, count * sizeof(float), p))[i] = v;
  }
  if (bar.sync(ncclCoopCta(), cuda::memory_order_release, 1000000ull) != ncclSuccess) return;
}

__global__ void ginRing(ncclDevComm devComm, ncclWindow_t win, size_t bytes, ncclGinSignal_t sig) {
  ncclGin gin{devComm, 0};
  ncclTeam world = ncclTeamWorld(devComm);
  const int next = (world.rank + 1) % world.nRanks;
  uint64_t before = gin.readSignal(sig, 64);
  gin.put(world, next, win, bytes, win, 0, bytes, ncclGin_SignalInc{sig}, ncclGin_None{}, ncclCoopCta());
  gin.put(world, next, win, bytes, win, 0, bytes, ncclGin_WeakSignalInc{sig});
  gin.put(world, next, win, bytes, win, 0, bytes, ncclGin_StrongVASignalAdd{win, 2 * bytes, 3}, ncclGin_WeakCounterInc{0});
  gin.putValue(world, next, win, 0, 42u, ncclGin_SignalAdd{sig, 2});
  gin.signal(world, next, ncclGin_StrongSignalInc{sig});
  gin.waitSignal(ncclCoopCta(), sig, before + 1);
  gin.flush(ncclCoopCta());
  ncclGinBarrierSession<ncclCoopCta> gbar{ncclCoopCta(), gin, ncclTeamTagWorld(), 0};
  gbar.sync(ncclCoopCta(), cuda::memory_order_acq_rel, ncclGinFenceLevel::Put | ncclGinFenceLevel::Get);
  ncclBarrierSession<ncclCoopCta> wbar{ncclCoopCta(), ncclTeamTagWorld(), gin, 1};
  wbar.sync(ncclCoopCta(), cuda::memory_order_acq_rel, ncclGinFenceLevel::Relaxed);
}

__global__ void teams(ncclDevComm devComm, int* out) {
  ncclTeam world = ncclTeamWorld(devComm), lsa = ncclTeamLsa(devComm), rail = ncclTeamRail(devComm);
  ncclTeam inner = ncclTeamInnerFactor(world, 2), outer = ncclTeamOuterFactor(world, 2);
  out[0] = ncclTeamRankToWorld(devComm, lsa, 0) + ncclTeamRankToLsa(devComm, world, world.rank) + ncclTeamRankToTeam(lsa, world, 0);
  ncclDevResourceHandle_t h = 256;
  out[2] = (int)ncclGetResourceBufferOffset(h) + (ncclGetResourceBufferPeerPointer(devComm, h, world, 0) != ncclGetResourceBufferLsaPointer(devComm, h, 0)) +
           (ncclGetResourceBufferLsaMultimemPointer(devComm, h) != nullptr);
  out[1] = ncclTeamRankIsMember(inner, world, 1) + ncclTeamRankInDifference(world, inner, 0) + outer.nRanks + rail.nRanks;
}

__global__ void reduceCopy(ncclDevComm devComm, ncclWindow_t in, ncclWindow_t out, float* local, __nv_bfloat16* localH, size_t count) {
  ncclCoopCta cta;
  ncclTeam lsa = ncclTeamLsa(devComm);
  ncclLsaReduceSumCopy<float>(cta, in, 0, out, 0, count, lsa);
  ncclLsaReduceSumCopy<float>(cta, in, 0, out, 0, count, devComm);
  ncclLsaReduceSum<float>(cta, in, 0, local, count, lsa);
  ncclLsaCopy<float>(cta, local, out, 0, count, devComm);
  ncclLsaReduceSumLsaCopy<__nv_bfloat16>(cta, [=](int i) { return (__nv_bfloat16*)ncclGetLsaPointer(in, 0, i); }, lsa.nRanks,
                                         [=](int j) { return (__nv_bfloat16*)ncclGetLsaPointer(out, 0, j); }, lsa.nRanks, count);
  ncclLocalReduceSum<__nv_bfloat16>(cta, [=](int i) { return localH + i * count; }, 2, localH, count);
  ncclLocalCopy<float>(cta, local, [=](int j) { return local + (j + 1) * count; }, 2, count);
  ncclSymPtr<float> src(in, 0), dst(out, 0);
  ncclLsaReduceSumCopy<float>(cta, src, dst, count, lsa);
  ncclMultimemReduceSumMultimemCopy<float>(cta, (float*)ncclGetMultimemPointer(in, 0), (float*)ncclGetMultimemPointer(out, 0), count);
}

int main() {
  ncclDevCommRequirements reqs = NCCL_DEV_COMM_REQUIREMENTS_INITIALIZER;
  reqs.lsaBarrierCount = 4;
  ncclCommProperties props = NCCL_COMM_PROPERTIES_INITIALIZER;
  (void)reqs; (void)props;
  return 0;
}
