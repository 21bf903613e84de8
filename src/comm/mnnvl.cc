// Multi-node NVLink detection: fabric identity from NVML, cliques from the gathered records, a probe allocation.
// Reference parity: src/mnnvl.cc:13-100, src/init.cc:744-776,1070-1075.
#include "mnnvl.h"

#include <string.h>

#include "../core/cudawrap.h"
#include "../core/nvmlwrap.h"
#include "../mem/allocator.h"
#include "comm.h"

namespace b200 {

B200_PARAM(MnnvlEnable, "MNNVL_ENABLE", 2, "Multi-node NVLink: 0 off, 1 look for a fabric even on one host, 2 look for it when the job spans hosts")
B200_PARAM(MnnvlUuid, "MNNVL_UUID", -1, "Replaces both halves of the fabric's cluster UUID reported by NVML (testing, partitioning by hand)")
B200_PARAM(MnnvlCliqueId, "MNNVL_CLIQUE_ID", -1, "Replaces the fabric clique id reported by NVML")

namespace {
// Layout of NVML's nvmlGpuFabricInfoV_t (public nvml.h), version 2.
struct NvmlFabricInfoV {
  unsigned int version;
  unsigned char clusterUuid[16];
  int status;
  unsigned int cliqueId;
  unsigned char state;
  unsigned int healthMask;
};
constexpr unsigned int kNvmlFabricInfoV2 = (unsigned int)sizeof(NvmlFabricInfoV) | (2u << 24);
}  // namespace

void fabricInfoQuery(const char* busId, FabricInfo* out) {
  memset(out, 0, sizeof(*out));
  out->state = FABRIC_NOT_SUPPORTED;
  const NvmlApi* nv = nvmlApi();
  nvmlDevice_t dev;
  if (nv && nv->deviceGetGpuFabricInfoV && busId && nv->deviceGetHandleByPciBusId(busId, &dev) == 0) {
    union { NvmlFabricInfoV fi; unsigned char room[128]; } u;   // room to spare should a driver write a later, longer version
    memset(&u, 0, sizeof(u));
    NvmlFabricInfoV& fi = u.fi;
    fi.version = kNvmlFabricInfoV2;
    if (nv->deviceGetGpuFabricInfoV(dev, &fi) == 0) {
      memcpy(out->clusterUuid, fi.clusterUuid, kFabricUuidLen);
      out->cliqueId = fi.cliqueId;
      out->state = fi.state;
      out->healthMask = fi.healthMask;
      out->status = fi.status;
    }
  }
  if (out->state == FABRIC_NOT_SUPPORTED) return;
  if (paramMnnvlUuid() != -1) {
    uint64_t half = (uint64_t)paramMnnvlUuid();
    memcpy(out->clusterUuid, &half, 8);
    memcpy(out->clusterUuid + 8, &half, 8);
  }
  if (paramMnnvlCliqueId() >= 0) out->cliqueId = (uint32_t)paramMnnvlCliqueId();
}

bool mnnvlClique(const FabricInfo* infos, int n, int me, Clique* out) {
  *out = Clique();
  if (me < 0 || me >= n) return false;
  static const uint8_t zero[kFabricUuidLen] = {};
  for (int i = 0; i < n; ++i) {
    if (infos[i].state != FABRIC_COMPLETED) return false;
    if (memcmp(infos[i].clusterUuid, zero, kFabricUuidLen) == 0) return false;
  }
  out->id = infos[me].cliqueId;
  for (int i = 0; i < n; ++i) {
    if (memcmp(infos[i].clusterUuid, infos[me].clusterUuid, kFabricUuidLen) != 0) continue;
    out->domainSize++;
    if (infos[i].cliqueId != infos[me].cliqueId) continue;
    if (i == me) out->rank = (int)out->ranks.size();
    out->ranks.push_back(i);
  }
  return out->ranks.size() > 1 || out->domainSize > 1;
}

// One minimal allocation with a fabric handle, exported and imported again: shows whether the IMEX channel that the
// driver needs for fabric handles is set up for this process.
static bool fabricProbe(int cudaDev) {
  const CuApi* cu = cuApi();
  if (!cu) return false;
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = cudaDev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_FABRIC;
  size_t gran = 0;
  if (cu->cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM) != CUDA_SUCCESS || gran == 0) return false;
  CUmemGenericAllocationHandle h = 0, back = 0;
  if (cu->cuMemCreate(&h, gran, &prop, 0) != CUDA_SUCCESS) return false;
  CUmemFabricHandle fh;
  bool ok = cu->cuMemExportToShareableHandle(&fh, h, CU_MEM_HANDLE_TYPE_FABRIC, 0) == CUDA_SUCCESS &&
            cu->cuMemImportFromShareableHandle(&back, &fh, CU_MEM_HANDLE_TYPE_FABRIC) == CUDA_SUCCESS;
  if (back) cu->cuMemRelease(back);
  cu->cuMemRelease(h);
  return ok;
}

ncclResult_t mnnvlCheck(ncclComm* comm) {
  comm->mnnvl = false;
  const int enable = (int)paramMnnvlEnable();
  if (enable == 0 || comm->hostOnly) return ncclSuccess;
  if (!(enable == 1 || comm->nNodes > 1)) return ncclSuccess;
  const int n = comm->nRanks;
  std::vector<FabricInfo> infos(n);
  for (int i = 0; i < n; ++i) infos[i] = comm->peers[i].fabric;
  if (!mnnvlClique(infos.data(), n, comm->rank, &comm->clique)) return ncclSuccess;
  if (!cuFabricSupported(comm->cudaDev)) return ncclSuccess;
  if (!fabricProbe(comm->cudaDev)) {
    WARN("multi-node NVLink (clique of %zu ranks) is reported by the fabric but fabric memory handles do not work in this process: check the IMEX "
         "channels (/dev/nvidia-caps-imex-channels, nvidia-imex-ctl -N), or set NCCL_MNNVL_ENABLE=0", comm->clique.ranks.size());
    return ncclSystemError;
  }
  comm->mnnvl = true;
  memSetHandleType(CU_MEM_HANDLE_TYPE_FABRIC);
  INFO(SUB_INIT, "multi-node NVLink: clique 0x%x of %zu ranks (this rank is number %d), %d ranks in the fabric", comm->clique.id, comm->clique.ranks.size(),
       comm->clique.rank, comm->clique.domainSize);
  return ncclSuccess;
}

}  // namespace b200

// Test hook: the clique of rank `me` from n records of {uuid[16], cliqueId, state}; writes the member ranks, returns the
// clique size (0 when the ranks do not form a multi-rank fabric) and the domain size through *domain.
extern "C" int b200MnnvlClique(const b200::FabricInfo* infos, int n, int me, int* ranks, int* domain) {
  b200::Clique c;
  if (!b200::mnnvlClique(infos, n, me, &c)) { if (domain) *domain = c.domainSize; return 0; }
  for (size_t i = 0; i < c.ranks.size(); ++i) ranks[i] = c.ranks[i];
  if (domain) *domain = c.domainSize;
  return (int)c.ranks.size();
}

// Test hooks: a table of NVML entry points built by the caller (a fake NVML; null restores the real one), and the
// fabric query as the communicator bring-up runs it.
extern "C" void b200NvmlSetApiForTest(const b200::NvmlApi* fake) { b200::nvmlSetApiForTest(fake); }
extern "C" void b200FabricInfoQuery(const char* busId, b200::FabricInfo* out) { b200::fabricInfoQuery(busId, out); }
