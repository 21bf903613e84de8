// Multi-node NVLink: ranks on different hosts whose GPUs sit in one NVLink fabric partition ("clique") form one
// load/store domain. The fabric identity of each GPU comes from NVML (cluster UUID + clique id); when every rank of
// a communicator is in this rank's clique, device memory is created with fabric handles, which are plain bytes that
// travel over the bootstrap network instead of file descriptors over UNIX sockets, and the symmetric data plane then
// spans the hosts.
// Reference parity: src/mnnvl.cc (ncclMnnvlCheck), src/init.cc:744-776 (fabric info, NCCL_MNNVL_UUID / _CLIQUE_ID), :1070.
#pragma once
#include <stdint.h>

#include <vector>

#include "../core/core.h"

struct ncclComm;

namespace b200 {

constexpr int kFabricUuidLen = 16;
enum { FABRIC_NOT_SUPPORTED = 0, FABRIC_NOT_STARTED = 1, FABRIC_IN_PROGRESS = 2, FABRIC_COMPLETED = 3 };

struct FabricInfo {
  uint8_t clusterUuid[kFabricUuidLen];
  uint32_t cliqueId;
  int32_t state;        // FABRIC_*
  uint32_t healthMask;
  int32_t status;       // NVML's result of the fabric probe
};

struct Clique {
  uint32_t id = 0;
  int rank = -1;        // this rank's position in `ranks`
  int domainSize = 0;   // ranks with the same cluster UUID (any clique)
  std::vector<int> ranks;
};

// Fabric identity of the GPU with this PCI bus id ("0000:1b:00.0"); zeroed with state NOT_SUPPORTED when NVML does not
// know. NCCL_MNNVL_UUID / NCCL_MNNVL_CLIQUE_ID replace what NVML reports.
void fabricInfoQuery(const char* busId, FabricInfo* out);

// Clique of rank `me` among `n` gathered records. False when the fabric is not ready on some rank, when a UUID is
// zero, or when nobody shares this rank's fabric (clique and domain of one).
bool mnnvlClique(const FabricInfo* infos, int n, int me, Clique* out);

// Decides whether this communicator uses fabric handles (comm->mnnvl) and fills comm->clique. Fails only when the
// fabric says it is usable and a probe allocation shows that it is not (IMEX channel set-up).
ncclResult_t mnnvlCheck(ncclComm* comm);

}  // namespace b200
