// A kernel of the kind a DSL compiler would emit: it knows the device API only as C symbols.
#include "nccl_device_c.h"

extern "C" __global__ void irAllGatherWord(const ncclDevComm_t* comm, ncclWindow_t win, unsigned* status) {
  extern __shared__ __align__(8) unsigned char storage[];
  ncclCoopAny cta;
  ncclCoopAnyInitCta(&cta);
  const int me = ncclDevComm_LsaRank(comm), n = ncclDevComm_LsaSize(comm);
  ncclLsaBarrierSessionInit(storage, comm, blockIdx.x);
  // every rank writes its number into slot `me` of every peer, then all ranks meet
  for (int p = ncclCoopThreadRank(&cta); p < n; p += ncclCoopSize(&cta)) {
    unsigned* dst = (unsigned*)ncclGetLsaPointer_C(win, sizeof(unsigned) * me, p);
    *dst = (unsigned)me + 1u;
  }
  int rc = ncclLsaBarrierSessionSync(storage, 1, 1, 1ull << 30);
  ncclCoopSync(&cta);
  if (ncclCoopThreadRank(&cta) == 0) status[blockIdx.x] = (unsigned)rc | (ncclDevComm_TestAbort(comm) ? 0x100u : 0u);
  ncclLsaBarrierSessionFinish(storage);
}

int main() { return 0; }
