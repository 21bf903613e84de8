// Host thread of the proxy mode of the GPU-initiated put / signal surface (gin_proxy.cu).
#pragma once
#include "nccl.h"
#include "nccl_device/core.h"

namespace b200 {

struct GinProxy;
// Allocates the descriptor ring (at least `depth` entries, a power of two) and the completion words on `dev`, starts the
// thread and fills the ginProxy* fields of `dc`.
ncclResult_t ginProxyCreate(int dev, int depth, GinProxy** out, ncclDevComm_t* dc);
void ginProxyDestroy(GinProxy* p);
unsigned long long ginProxyServed(const GinProxy* p);   // operations taken from the ring so far
int ginProxyError(const GinProxy* p);                   // first error of the thread (ncclResult_t), 0 = none

}  // namespace b200
