// NVML entry points loaded at run time (libnvidia-ml.so.1 is optional).
// Reference parity: src/misc/nvmlwrap.cc (dlopen'd NVML: device handles, NVLink state and remote
// PCI info, P2P status). Only reads settings; nothing here changes the state of a GPU.
#pragma once
#include "core.h"

namespace b200 {

typedef struct nvmlDevice_st* nvmlDevice_t;
struct nvmlPciInfo_t {
  char busIdLegacy[16];
  unsigned int domain, bus, device, pciDeviceId, pciSubSystemId;
  char busId[32];
};

struct NvmlApi {
  int (*deviceGetCount)(unsigned int*);
  int (*deviceGetHandleByIndex)(unsigned int, nvmlDevice_t*);
  int (*deviceGetHandleByPciBusId)(const char*, nvmlDevice_t*);
  int (*deviceGetIndex)(nvmlDevice_t, unsigned int*);
  int (*deviceGetNvLinkState)(nvmlDevice_t, unsigned int, unsigned int*);
  int (*deviceGetNvLinkRemotePciInfo)(nvmlDevice_t, unsigned int, nvmlPciInfo_t*);
  int (*deviceGetP2PStatus)(nvmlDevice_t, nvmlDevice_t, int, int*);
  int (*deviceGetCudaComputeCapability)(nvmlDevice_t, int*, int*);
  int (*deviceGetGpuFabricInfoV)(nvmlDevice_t, void* /* nvmlGpuFabricInfoV_t */);   // optional: null with older drivers
};

// Null when NVML is not installed or fails to initialise.
const NvmlApi* nvmlApi();
// Test hook: replaces the table (a fake NVML) for code that must not touch real devices.
void nvmlSetApiForTest(const NvmlApi* fake);

}  // namespace b200
