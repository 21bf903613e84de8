#include "nvmlwrap.h"

#include <dlfcn.h>

#include <mutex>

namespace b200 {

static NvmlApi gNvml;
static const NvmlApi* gActive = nullptr;
static std::once_flag gOnce;
static const NvmlApi* gFake = nullptr;

void nvmlSetApiForTest(const NvmlApi* fake) { gFake = fake; }

const NvmlApi* nvmlApi() {
  if (gFake) return gFake;
  std::call_once(gOnce, [] {
    void* h = dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
    if (!h) return;
    int (*init)() = (int (*)())dlsym(h, "nvmlInit_v2");
    if (!init || init() != 0) return;
    bool ok = true;
    auto load = [&](void** fn, const char* a, const char* b) {
      *fn = dlsym(h, a);
      if (!*fn && b) *fn = dlsym(h, b);
      if (!*fn) ok = false;
    };
    load((void**)&gNvml.deviceGetCount, "nvmlDeviceGetCount_v2", "nvmlDeviceGetCount");
    load((void**)&gNvml.deviceGetHandleByIndex, "nvmlDeviceGetHandleByIndex_v2", "nvmlDeviceGetHandleByIndex");
    load((void**)&gNvml.deviceGetHandleByPciBusId, "nvmlDeviceGetHandleByPciBusId_v2", "nvmlDeviceGetHandleByPciBusId");
    load((void**)&gNvml.deviceGetIndex, "nvmlDeviceGetIndex", nullptr);
    load((void**)&gNvml.deviceGetNvLinkState, "nvmlDeviceGetNvLinkState", nullptr);
    load((void**)&gNvml.deviceGetNvLinkRemotePciInfo, "nvmlDeviceGetNvLinkRemotePciInfo_v2", "nvmlDeviceGetNvLinkRemotePciInfo");
    load((void**)&gNvml.deviceGetP2PStatus, "nvmlDeviceGetP2PStatus", nullptr);
    load((void**)&gNvml.deviceGetCudaComputeCapability, "nvmlDeviceGetCudaComputeCapability", nullptr);
    gNvml.deviceGetGpuFabricInfoV = (int (*)(nvmlDevice_t, void*))dlsym(h, "nvmlDeviceGetGpuFabricInfoV");
    if (ok) gActive = &gNvml;
  });
  return gActive;
}

}  // namespace b200
