// Resolves the CUDA driver functions the memory runtime needs.
// Reference parity: src/misc/cudawrap.cc (driver table through cudaGetDriverEntryPoint).
#include "cudawrap.h"

#include <atomic>

#include <mutex>

namespace b200 {

B200_PARAM(CuMemEnable, "CUMEM_ENABLE", 1, "Allocate with the virtual-memory API so buffers can be shared and multicast-bound")
B200_PARAM(NvlsEnable, "NVLS_ENABLE", 1, "Use NVLink SHARP multicast (multimem) when the hardware has it")

static CuApi gApi;
static bool gOk = false;
static std::once_flag gOnce;

template <typename F>
static bool load(F& fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || !p) {
    (void)cudaGetLastError();
    fn = nullptr;
    return false;
  }
  fn = (F)p;
  return true;
}

const CuApi* cuApi() {
  std::call_once(gOnce, [] {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { (void)cudaGetLastError(); return; }
    bool ok = true;
#define L(name) ok &= load(gApi.name, #name)
    L(cuGetErrorString); L(cuDeviceGet); L(cuDeviceGetAttribute); L(cuCtxGetCurrent);
    L(cuMemGetAllocationGranularity); L(cuMemCreate); L(cuMemRelease); L(cuMemAddressReserve);
    L(cuMemAddressFree); L(cuMemMap); L(cuMemUnmap); L(cuMemSetAccess); L(cuMemExportToShareableHandle);
    L(cuMemImportFromShareableHandle); L(cuMemRetainAllocationHandle); L(cuMemGetAddressRange);
    L(cuStreamWriteValue32); L(cuStreamWaitValue32); L(cuPointerGetAttribute);
#undef L
    // multicast entry points are optional (older drivers)
    load(gApi.cuStreamWriteValue64, "cuStreamWriteValue64");
    load(gApi.cuMulticastCreate, "cuMulticastCreate");
    load(gApi.cuMulticastAddDevice, "cuMulticastAddDevice");
    load(gApi.cuMulticastBindMem, "cuMulticastBindMem");
    load(gApi.cuMulticastUnbind, "cuMulticastUnbind");
    load(gApi.cuMulticastGetGranularity, "cuMulticastGetGranularity");
    gOk = ok;
    if (!ok) INFO(SUB_INIT, "CUDA driver entry points incomplete: virtual-memory features disabled");
  });
  return gOk ? &gApi : nullptr;
}

const char* cuErrStr(CUresult r) {
  const char* s = "unknown";
  const CuApi* a = cuApi();
  if (a && a->cuGetErrorString) a->cuGetErrorString(r, &s);
  return s ? s : "unknown";
}

static int devAttr(int cudaDev, CUdevice_attribute attr) {
  const CuApi* a = cuApi();
  if (!a) return 0;
  CUdevice d;
  int v = 0;
  if (a->cuDeviceGet(&d, cudaDev) != CUDA_SUCCESS) return 0;
  if (a->cuDeviceGetAttribute(&v, attr, d) != CUDA_SUCCESS) return 0;
  return v;
}

bool cuMemSupported(int cudaDev) {
  if (!paramCuMemEnable()) return false;
  return devAttr(cudaDev, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED) &&
         devAttr(cudaDev, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED);
}

bool cuFabricSupported(int cudaDev) { return cuMemSupported(cudaDev) && devAttr(cudaDev, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_FABRIC_SUPPORTED); }

static std::atomic<int> gHandleType{(int)CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR};
CUmemAllocationHandleType memHandleType() { return (CUmemAllocationHandleType)gHandleType.load(std::memory_order_relaxed); }
void memSetHandleType(CUmemAllocationHandleType t) { gHandleType.store((int)t, std::memory_order_relaxed); }

bool cuMulticastSupported(int cudaDev) {
  if (!paramNvlsEnable()) return false;
  const CuApi* a = cuApi();
  if (!a || !a->cuMulticastCreate) return false;
  return cuMemSupported(cudaDev) && devAttr(cudaDev, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED);
}

}  // namespace b200
