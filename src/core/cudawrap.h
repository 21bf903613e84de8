// CUDA driver entry points resolved at run time through the runtime (no link-time dependency
// on libcuda, so the library loads on machines without a GPU driver).
// Reference parity: src/misc/cudawrap.cc (CUPFN table, ncclCuMemEnable, :338).
#pragma once
#include <cuda.h>

#include "core.h"

namespace b200 {

struct CuApi {
  CUresult (*cuGetErrorString)(CUresult, const char**);
  CUresult (*cuDeviceGet)(CUdevice*, int);
  CUresult (*cuDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*cuCtxGetCurrent)(CUcontext*);
  CUresult (*cuMemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*cuMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*cuMemRelease)(CUmemGenericAllocationHandle);
  CUresult (*cuMemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*cuMemAddressFree)(CUdeviceptr, size_t);
  CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*cuMemUnmap)(CUdeviceptr, size_t);
  CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*cuMemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*cuMemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*cuMemRetainAllocationHandle)(CUmemGenericAllocationHandle*, void*);
  CUresult (*cuMemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr);
  CUresult (*cuMulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*cuMulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*cuMulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*cuMulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*cuMulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*cuStreamWriteValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
  CUresult (*cuStreamWaitValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
  CUresult (*cuStreamWriteValue64)(CUstream, CUdeviceptr, cuuint64_t, unsigned int);   // optional
  CUresult (*cuPointerGetAttribute)(void*, CUpointer_attribute, CUdeviceptr);
};

// Null when no driver is present. The table is filled once.
const CuApi* cuApi();
const char* cuErrStr(CUresult r);
bool cuMemSupported(int cudaDev);       // VMM with POSIX-fd handles (NCCL_CUMEM_ENABLE, default on)
bool cuMulticastSupported(int cudaDev); // NVLS multicast objects (NCCL_NVLS_ENABLE, default on)
bool cuFabricSupported(int cudaDev);    // memory can be created with fabric handles (multi-node NVLink)
// Handle type that shareable device memory is created with: POSIX file descriptors, or fabric handles once a
// communicator found that its ranks share an NVLink fabric across hosts (process-wide, like the allocations it governs).
CUmemAllocationHandleType memHandleType();
void memSetHandleType(CUmemAllocationHandleType t);

#define CUCHECK(call)                                                                  \
  do {                                                                                 \
    CUresult _r = (call);                                                              \
    if (_r != CUDA_SUCCESS) {                                                          \
      WARN("CUDA driver failure '%s' at %s:%d", ::b200::cuErrStr(_r), __FILE__, __LINE__); \
      return ncclUnhandledCudaError;                                                   \
    }                                                                                  \
  } while (0)

}  // namespace b200
