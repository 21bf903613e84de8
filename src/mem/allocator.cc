// ncclMemAlloc / ncclMemFree: physical memory from cuMemCreate with a shareable handle (POSIX fd; fabric
// handles when multi-node NVLink is in use),
// mapped read-write for every device that can reach it, so that windows over it can be mapped by
// peers and bound to NVLink multicast objects. Falls back to cudaMalloc without the VMM API.
// Reference parity: src/allocator.cc:17-139.
#include "allocator.h"

#include <map>
#include <mutex>

namespace b200 {

static std::mutex gLock;
static std::map<uintptr_t, MemAlloc> gAllocs;  // keyed by base address
static uint64_t gTotal = 0;

size_t shareableGranularity(int dev) {
  const CuApi* cu = cuApi();
  size_t gran = 2 << 20;
  if (!cu) return gran;
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = memHandleType();
  size_t g = 0;
  if (cu->cuMemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && g > gran) gran = g;
  if (cuMulticastSupported(dev)) {
    CUmulticastObjectProp mp = {};
    mp.numDevices = 2;
    mp.size = gran;
    mp.handleTypes = memHandleType();
    size_t mg = 0;
    if (cu->cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) == CUDA_SUCCESS && mg > gran) gran = mg;
  }
  return gran;
}

ncclResult_t memAlloc(void** ptr, size_t size, int dev) {
  if (!ptr) return ncclInvalidArgument;
  *ptr = nullptr;
  if (size == 0) return ncclSuccess;
  if (dev < 0) CUDACHECK(cudaGetDevice(&dev));
  MemAlloc m;
  m.dev = dev;
  m.requested = size;
  const CuApi* cu = cuApi();
  if (cu && cuMemSupported(dev)) {
    CUDACHECK(cudaFree(0));  // make sure the primary context exists and is current
    size_t gran = shareableGranularity(dev);
    m.size = alignUp(size, gran);
    CUmemAllocationProp prop = {};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = dev;
    prop.requestedHandleTypes = memHandleType();
    int rdma = 0;
    CUdevice cudev;
    if (cu->cuDeviceGet(&cudev, dev) == CUDA_SUCCESS)
      cu->cuDeviceGetAttribute(&rdma, CU_DEVICE_ATTRIBUTE_GPU_DIRECT_RDMA_WITH_CUDA_VMM_SUPPORTED, cudev);
    if (rdma) prop.allocFlags.gpuDirectRDMACapable = 1;
    CUCHECK(cu->cuMemCreate(&m.handle, m.size, &prop, 0));
    m.handleType = (int)prop.requestedHandleTypes;
    CUdeviceptr va = 0;
    CUresult r = cu->cuMemAddressReserve(&va, m.size, gran, 0, 0);
    if (r != CUDA_SUCCESS) { cu->cuMemRelease(m.handle); WARN("cuMemAddressReserve: %s", cuErrStr(r)); return ncclUnhandledCudaError; }
    r = cu->cuMemMap(va, m.size, 0, m.handle, 0);
    if (r != CUDA_SUCCESS) { cu->cuMemAddressFree(va, m.size); cu->cuMemRelease(m.handle); WARN("cuMemMap: %s", cuErrStr(r)); return ncclUnhandledCudaError; }
    // read-write for the owner and for every device that can reach it peer-to-peer, so that several
    // ranks in one process (ncclCommInitAll) can use the same pointer
    int ndev = 0;
    cudaGetDeviceCount(&ndev);
    std::vector<CUmemAccessDesc> acc;
    for (int d = 0; d < ndev; ++d) {
      int can = d == dev;
      if (!can) { if (cudaDeviceCanAccessPeer(&can, d, dev) != cudaSuccess) { can = 0; (void)cudaGetLastError(); } }
      if (!can) continue;
      CUmemAccessDesc ad = {};
      ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      ad.location.id = d;
      ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      acc.push_back(ad);
    }
    r = cu->cuMemSetAccess(va, m.size, acc.data(), acc.size());
    if (r != CUDA_SUCCESS) {
      cu->cuMemUnmap(va, m.size); cu->cuMemAddressFree(va, m.size); cu->cuMemRelease(m.handle);
      WARN("cuMemSetAccess: %s", cuErrStr(r));
      return ncclUnhandledCudaError;
    }
    m.ptr = (void*)va;
    m.vmm = true;
  } else {
    int cur;
    CUDACHECK(cudaGetDevice(&cur));
    if (cur != dev) CUDACHECK(cudaSetDevice(dev));
    cudaError_t e = cudaMalloc(&m.ptr, size);
    if (cur != dev) cudaSetDevice(cur);
    if (e != cudaSuccess) { (void)cudaGetLastError(); WARN("cudaMalloc(%zu) failed: %s", size, cudaGetErrorString(e)); return ncclUnhandledCudaError; }
    m.size = size;
  }
  {
    std::lock_guard<std::mutex> g(gLock);
    gAllocs[(uintptr_t)m.ptr] = m;
    gTotal += m.size;
  }
  INFO(SUB_ALLOC, "memAlloc %zu bytes (mapped %zu) at %p dev %d %s", size, m.size, m.ptr, dev, m.vmm ? "vmm" : "cudaMalloc");
  *ptr = m.ptr;
  return ncclSuccess;
}

ncclResult_t memFree(void* ptr) {
  if (!ptr) return ncclSuccess;
  MemAlloc m;
  {
    std::lock_guard<std::mutex> g(gLock);
    auto it = gAllocs.find((uintptr_t)ptr);
    if (it == gAllocs.end()) { WARN("ncclMemFree: %p was not allocated by ncclMemAlloc", ptr); return ncclInvalidArgument; }
    m = it->second;
    gAllocs.erase(it);
    if (!m.detached) gTotal -= m.size;
  }
  if (m.vmm) {
    const CuApi* cu = cuApi();
    if (!m.detached) {
      CUCHECK(cu->cuMemUnmap((CUdeviceptr)m.ptr, m.size));
      CUCHECK(cu->cuMemRelease(m.handle));
    }
    CUCHECK(cu->cuMemAddressFree((CUdeviceptr)m.ptr, m.size));
  } else {
    CUDACHECK(cudaFree(m.ptr));
  }
  return ncclSuccess;
}

static ncclResult_t mapPhysical(MemAlloc& m) {
  const CuApi* cu = cuApi();
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = m.dev;
  prop.requestedHandleTypes = memHandleType();
  int rdma = 0;
  CUdevice cudev;
  if (cu->cuDeviceGet(&cudev, m.dev) == CUDA_SUCCESS)
    cu->cuDeviceGetAttribute(&rdma, CU_DEVICE_ATTRIBUTE_GPU_DIRECT_RDMA_WITH_CUDA_VMM_SUPPORTED, cudev);
  if (rdma) prop.allocFlags.gpuDirectRDMACapable = 1;
  CUCHECK(cu->cuMemCreate(&m.handle, m.size, &prop, 0));
    m.handleType = (int)prop.requestedHandleTypes;
  CUresult r = cu->cuMemMap((CUdeviceptr)m.ptr, m.size, 0, m.handle, 0);
  if (r != CUDA_SUCCESS) { cu->cuMemRelease(m.handle); WARN("cuMemMap (re-attach): %s", cuErrStr(r)); return ncclUnhandledCudaError; }
  int ndev = 0;
  cudaGetDeviceCount(&ndev);
  std::vector<CUmemAccessDesc> acc;
  for (int d = 0; d < ndev; ++d) {
    int can = d == m.dev;
    if (!can) { if (cudaDeviceCanAccessPeer(&can, d, m.dev) != cudaSuccess) { can = 0; (void)cudaGetLastError(); } }
    if (!can) continue;
    CUmemAccessDesc ad = {};
    ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    ad.location.id = d;
    ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    acc.push_back(ad);
  }
  r = cu->cuMemSetAccess((CUdeviceptr)m.ptr, m.size, acc.data(), acc.size());
  if (r != CUDA_SUCCESS) { cu->cuMemUnmap((CUdeviceptr)m.ptr, m.size); cu->cuMemRelease(m.handle); WARN("cuMemSetAccess (re-attach): %s", cuErrStr(r)); return ncclUnhandledCudaError; }
  return ncclSuccess;
}

ncclResult_t memDetachPhysical(void* ptr) {
  std::lock_guard<std::mutex> g(gLock);
  auto it = gAllocs.find((uintptr_t)ptr);
  if (it == gAllocs.end()) return ncclInvalidArgument;
  MemAlloc& m = it->second;
  if (!m.vmm) return ncclInvalidUsage;
  if (m.detached) return ncclSuccess;
  const CuApi* cu = cuApi();
  CUCHECK(cu->cuMemUnmap((CUdeviceptr)m.ptr, m.size));
  CUCHECK(cu->cuMemRelease(m.handle));
  m.handle = 0;
  m.detached = true;
  gTotal -= m.size;
  return ncclSuccess;
}

ncclResult_t memAttachPhysical(void* ptr) {
  std::lock_guard<std::mutex> g(gLock);
  auto it = gAllocs.find((uintptr_t)ptr);
  if (it == gAllocs.end()) return ncclInvalidArgument;
  MemAlloc& m = it->second;
  if (!m.vmm) return ncclInvalidUsage;
  if (!m.detached) return ncclSuccess;
  NCCLCHECK(mapPhysical(m));
  m.detached = false;
  gTotal += m.size;
  return ncclSuccess;
}

bool memLookup(const void* ptr, MemAlloc* out) {
  std::lock_guard<std::mutex> g(gLock);
  auto it = gAllocs.upper_bound((uintptr_t)ptr);
  if (it == gAllocs.begin()) return false;
  --it;
  if ((uintptr_t)ptr >= it->first + it->second.size) return false;
  if (out) *out = it->second;
  return true;
}

uint64_t memTotalBytes() {
  std::lock_guard<std::mutex> g(gLock);
  return gTotal;
}

}  // namespace b200

extern "C" {
ncclResult_t ncclMemAlloc(void** ptr, size_t size) { return b200::memAlloc(ptr, size); }
ncclResult_t ncclMemFree(void* ptr) { return b200::memFree(ptr); }
ncclResult_t pncclMemAlloc(void** ptr, size_t size) { return ncclMemAlloc(ptr, size); }
ncclResult_t pncclMemFree(void* ptr) { return ncclMemFree(ptr); }
}
