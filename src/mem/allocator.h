// Device memory allocations that can be shared between ranks and bound to multicast objects.
// Reference parity: ncclMemAlloc/ncclMemFree in src/allocator.cc:17-139.
#pragma once
#include "../core/cudawrap.h"

namespace b200 {

struct MemAlloc {
  void* ptr = nullptr;
  size_t size = 0;        // mapped size (multiple of the granularity)
  size_t requested = 0;
  int dev = -1;
  bool vmm = false;       // created with cuMemCreate (exportable, multicast-bindable)
  CUmemGenericAllocationHandle handle = 0;
  int handleType = 0;     // CUmemAllocationHandleType the physical memory was created with
  bool detached = false;  // the physical memory was given back (memDetachPhysical); the address range is still reserved
};

// Granularity used for every shareable allocation on `dev` (covers allocation and multicast minimums).
size_t shareableGranularity(int dev);
ncclResult_t memAlloc(void** ptr, size_t size, int dev = -1);
ncclResult_t memFree(void* ptr);
// Allocation of this process that contains `ptr` (null when `ptr` was not returned by memAlloc).
bool memLookup(const void* ptr, MemAlloc* out);
uint64_t memTotalBytes();
// Gives the physical memory behind an allocation back to the driver while keeping its address range reserved, and
// maps new physical memory at the same addresses later: pointers handed out earlier stay valid across the pair, the
// contents do not survive. Only for allocations made through the virtual-memory API (ncclInvalidUsage otherwise).
ncclResult_t memDetachPhysical(void* ptr);
ncclResult_t memAttachPhysical(void* ptr);

}  // namespace b200
