// Compiled (not run) by tests/test_device_api_compile.py: the utility helpers of the device API, plus a
// host-side check of the reciprocal arithmetic used by ncclFastDiv32 (same formula, plain C++).
#include "nccl_device.h"
#include "nccl_device/utility.h"

__global__ void utilityKernel(uint32_t* out, uint32_t n, uint32_t d, const char* base) {
  using namespace nccl_device;
  ncclFastDiv32 f = ncclFastDiv32::make(d);
  uint32_t q, r;
  f.divmod(n, &q, &r);
  out[0] = q;
  out[1] = r;
  out[2] = rollingLessEq(q, r) ? rollingMax(q, r) : rollingMin(q, r);
  out[3] = ncclLaneId() + (ncclLaneMaskLt() & 1u);
  out[4] = ncclIsAligned(ncclPtrAddBytes(base, 16), 16) ? (uint32_t)ncclDivUp(n, 7) : (uint32_t)ncclAlignUp(n, 8);
  out[5] = (uint32_t)ncclGlobalTimerNs();
}

// The correction step makes q exact: floor(2^32 / d) * x >> 32 is short of x / d by at most one.
static bool reciprocalIsExact() {
  const uint32_t ds[] = {1, 2, 3, 5, 7, 8, 9, 100, 1000, 65535, 65536, 65537, 1u << 31, 0xFFFFFFFFu};
  const uint32_t xs[] = {0, 1, 2, 6, 7, 8, 63, 64, 65, 999, 1000, 1001, 0x7FFFFFFFu, 0x80000000u, 0xFFFFFFFEu, 0xFFFFFFFFu};
  for (uint32_t d : ds)
    for (uint32_t x : xs) {
      uint32_t rcp = d <= 1 ? 0u : (uint32_t)(0x100000000ull / d);
      uint32_t q = d <= 1 ? x : (uint32_t)(((uint64_t)x * rcp) >> 32);
      if (d > 1 && x - q * d >= d) ++q;
      if (q != x / d) return false;
    }
  return true;
}
int main() { return reciprocalIsExact() ? 0 : 1; }
