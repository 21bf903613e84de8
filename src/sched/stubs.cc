#include "../comm/device_plane.h"
namespace b200 {
ncclResult_t ringTreeRun(ncclComm*, const Task&, int) { WARN("ring/tree kernels are not built yet"); return ncclInvalidUsage; }
ncclResult_t ceCollRun(ncclComm*, const Task&, bool* handled) { *handled = false; return ncclSuccess; }
ncclResult_t signalRun(ncclComm*, const Task&) { WARN("one-sided operations are not built yet"); return ncclInvalidUsage; }
}  // namespace b200
