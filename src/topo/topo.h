// Topology detection, path computation, channel-graph search and the analytic tuning model.
// Reference parity: src/graph/{xml,topo,paths,search,connect,rings,trees,tuning}.cc.
#pragma once
#include "../comm/comm.h"

namespace b200 {
ncclResult_t topoInit(ncclComm* comm);
void topoDestroy(ncclComm* comm);
}  // namespace b200
