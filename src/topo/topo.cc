#include "topo.h"
namespace b200 {
ncclResult_t topoInit(ncclComm*) { return ncclSuccess; }
void topoDestroy(ncclComm*) {}
}  // namespace b200
