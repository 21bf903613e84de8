#include "ras.h"
namespace b200 {
void rasCommAdd(ncclComm*) {}
void rasCommRemove(ncclComm*) {}
}  // namespace b200
