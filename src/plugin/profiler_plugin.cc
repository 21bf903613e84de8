// External profiler plugin glue (filled in by plugin loading; no plugin = no events).
#include "profiler.h"

namespace b200 {
__attribute__((weak)) void* profilerPluginStart(ncclComm*, const Task&) { return nullptr; }
__attribute__((weak)) void profilerPluginStop(void*) {}
void profilerCommInit(ncclComm*) {}
void profilerCommFini(ncclComm*) {}
}  // namespace b200
