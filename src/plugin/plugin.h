// Plugin loading and the glue between the core and each plugin kind.
// Reference parity: src/plugin/plugin_open.cc (library names and search), src/plugin/net.cc,
// tuner.cc, profiler.cc, env.cc.
#pragma once
#include <string>

#include "../comm/comm.h"
#include "plugin/nccl_env.h"
#include "plugin/nccl_net.h"
#include "plugin/nccl_profiler.h"
#include "plugin/nccl_tuner.h"

namespace b200 {

enum PluginKind { PLUGIN_NET = 0, PLUGIN_TUNER = 1, PLUGIN_PROFILER = 2, PLUGIN_ENV = 3, PLUGIN_KINDS = 4 };

// dlopen()s the library chosen by the kind's environment variable (NCCL_NET_PLUGIN,
// NCCL_TUNER_PLUGIN, NCCL_PROFILER_PLUGIN, NCCL_ENV_PLUGIN):
//   unset        -> "libnccl-<kind>.so" if the dynamic loader finds it, else no plugin
//   "none"       -> no plugin
//   has '/' or ".so" -> that file
//   NAME         -> "libnccl-<kind>-NAME.so"
// Returns nullptr when there is nothing to load. `resolved` receives the name that was opened.
void* pluginOpen(PluginKind kind, std::string* resolved);
void* pluginSymbol(void* lib, const char* name);
const char* pluginKindName(PluginKind kind);

void pluginLogger(ncclDebugLogLevel level, unsigned long flags, const char* file, int line, const char* fmt, ...);

// ---- net plugin of an earlier interface (v11 ... v8): adapter with the current signature, or null (net_compat.cc)
ncclNet_t* netCompatWrap(void* lib, int* version);

// ---- table for GPU-initiated networking found in the network plugin library (net.cc): what it reported
struct GinPluginInfo {
  bool present = false;
  std::string name;
  int devices = 0;
  bool strongSignals = false, vaSignals = false;
};
const GinPluginInfo* netGinPluginInfo();

// ---- env plugin: consulted by every parameter read (core/param.cc)
void envPluginInit();                       // idempotent; called before the first parameter is read
const char* envPluginGet(const char* name); // value from the plugin, or from getenv() when none is loaded
void envPluginFinalize();

// ---- tuner plugin: per communicator
struct TunerState {
  void* lib = nullptr;
  ncclTuner_v6_t* v6 = nullptr;
  ncclTuner_v5_t* v5 = nullptr;
  ncclTuner_v4_t* v4 = nullptr;   // older interfaces: same roles, fewer arguments
  ncclTuner_v3_t* v3 = nullptr;
  ncclTuner_v2_t* v2 = nullptr;
  int version = 0;
  void* ctx = nullptr;
  std::string name;
};
ncclResult_t tunerLoad(ncclComm* comm);     // no-op when no tuner plugin is configured
void tunerUnload(ncclComm* comm);
// Lets the plugin choose for one collective. Returns true and fills algo (comm.h Algo) / ctas when
// the plugin expressed a choice that this data plane can run.
bool tunerPick(ncclComm* comm, int func, size_t bytes, int numPipeOps, bool registered, int* algo, int* ctas);

// ---- profiler plugin: per communicator
struct ProfilerState {
  void* lib = nullptr;
  ncclProfiler_v6_t* prof = nullptr;
  void* ctx = nullptr;
  int mask = 0;
  std::string name;
  uint64_t seq[FUNC_COUNT] = {};
};
ncclResult_t profilerLoad(ncclComm* comm);
void profilerUnload(ncclComm* comm);
void* profStart(ncclComm* comm, ncclProfilerEventDescr_t* d);   // nullptr when the type is not enabled
void profStop(ncclComm* comm, void* handle);
// What the proxy hands to a network backend as the profiler handle of a send / receive (`phandle`): the backend passes it back
// through the callback below when it starts an event of its own, which then hangs under `parent`.
struct ProfNetParent { ncclComm* comm; void* parent; };
// The ncclProfilerCallback_t given to network backends at init (start / stop / update of ncclProfileNetPlugin events).
ncclResult_t profilerNetCallback(void** eHandle, int type, void* pHandle, int64_t pluginId, void* extData);
void profState(ncclComm* comm, void* handle, ncclProfilerEventState_t st, ncclProfilerEventStateArgs_t* a);
// Task events of the data plane (profiler_plugin.cc).
void* profilerTaskStart(ncclComm* comm, const Task& t);
void profilerTaskStop(ncclComm* comm, const Task& t, void* handle, const char* algo, const char* proto, int nCtas);
void profilerPoll(ncclComm* comm, bool drain);

}  // namespace b200
