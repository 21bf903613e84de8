// Environment plugin glue: when NCCL_ENV_PLUGIN names a library exporting ncclEnvPlugin_v2 (or
// _v1), every NCCL_* lookup of the library goes to its getEnv first.
// Reference parity: src/plugin/env.cc:20-117, src/plugin/env/env_v1.cc, env_v2.cc.
#include <mutex>

#include "plugin.h"

namespace b200 {

static std::once_flag gEnvOnce;
static void* gEnvLib = nullptr;
static ncclEnv_v2_t* gEnvV2 = nullptr;
static ncclEnv_v1_t* gEnvV1 = nullptr;

static const char* envFromPlugin(const char* name) {
  if (gEnvV2 && gEnvV2->getEnv) return gEnvV2->getEnv(name);
  if (gEnvV1 && gEnvV1->getEnv) return gEnvV1->getEnv(name);
  return nullptr;
}

void envPluginInit() {
  std::call_once(gEnvOnce, [] {
    const char* want = getenv("NCCL_ENV_PLUGIN");
    if (!want || !*want) return;   // the default source is the process environment: nothing to load
    std::string resolved;
    gEnvLib = pluginOpen(PLUGIN_ENV, &resolved);
    if (!gEnvLib) return;
    gEnvV2 = (ncclEnv_v2_t*)pluginSymbol(gEnvLib, "ncclEnvPlugin_v2");
    if (!gEnvV2) gEnvV1 = (ncclEnv_v1_t*)pluginSymbol(gEnvLib, "ncclEnvPlugin_v1");
    if (!gEnvV2 && !gEnvV1) {
      WARN("env plugin %s exports neither ncclEnvPlugin_v2 nor ncclEnvPlugin_v1", resolved.c_str());
      return;
    }
    ncclResult_t r = gEnvV2 ? gEnvV2->init(NCCL_MAJOR, NCCL_MINOR, NCCL_PATCH, NCCL_SUFFIX, pluginLogger)
                            : gEnvV1->init(NCCL_MAJOR, NCCL_MINOR, NCCL_PATCH, NCCL_SUFFIX);
    if (r != ncclSuccess) {
      WARN("env plugin %s failed to initialise (%d); using the process environment", resolved.c_str(), (int)r);
      gEnvV2 = nullptr;
      gEnvV1 = nullptr;
      return;
    }
    setEnvProvider(envFromPlugin);
    INFO(SUB_ENV, "env plugin %s (%s) is the source of NCCL settings", gEnvV2 ? gEnvV2->name : gEnvV1->name, resolved.c_str());
  });
}

const char* envPluginGet(const char* name) { return getEnv(name); }

void envPluginFinalize() {
  if (gEnvV2 && gEnvV2->finalize) gEnvV2->finalize();
  else if (gEnvV1 && gEnvV1->finalize) gEnvV1->finalize();
  setEnvProvider(nullptr);
  gEnvV2 = nullptr;
  gEnvV1 = nullptr;
}

}  // namespace b200
