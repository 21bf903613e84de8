// Finds and opens plugin libraries. See plugin.h for the naming rules.
// Reference parity: src/plugin/plugin_open.cc:20-189.
#include <dlfcn.h>
#include <stdarg.h>

#include "plugin.h"

namespace b200 {

static const char* kKindNames[PLUGIN_KINDS] = {"net", "tuner", "profiler", "env"};
static const char* kKindEnv[PLUGIN_KINDS] = {"NCCL_NET_PLUGIN", "NCCL_TUNER_PLUGIN", "NCCL_PROFILER_PLUGIN", "NCCL_ENV_PLUGIN"};

const char* pluginKindName(PluginKind kind) { return kKindNames[kind]; }

void* pluginOpen(PluginKind kind, std::string* resolved) {
  // The env plugin itself cannot come from an env plugin: read the process environment directly.
  const char* v = kind == PLUGIN_ENV ? getenv(kKindEnv[kind]) : envPluginGet(kKindEnv[kind]);
  std::vector<std::string> tries;
  if (v && *v) {
    if (strcasecmp(v, "none") == 0) return nullptr;
    std::string s(v);
    if (s.find('/') != std::string::npos || s.find(".so") != std::string::npos) tries.push_back(s);
    else {
      tries.push_back(std::string("libnccl-") + kKindNames[kind] + "-" + s + ".so");
      tries.push_back(std::string("libnccl-") + kKindNames[kind] + ".so");
    }
  } else {
    tries.push_back(std::string("libnccl-") + kKindNames[kind] + ".so");
  }
  for (auto& t : tries) {
    void* h = dlopen(t.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (h) {
      if (resolved) *resolved = t;
      INFO(SUB_INIT, "%s plugin: loaded %s", kKindNames[kind], t.c_str());
      return h;
    }
    if (v && *v) INFO(SUB_INIT, "%s plugin: could not open %s: %s", kKindNames[kind], t.c_str(), dlerror());
  }
  // A library may carry several plugins: a tuner that was not asked for by name is looked for in the library that
  // NCCL_NET_PLUGIN names (the caller then finds its symbol there or not).
  if (kind == PLUGIN_TUNER && !(v && *v)) {
    const char* net = envPluginGet(kKindEnv[PLUGIN_NET]);
    if (net && *net && strcasecmp(net, "none") != 0) {
      std::string s(net);
      std::vector<std::string> netTries;
      if (s.find('/') != std::string::npos || s.find(".so") != std::string::npos) netTries.push_back(s);
      else { netTries.push_back("libnccl-net-" + s + ".so"); netTries.push_back("libnccl-net.so"); }
      for (auto& t : netTries) {
        void* h = dlopen(t.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (!h) continue;
        if (dlsym(h, "ncclTunerPlugin_v6") || dlsym(h, "ncclTunerPlugin_v5") || dlsym(h, "ncclTunerPlugin_v4") || dlsym(h, "ncclTunerPlugin_v3") ||
            dlsym(h, "ncclTunerPlugin_v2")) {
          if (resolved) *resolved = t;
          INFO(SUB_INIT, "tuner plugin: found in the network plugin's library %s", t.c_str());
          return h;
        }
        dlclose(h);
      }
    }
  }
  if (v && *v) WARN("%s plugin \"%s\" was requested with %s but could not be loaded; using the built-in implementation", kKindNames[kind], v, kKindEnv[kind]);
  return nullptr;
}

void* pluginSymbol(void* lib, const char* name) { return lib ? dlsym(lib, name) : nullptr; }

void pluginLogger(ncclDebugLogLevel level, unsigned long flags, const char* file, int line, const char* fmt, ...) {
  const LogLevel lvl = level == NCCL_LOG_WARN ? LOG_WARN : level == NCCL_LOG_INFO ? LOG_INFO : level == NCCL_LOG_TRACE ? LOG_TRACE : LOG_NONE;
  if (lvl == LOG_NONE || (lvl != LOG_WARN && debugLevel() < (int)lvl)) return;
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  debugLog(lvl, (uint64_t)flags, file, line, "%s", buf);
}

}  // namespace b200
