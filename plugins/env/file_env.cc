// Example environment plugin: NCCL settings come from a KEY=VALUE file (NCCL_ENV_PLUGIN_FILE)
// and fall back to the process environment for names the file does not define.
// Reference parity: plugins/env/example/plugin.c.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <string>

#include "plugin/nccl_env.h"

namespace {
std::map<std::string, std::string> gVars;

ncclResult_t eInit(uint8_t, uint8_t, uint8_t, const char*, ncclDebugLogger_t log) {
  const char* path = getenv("NCCL_ENV_PLUGIN_FILE");
  if (!path) return ncclSuccess;
  FILE* f = fopen(path, "r");
  if (!f) return ncclSuccess;
  char line[1024];
  while (fgets(line, sizeof(line), f)) {
    if (line[0] == '#') continue;
    char* eq = strchr(line, '=');
    if (!eq) continue;
    *eq = 0;
    char* v = eq + 1;
    v[strcspn(v, "\r\n")] = 0;
    gVars[line] = v;
  }
  fclose(f);
  if (log) log(NCCL_LOG_INFO, NCCL_ENV, __FILE__, __LINE__, "file env plugin: %zu setting(s) from %s", gVars.size(), path);
  return ncclSuccess;
}
ncclResult_t eFinalize(void) { gVars.clear(); return ncclSuccess; }
const char* eGetEnv(const char* name) {
  auto it = gVars.find(name);
  return it != gVars.end() ? it->second.c_str() : getenv(name);
}
}  // namespace

extern "C" __attribute__((visibility("default"))) const ncclEnv_v2_t ncclEnvPlugin_v2 = {"file", eInit, eFinalize, eGetEnv};
