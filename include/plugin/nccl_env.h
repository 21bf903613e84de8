/*
 * Environment plugin interface: a library exporting `ncclEnvPlugin_v2` (or `_v1`, whose init has
 * no logger argument) replaces getenv() as the source of every NCCL_* setting.
 * Reference parity: src/include/plugin/nccl_env.h, env/env_v1.h, env/env_v2.h.
 */
#ifndef NCCL_B200_PLUGIN_ENV_H_
#define NCCL_B200_PLUGIN_ENV_H_
#include "nccl_common.h"

typedef struct {
  const char* name;
  ncclResult_t (*init)(uint8_t major, uint8_t minor, uint8_t patch, const char* suffix);
  ncclResult_t (*finalize)(void);
  /* The returned string must stay valid until finalize or the next getEnv of the same name. */
  const char* (*getEnv)(const char* name);
} ncclEnv_v1_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(uint8_t major, uint8_t minor, uint8_t patch, const char* suffix, ncclDebugLogger_t logFunction);
  ncclResult_t (*finalize)(void);
  const char* (*getEnv)(const char* name);
} ncclEnv_v2_t;

typedef ncclEnv_v2_t ncclEnv_t;
#define NCCL_ENV_PLUGIN_SYMBOL "ncclEnvPlugin_v2"

#endif
