// Core host-side facilities shared by every layer: result propagation macros,
// logging, parameters, small utilities.
// Reference parity: src/include/checks.h, src/include/debug.h, src/include/param.h,
// src/include/utils.h, src/include/bitops.h (behaviour, not code).
#pragma once
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <string>
#include <vector>

#include "nccl.h"

namespace b200 {

// ---------------------------------------------------------------- logging
enum LogLevel { LOG_NONE = 0, LOG_VERSION = 1, LOG_WARN = 2, LOG_INFO = 3, LOG_ABORT = 4, LOG_TRACE = 5 };
// Sub-system bits, same names and order as NCCL_DEBUG_SUBSYS (reference: src/include/nccl_common.h).
enum LogSubsys : uint64_t {
  SUB_INIT = 1, SUB_COLL = 2, SUB_P2P = 4, SUB_SHM = 8, SUB_NET = 16, SUB_GRAPH = 32, SUB_TUNING = 64,
  SUB_ENV = 128, SUB_ALLOC = 256, SUB_CALL = 512, SUB_PROXY = 1024, SUB_NVLS = 2048, SUB_BOOTSTRAP = 4096,
  SUB_REG = 8192, SUB_PROFILE = 16384, SUB_RAS = 32768, SUB_ALL = ~0ull
};
void debugLog(LogLevel level, uint64_t subsys, const char* file, int line, const char* fmt, ...)
    __attribute__((format(printf, 5, 6)));
int debugLevel();
const char* lastErrorString();       // thread-independent last WARN text (ncclGetLastError)
void setThreadName(const char* fmt, ...);
// NVTX range around a public call (core/nvtx.cc); a no-op unless a profiling tool is attached.
void nvtxRangeBegin(const char* func, size_t bytes, uint64_t commHash, int rank);
void nvtxRangeEnd();

#define WARN(...) ::b200::debugLog(::b200::LOG_WARN, ::b200::SUB_ALL, __FILE__, __LINE__, __VA_ARGS__)
#define INFO(sub, ...) ::b200::debugLog(::b200::LOG_INFO, (sub), __FILE__, __LINE__, __VA_ARGS__)
#define TRACE(sub, ...) ::b200::debugLog(::b200::LOG_TRACE, (sub), __FILE__, __LINE__, __VA_ARGS__)

// ---------------------------------------------------------------- checks
#define NCCLCHECK(call)                                                         \
  do {                                                                          \
    ncclResult_t _r = (call);                                                   \
    if (_r != ncclSuccess && _r != ncclInProgress) {                            \
      INFO(::b200::SUB_ALL, "%s:%d -> %d", __FILE__, __LINE__, (int)_r);        \
      return _r;                                                                \
    }                                                                           \
  } while (0)
#define NCCLCHECKGOTO(call, res, label)                                         \
  do {                                                                          \
    (res) = (call);                                                             \
    if ((res) != ncclSuccess && (res) != ncclInProgress) {                      \
      INFO(::b200::SUB_ALL, "%s:%d -> %d", __FILE__, __LINE__, (int)(res));     \
      goto label;                                                               \
    }                                                                           \
  } while (0)
#define CUDACHECK(call)                                                         \
  do {                                                                          \
    cudaError_t _e = (call);                                                    \
    if (_e != cudaSuccess) {                                                    \
      WARN("CUDA failure '%s' at %s:%d", cudaGetErrorString(_e), __FILE__, __LINE__); \
      (void)cudaGetLastError();                                                 \
      return ncclUnhandledCudaError;                                            \
    }                                                                           \
  } while (0)
#define CUDACHECKGOTO(call, res, label)                                         \
  do {                                                                          \
    cudaError_t _e = (call);                                                    \
    if (_e != cudaSuccess) {                                                    \
      WARN("CUDA failure '%s' at %s:%d", cudaGetErrorString(_e), __FILE__, __LINE__); \
      (void)cudaGetLastError();                                                 \
      (res) = ncclUnhandledCudaError;                                           \
      goto label;                                                               \
    }                                                                           \
  } while (0)
#define SYSCHECK(call, name)                                                    \
  do {                                                                          \
    long _rc;                                                                   \
    do { _rc = (long)(call); } while (_rc == -1 && errno == EINTR);             \
    if (_rc == -1) {                                                            \
      WARN("Call to " name " failed: %s", strerror(errno));                     \
      return ncclSystemError;                                                   \
    }                                                                           \
  } while (0)

// ---------------------------------------------------------------- parameters
// Cached integer parameter read from NCCL_<NAME> (env, conf files, env plugin).
// Reference parity: NCCL_PARAM in src/include/param.h:21-31, files in src/misc/param.cc:27-108.
int64_t paramInt(const char* name /* without NCCL_ */, int64_t deflt, int64_t* cache);
const char* getEnv(const char* fullName);  // goes through conf files + env plugin
void setEnvProvider(const char* (*fn)(const char*));
void loadConfFiles();

enum ParamType { PT_I64, PT_U64, PT_STR, PT_BOOL };
struct ParamDef {
  const char* key;     // full env name, "NCCL_DEBUG"
  ParamType type;
  const char* deflt;   // textual default
  const char* doc;
  bool documented;     // listed in the user guide (dumped without NCCL_PARAM_DUMP_ALL)
};
void registerParam(const ParamDef& d);
const std::vector<ParamDef>& paramRegistry();
struct ParamRegistrar { ParamRegistrar(const ParamDef& d) { registerParam(d); } };

// B200_PARAM(Name, "ENV_SUFFIX", default, "doc") defines  int64_t param##Name().
#define B200_PARAM(Name, env, deflt, doc)                                                   \
  static const std::string _pdef_##Name = std::to_string((long long)(deflt));                \
  static ::b200::ParamRegistrar _preg_##Name(                                               \
      {"NCCL_" env, ::b200::PT_I64, _pdef_##Name.c_str(), doc, true});                      \
  int64_t param##Name() {                                                                   \
    static int64_t cache = INT64_MIN;                                                       \
    return ::b200::paramInt(env, (deflt), &cache);                                          \
  }

// ---------------------------------------------------------------- utils
uint64_t hostHash();                 // hash of hostname + boot id, overridable by NCCL_HOSTID
uint64_t pidHash();
uint64_t hashBytes(const void* p, size_t n, uint64_t seed = 0xcbf29ce484222325ull);
inline uint64_t hashCombine(uint64_t a, uint64_t b) { return a ^ (b + 0x9e3779b97f4a7c15ull + (a << 6) + (a >> 2)); }
uint64_t nowNs();
uint64_t randomU64();
std::string hostName();
int64_t busIdToInt64(const char* busId);
void int64ToBusId(int64_t id, char* out /* >=16 */);

template <typename T> inline T alignUp(T x, T a) { return (x + a - 1) / a * a; }
template <typename T> inline T divUp(T x, T y) { return (x + y - 1) / y; }
inline int log2i(uint64_t x) { return 63 - __builtin_clzll(x | 1); }
inline uint64_t pow2Up(uint64_t x) { return x <= 1 ? 1 : 1ull << (64 - __builtin_clzll(x - 1)); }

size_t typeSize(ncclDataType_t t);
const char* typeName(ncclDataType_t t);
const char* opName(int op);

}  // namespace b200
