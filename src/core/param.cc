// Parameters: environment variables, configuration files, typed registry and the
// public ncclParam* query API.
// Reference parity: src/misc/param.cc:27-108 (NCCL_CONF_FILE, ~/.nccl.conf, /etc/nccl.conf;
// env wins over files), src/param/*.cc + src/nccl.h.in:757-838 (typed registry API).
#include <errno.h>
#include <pwd.h>
#include <stdio.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <mutex>

#include "core.h"

namespace b200 {

static const char* (*gEnvProvider)(const char*) = nullptr;
void envPluginInit();   // plugin/env.cc
static std::once_flag gConfOnce;
static std::mutex gRegLock;

void setEnvProvider(const char* (*fn)(const char*)) { gEnvProvider = fn; }

static void loadOneConf(const char* path) {
  FILE* f = fopen(path, "r");
  if (!f) return;
  char line[2048];
  while (fgets(line, sizeof(line), f)) {
    char* p = line;
    while (*p == ' ' || *p == '\t') ++p;
    if (*p == '#' || *p == '\n' || *p == 0) continue;
    char* eq = strchr(p, '=');
    if (!eq) continue;
    *eq = 0;
    char* key = p;
    char* val = eq + 1;
    for (char* e = key + strlen(key) - 1; e >= key && (*e == ' ' || *e == '\t'); --e) *e = 0;
    while (*val == ' ' || *val == '\t') ++val;
    for (char* e = val + strlen(val) - 1; e >= val && (*e == '\n' || *e == '\r' || *e == ' '); --e) *e = 0;
    if (*key) setenv(key, val, 0);  // never overrides the real environment
  }
  fclose(f);
}

void loadConfFiles() {
  std::call_once(gConfOnce, [] {
    const char* explicitFile = getenv("NCCL_CONF_FILE");
    if (explicitFile) loadOneConf(explicitFile);
    const char* home = getenv("HOME");
    if (!home) {
      struct passwd* pw = getpwuid(getuid());
      if (pw) home = pw->pw_dir;
    }
    if (home) loadOneConf((std::string(home) + "/.nccl.conf").c_str());
    loadOneConf("/etc/nccl.conf");
  });
}

const char* getEnv(const char* name) {
  loadConfFiles();
  envPluginInit();
  if (gEnvProvider) {
    const char* v = gEnvProvider(name);
    if (v) return v;
  }
  return getenv(name);
}

int64_t paramInt(const char* name, int64_t deflt, int64_t* cache) {
  int64_t v = __atomic_load_n(cache, __ATOMIC_RELAXED);
  if (v != INT64_MIN) return v;
  std::string full = std::string("NCCL_") + name;
  const char* s = getEnv(full.c_str());
  v = deflt;
  if (s && *s) {
    errno = 0;
    char* end = nullptr;
    long long parsed = strtoll(s, &end, 0);
    if (errno || end == s) {
      INFO(SUB_ENV, "Invalid value %s for %s, using default %lld", s, full.c_str(), (long long)deflt);
    } else {
      v = parsed;
      INFO(SUB_ENV, "%s set by environment to %lld.", full.c_str(), (long long)v);
    }
  }
  __atomic_store_n(cache, v, __ATOMIC_RELAXED);
  return v;
}

static std::vector<ParamDef>& registryMut() {
  static std::vector<ParamDef> r;
  return r;
}
const std::vector<ParamDef>& paramRegistry() { return registryMut(); }
void registerParam(const ParamDef& d) {
  std::lock_guard<std::mutex> g(gRegLock);
  for (auto& e : registryMut()) if (!strcmp(e.key, d.key)) return;
  registryMut().push_back(d);
}

// String-valued and boolean parameters that have no B200_PARAM accessor.
static ParamRegistrar kStrParams[] = {
    {{"NCCL_DEBUG", PT_STR, "", "Log level: VERSION, WARN, INFO, TRACE", true}},
    {{"NCCL_DEBUG_SUBSYS", PT_STR, "INIT,BOOTSTRAP,ENV", "Comma list of subsystems to log; ^ inverts", true}},
    {{"NCCL_DEBUG_FILE", PT_STR, "", "Log file; %h = host, %p = pid", true}},
    {{"NCCL_CONF_FILE", PT_STR, "", "Extra configuration file read before ~/.nccl.conf", true}},
    {{"NCCL_SOCKET_IFNAME", PT_STR, "", "Interface name filter for bootstrap sockets (^ excludes, = exact)", true}},
    {{"NCCL_COMM_ID", PT_STR, "", "ip:port of the bootstrap root instead of a broadcast unique id", true}},
    {{"NCCL_HOSTID", PT_STR, "", "String hashed into the host identity instead of hostname+boot id", true}},
    {{"NCCL_ALGO", PT_STR, "", "Force one algorithm: Ring, Tree, NVLS, OneShot (LL), TwoShot (P2P, Direct), CE on GPU communicators; PAT or Ring on host-memory communicators", true}},
    {{"NCCL_PROTO", PT_STR, "", "Restrict protocols: LL,Simple (^ excludes)", true}},
    {{"NCCL_TOPO_FILE", PT_STR, "", "XML topology to load instead of probing the machine", true}},
    {{"NCCL_TOPO_DUMP_FILE", PT_STR, "", "Write the detected topology XML here", true}},
    {{"NCCL_GRAPH_FILE", PT_STR, "", "XML of precomputed channel graphs to load", true}},
    {{"NCCL_GRAPH_DUMP_FILE", PT_STR, "", "Write the computed channel graphs here", true}},
    {{"NCCL_TUNER_PLUGIN", PT_STR, "", "Tuner plugin library name", true}},
    {{"NCCL_NET_PLUGIN", PT_STR, "", "Network plugin library name", true}},
    {{"NCCL_PROFILER_PLUGIN", PT_STR, "", "Profiler plugin library name", true}},
    {{"NCCL_ENV_PLUGIN", PT_STR, "", "Environment plugin library name", true}},
    {{"NCCL_TUNING_FILE", PT_STR, "", "JSON table of measured algorithm crossover sizes", false}},
    {{"NCCL_SYM_KERNEL", PT_STR, "", "Force one symmetric kernel by name", true}},
    {{"NCCL_PROXY_DUMP_SIGNAL", PT_STR, "", "Signal number on which proxy threads log their operations in flight", true}},
    {{"NCCL_NET", PT_STR, "", "Insist on one network backend by name (a plugin's name, or Socket)", true}},
    {{"NCCL_PARAM_DUMP_ALL", PT_BOOL, "0", "Include undocumented parameters in ncclParamDumpAll", true}},
    {{"NCCL_DEBUG_TIMESTAMP_LEVELS", PT_STR, "WARN", "Log levels that carry a time stamp: comma list of VERSION, WARN, INFO, ABORT, TRACE or ALL; ^ inverts; empty = none", true}},
    {{"NCCL_DEBUG_TIMESTAMP_FORMAT", PT_STR, "[%F %T] ", "strftime format of the time stamp (local time); %Nf prints N digits of the fraction of the second; underscores become spaces", true}},
    {{"NCCL_SET_THREAD_NAME", PT_BOOL, "0", "Give the library's threads (proxy, RAS, bootstrap root, init) names the operating system shows", true}},
    {{"NCCL_RAS_ADDR", PT_STR, "localhost:28028", "Address of the RAS client socket (host:port)", true}},
    {{"NCCL_SOCKET_FAMILY", PT_STR, "", "AF_INET or AF_INET6: address family of bootstrap and socket-network interfaces", true}},
    {{"NCCL_P2P_LEVEL", PT_STR, "PHB", "Farthest path class over which GPUs use peer access: LOC, NVL, NVB, PIX, PXB, PXN, PHB, SYS", true}},
    {{"NCCL_CROSS_NIC", PT_STR, "", "Whether a ring may leave through another NIC than it entered by (channel search for jobs that span nodes): 0, 1 or 2", true}},
    {{"NCCL_GIN_TYPE", PT_STR, "", "Backend of the GPU-initiated put / signal surface: NONE (peer stores from the kernel) or PROXY (descriptors served by a host thread)", true}},
    {{"NCCL_PROFILE_EVENT_MASK", PT_STR, "", "Bit mask of the event types handed to the profiler plugin (overrides what the plugin asks for)", true}},
    // variables of the reference that configure parts this build does not have: accepted and ignored, listed so that a job
    // script written for the reference explains itself
    {{"NCCL_IBVERBS_LIB", PT_STR, "", "The reference's name of NCCL_B200_IBV_LIB (used when that is not set)", true}},
    {{"NCCL_PROXY_CPUSET", PT_STR, "", "CPUs of the proxy threads, in the form of the kernel's cpulist files (0-7,16-23); default: the CPUs next to the rank's GPU", true}},
    {{"NCCL_TOPO_DUMP_FILE_RANK", PT_STR, "", "Rank that writes NCCL_TOPO_DUMP_FILE (default: local rank 0 of every host)", true}},
    {{"NCCL_GRAPH_DUMP_FILE_RANK", PT_STR, "", "Rank that writes NCCL_GRAPH_DUMP_FILE (default 0)", true}},
    {{"NCCL_SHM_DISABLE", PT_STR, "", "1: ranks of one host never use shared-memory rings (they are opt-in here: NCCL_B200_HOST_SHM)", true}},
    {{"NCCL_IB_HCA", PT_STR, "", "Verbs devices the InfiniBand backend may use: name prefixes with optional :port, comma separated; =name wants the exact name, a leading ^ excludes", true}},
    {{"NCCL_IB_ADDR_FAMILY", PT_STR, "AF_INET", "Address family preferred when the RoCE GID index is chosen automatically: AF_INET or AF_INET6", true}},
    {{"NCCL_B200_IBV_LIB", PT_STR, "libibverbs.so.1", "Verbs library that the InfiniBand backend opens at run time", true}},
    {{"NCCL_IB_SPLIT_DATA_ON_QPS", PT_STR, "", "No effect: with several queue pairs per connection every RDMA-write message is split over them; NCCL_IB_AR_THRESHOLD, NCCL_IB_MERGE_NICS and the resiliency settings have no effect either", true}},
    {{"NCCL_NET_GDR_LEVEL", PT_STR, "", "No effect: the proxy stages through host memory on the built-in backends; a plugin decides about GPUDirect itself", true}},
    {{"NCCL_MNNVL_CROSS_CLIQUE", PT_STR, "", "No effect: ranks of other fabric cliques are reached through the network transport only", true}},
    {{"NCCL_GDRCOPY_ENABLE", PT_STR, "", "No effect: no GDRCopy mappings are used (flags and credits live in device or pinned host memory that both sides map); the other NCCL_GDRCOPY_* variables likewise", true}},
    {{"NCCL_LL_BUFFSIZE", PT_STR, "", "No effect: the flagged-line regions have a fixed size in the resource window; NCCL_LL128_BUFFSIZE, NCCL_LL128_NTHREADS and NCCL_LL128_C2C have no counterpart (there is no LL128 protocol)", true}},
    {{"NCCL_P2P_NVL_CHUNKSIZE", PT_STR, "", "No effect: send / receive moves data in mailbox chunks sized by the message (NCCL_P2P_PCI_CHUNKSIZE, NCCL_P2P_NET_CHUNKSIZE, NCCL_CHUNK_SIZE, NCCL_NVLS_CHUNKSIZE likewise)", true}},
    {{"NCCL_WORK_FIFO_BYTES", PT_STR, "", "No effect: every launch carries its arguments in the kernel parameters (no work FIFO; NCCL_WORK_ARGS_BYTES likewise)", true}},
    {{"NCCL_GRAPH_REGISTER", PT_STR, "", "No effect: buffers are registered only by ncclCommRegister / ncclCommWindowRegister (NCCL_LOCAL_REGISTER, NCCL_LEGACY_CUDA_REGISTER likewise)", true}},
    {{"NCCL_SYM_CTAS", PT_STR, "", "No effect: CTA counts come from the selection table, NCCL_MAX_CTAS / NCCL_MIN_CTAS and the communicator's configuration (NCCL_NVLS_NCHANNELS, NCCL_MAX_P2P_NCHANNELS likewise)", true}},
    {{"NCCL_PXN_DISABLE", PT_STR, "", "No effect: the channel search classifies relayed NIC paths, but traffic between NVLink domains is not relayed through peer GPUs (NCCL_P2P_PXN_LEVEL, NCCL_PXN_C2C likewise)", true}},
    {{"NCCL_IB_ADAPTIVE_ROUTING", PT_STR, "", "No effect in the verbs backend; neither have NCCL_IB_ECE_ENABLE, NCCL_IB_SUBNET_AWARE_ROUTING, NCCL_IB_DATA_DIRECT, NCCL_IB_OOO_RQ and the NCCL_IB_RESILIENCY_* family", true}},
    {{"NCCL_GIN_ENABLE", PT_STR, "", "No effect: GPU-initiated put / signal serves the NVLink domain (NCCL_GIN_TYPE chooses peer stores or the host proxy); the NCCL_GIN_GDAKI_* and NCCL_RMA_* variables have no counterpart", true}},
    {{"NCCL_NTHREADS", PT_STR, "", "No effect: the kernels' CTA sizes are fixed per kernel (512 threads, 32 for the bulk-copy forms)", true}},
    {{"NCCL_BUFFSIZE", PT_STR, "", "No effect: there are no per-channel FIFO buffers; NCCL_B200_SCRATCH_MB sizes the staging area for unregistered buffers", true}},
    {{"NCCL_LAUNCH_MODE", PT_STR, "", "No effect: every rank launches its own kernels (one process or thread per GPU)", true}},
    {{"NCCL_RUNTIME_CONNECT", PT_STR, "", "No effect: the symmetric resource window is mapped when the communicator is created", true}},
};

}  // namespace b200

using namespace b200;

struct ncclParamHandle {
  const ParamDef* def;
  std::string value;  // textual current value
};

static std::string currentValue(const ParamDef* d) {
  const char* v = getEnv(d->key);
  return v ? std::string(v) : std::string(d->deflt ? d->deflt : "");
}

template <typename T>
static ncclResult_t getInt(ncclParamHandle_t h, T* out) {
  if (!h || !out) return ncclInvalidArgument;
  if (h->def->type == PT_STR) return ncclInvalidUsage;
  h->value = currentValue(h->def);
  const char* s = h->value.c_str();
  long long v = 0;
  if (h->def->type == PT_BOOL) {
    v = (*s == '1' || *s == 't' || *s == 'T' || *s == 'y' || *s == 'Y') ? 1 : 0;
  } else {
    v = strtoll(s, nullptr, 0);
  }
  if ((long long)(T)v != v) return ncclInvalidArgument;
  *out = (T)v;
  return ncclSuccess;
}

extern "C" {

ncclResult_t ncclParamBind(ncclParamHandle_t* out, const char* key) {
  if (!out || !key) return ncclInvalidArgument;
  for (auto& d : paramRegistry()) {
    if (!strcmp(d.key, key)) {
      *out = new ncclParamHandle{&d, currentValue(&d)};
      return ncclSuccess;
    }
  }
  *out = nullptr;
  return ncclInvalidArgument;
}

ncclResult_t ncclParamGetI8(ncclParamHandle_t h, int8_t* o) { return getInt(h, o); }
ncclResult_t ncclParamGetI16(ncclParamHandle_t h, int16_t* o) { return getInt(h, o); }
ncclResult_t ncclParamGetI32(ncclParamHandle_t h, int32_t* o) { return getInt(h, o); }
ncclResult_t ncclParamGetI64(ncclParamHandle_t h, int64_t* o) { return getInt(h, o); }
ncclResult_t ncclParamGetU8(ncclParamHandle_t h, uint8_t* o) { return getInt(h, o); }
ncclResult_t ncclParamGetU16(ncclParamHandle_t h, uint16_t* o) { return getInt(h, o); }
ncclResult_t ncclParamGetU32(ncclParamHandle_t h, uint32_t* o) { return getInt(h, o); }
ncclResult_t ncclParamGetU64(ncclParamHandle_t h, uint64_t* o) { return getInt(h, o); }

ncclResult_t ncclParamGetStr(ncclParamHandle_t h, const char** out) {
  if (!h || !out) return ncclInvalidArgument;
  h->value = currentValue(h->def);
  *out = h->value.c_str();
  return ncclSuccess;
}

ncclResult_t ncclParamGet(ncclParamHandle_t h, void* out, int maxLen, int* len) {
  if (!h || !out || maxLen <= 0) return ncclInvalidArgument;
  h->value = currentValue(h->def);
  int n = (int)std::min<size_t>(h->value.size(), (size_t)maxLen - 1);
  memcpy(out, h->value.data(), n);
  ((char*)out)[n] = 0;
  if (len) *len = n;
  return ncclSuccess;
}

ncclResult_t ncclParamGetParameter(const char* key, const char** value, int* valueLen) {
  static thread_local std::string tls;
  if (!key || !value) return ncclInvalidArgument;
  for (auto& d : paramRegistry()) {
    if (!strcmp(d.key, key)) {
      tls = currentValue(&d);
      *value = tls.c_str();
      if (valueLen) *valueLen = (int)tls.size();
      return ncclSuccess;
    }
  }
  return ncclInvalidArgument;
}

ncclResult_t ncclParamGetAllParameterKeys(const char*** table, int* tableLen) {
  static std::vector<const char*> keys;
  static std::mutex m;
  if (!table || !tableLen) return ncclInvalidArgument;
  std::lock_guard<std::mutex> g(m);
  keys.clear();
  for (auto& d : paramRegistry()) keys.push_back(d.key);
  std::sort(keys.begin(), keys.end(), [](const char* a, const char* b) { return strcmp(a, b) < 0; });
  *table = keys.data();
  *tableLen = (int)keys.size();
  return ncclSuccess;
}

void ncclParamDumpAll(void) {
  const char* all = getEnv("NCCL_PARAM_DUMP_ALL");
  bool dumpAll = all && (*all == '1' || *all == 't' || *all == 'T');
  const char** keys;
  int n;
  ncclParamGetAllParameterKeys(&keys, &n);
  for (int i = 0; i < n; ++i) {
    for (auto& d : paramRegistry()) {
      if (strcmp(d.key, keys[i])) continue;
      if (!d.documented && !dumpAll) continue;
      const char* env = getEnv(d.key);
      printf("%-40s = %-24s %s  # %s\n", d.key, currentValue(&d).c_str(), env ? "(env)" : "(default)", d.doc);
    }
  }
  fflush(stdout);
}

#define PTWIN(ret, name, params, args) ret p##name params { return name args; }
PTWIN(ncclResult_t, ncclParamBind, (ncclParamHandle_t * o, const char* k), (o, k))
PTWIN(ncclResult_t, ncclParamGetI8, (ncclParamHandle_t h, int8_t* o), (h, o))
PTWIN(ncclResult_t, ncclParamGetI16, (ncclParamHandle_t h, int16_t* o), (h, o))
PTWIN(ncclResult_t, ncclParamGetI32, (ncclParamHandle_t h, int32_t* o), (h, o))
PTWIN(ncclResult_t, ncclParamGetI64, (ncclParamHandle_t h, int64_t* o), (h, o))
PTWIN(ncclResult_t, ncclParamGetU8, (ncclParamHandle_t h, uint8_t* o), (h, o))
PTWIN(ncclResult_t, ncclParamGetU16, (ncclParamHandle_t h, uint16_t* o), (h, o))
PTWIN(ncclResult_t, ncclParamGetU32, (ncclParamHandle_t h, uint32_t* o), (h, o))
PTWIN(ncclResult_t, ncclParamGetU64, (ncclParamHandle_t h, uint64_t* o), (h, o))
PTWIN(ncclResult_t, ncclParamGetStr, (ncclParamHandle_t h, const char** o), (h, o))
PTWIN(ncclResult_t, ncclParamGet, (ncclParamHandle_t h, void* o, int m, int* l), (h, o, m, l))
PTWIN(ncclResult_t, ncclParamGetParameter, (const char* k, const char** v, int* l), (k, v, l))
PTWIN(ncclResult_t, ncclParamGetAllParameterKeys, (const char*** t, int* l), (t, l))
void pncclParamDumpAll(void) { ncclParamDumpAll(); }

}  // extern "C"
