// Logging: NCCL_DEBUG level, NCCL_DEBUG_SUBSYS mask, NCCL_DEBUG_FILE (%h host, %p pid),
// optional timestamps. Reference parity: src/debug.cc:45-110,197-220 (same env names,
// same "host:pid:tid [dev] NCCL LEVEL msg" line shape).
#include <pthread.h>
#include <time.h>
#include <errno.h>
#include <stdarg.h>
#include <stdio.h>
#include <sys/syscall.h>
#include <sys/time.h>
#include <unistd.h>

#include <mutex>
#include <string>

#include "core.h"

namespace b200 {

static std::once_flag gOnce;
static int gLevel = -1;
static uint64_t gMask = SUB_INIT | SUB_BOOTSTRAP | SUB_ENV;
static FILE* gFile = nullptr;
static char gHost[256];
static int gPid;
// which levels carry a time stamp (bit = LogLevel value), and its strftime format
static uint32_t gTsLevels = 1u << LOG_WARN;
static std::string gTsFormat = "[%F %T] ";
static std::mutex gLock;
static char gLastError[1024] = "";
static thread_local char tName[32] = "";

struct SubName { const char* name; uint64_t bit; };
static const SubName kSubs[] = {
    {"INIT", SUB_INIT}, {"COLL", SUB_COLL}, {"P2P", SUB_P2P}, {"SHM", SUB_SHM}, {"NET", SUB_NET},
    {"GRAPH", SUB_GRAPH}, {"TUNING", SUB_TUNING}, {"ENV", SUB_ENV}, {"ALLOC", SUB_ALLOC}, {"CALL", SUB_CALL},
    {"PROXY", SUB_PROXY}, {"NVLS", SUB_NVLS}, {"BOOTSTRAP", SUB_BOOTSTRAP}, {"REG", SUB_REG},
    {"PROFILE", SUB_PROFILE}, {"RAS", SUB_RAS}, {"ALL", SUB_ALL}};

static void initOnce() {
  const char* lv = getenv("NCCL_DEBUG");
  gLevel = LOG_NONE;
  if (lv) {
    if (!strcasecmp(lv, "VERSION")) gLevel = LOG_VERSION;
    else if (!strcasecmp(lv, "WARN")) gLevel = LOG_WARN;
    else if (!strcasecmp(lv, "INFO")) gLevel = LOG_INFO;
    else if (!strcasecmp(lv, "ABORT")) gLevel = LOG_ABORT;
    else if (!strcasecmp(lv, "TRACE")) gLevel = LOG_TRACE;
  }
  const char* subs = getenv("NCCL_DEBUG_SUBSYS");
  if (subs) {
    bool invert = subs[0] == '^';
    if (invert) subs++;
    uint64_t m = 0;
    std::string s(subs);
    size_t pos = 0;
    while (pos <= s.size()) {
      size_t c = s.find(',', pos);
      std::string tok = s.substr(pos, c == std::string::npos ? std::string::npos : c - pos);
      for (auto& k : kSubs) if (!strcasecmp(tok.c_str(), k.name)) m |= k.bit;
      if (c == std::string::npos) break;
      pos = c + 1;
    }
    gMask = invert ? ~m : m;
  }
  gethostname(gHost, sizeof(gHost) - 1);
  for (char* p = gHost; *p; ++p) if (*p == '.') { *p = 0; break; }
  gPid = getpid();
  gFile = stdout;
  const char* f = getenv("NCCL_DEBUG_FILE");
  if (f && gLevel > LOG_VERSION) {
    std::string out;
    for (const char* p = f; *p; ++p) {
      if (*p == '%' && p[1] == 'h') { out += gHost; ++p; }
      else if (*p == '%' && p[1] == 'p') { out += std::to_string(gPid); ++p; }
      else if (*p == '%' && p[1] == '%') { out += '%'; ++p; }
      else out += *p;
    }
    FILE* fp = fopen(out.c_str(), "w");
    if (fp) { setvbuf(fp, nullptr, _IOLBF, 0); gFile = fp; }
  }
  // NCCL_DEBUG_TIMESTAMP_LEVELS: comma list of VERSION, WARN, INFO, ABORT, TRACE or ALL; ^ inverts; empty = none; default WARN
  gTsLevels = 1u << LOG_WARN;
  if (const char* ts = getenv("NCCL_DEBUG_TIMESTAMP_LEVELS")) {
    const bool invert = *ts == '^';
    uint32_t m = 0;
    std::string list(ts + (invert ? 1 : 0));
    size_t pos = 0;
    while (pos <= list.size()) {
      size_t c = list.find(',', pos);
      std::string w = list.substr(pos, c == std::string::npos ? std::string::npos : c - pos);
      if (!strcasecmp(w.c_str(), "ALL")) m = ~0u;
      else if (!strcasecmp(w.c_str(), "VERSION")) m |= 1u << LOG_VERSION;
      else if (!strcasecmp(w.c_str(), "WARN")) m |= 1u << LOG_WARN;
      else if (!strcasecmp(w.c_str(), "INFO")) m |= 1u << LOG_INFO;
      else if (!strcasecmp(w.c_str(), "TRACE")) m |= 1u << LOG_TRACE;
      else if (!strcasecmp(w.c_str(), "ABORT")) m |= 1u << LOG_ABORT;
      if (c == std::string::npos) break;
      pos = c + 1;
    }
    gTsLevels = invert ? ~m : m;
  }
  // NCCL_DEBUG_TIMESTAMP_FORMAT: a strftime format (local time; TZ changes the zone); %Nf with N = 1..9 prints N digits of
  // the fraction of the second; underscores become spaces; set but empty = no time stamp
  gTsFormat = "[%F %T] ";
  if (const char* tf = getenv("NCCL_DEBUG_TIMESTAMP_FORMAT")) {
    gTsFormat = tf;
    for (char& ch : gTsFormat) if (ch == '_') ch = ' ';
  }
}

// Formats the time stamp of a log line of `level` into out (empty when that level carries none).
static void formatStamp(int level, char* out, size_t len) {
  out[0] = 0;
  if (!(gTsLevels & (1u << level)) || gTsFormat.empty()) return;
  struct timespec ts;
  clock_gettime(CLOCK_REALTIME, &ts);
  // expand %Nf ourselves, hand the rest to strftime
  std::string fmt;
  for (size_t i = 0; i < gTsFormat.size(); ++i) {
    if (gTsFormat[i] == '%' && i + 2 < gTsFormat.size() && gTsFormat[i + 1] >= '1' && gTsFormat[i + 1] <= '9' && gTsFormat[i + 2] == 'f') {
      char frac[16];
      snprintf(frac, sizeof(frac), "%09ld", ts.tv_nsec);
      fmt.append(frac, (size_t)(gTsFormat[i + 1] - '0'));
      i += 2;
    } else if (gTsFormat[i] == '%' && i + 1 < gTsFormat.size() && gTsFormat[i + 1] == '%') {
      fmt += "%%";
      ++i;
    } else {
      fmt += gTsFormat[i];
    }
  }
  struct tm tmv;
  localtime_r(&ts.tv_sec, &tmv);
  if (strftime(out, len, fmt.c_str(), &tmv) == 0) out[0] = 0;
}

int debugLevel() {
  std::call_once(gOnce, initOnce);
  return gLevel;
}

// Reads NCCL_DEBUG, NCCL_DEBUG_SUBSYS, NCCL_DEBUG_FILE and NCCL_DEBUG_TIMESTAMP_LEVELS again.
void debugReload() {
  std::call_once(gOnce, [] {});   // a later first use must not undo this reload
  std::lock_guard<std::mutex> g(gLock);
  if (gFile && gFile != stdout) fclose(gFile);
  gMask = SUB_INIT | SUB_BOOTSTRAP | SUB_ENV;
  initOnce();
}

const char* lastErrorString() { return gLastError; }

void setThreadName(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tName, sizeof(tName), fmt, ap);
  va_end(ap);
  // NCCL_SET_THREAD_NAME=1: the operating system sees the name too (debuggers, top -H); 15 characters at most
  static const bool visible = [] { const char* e = getenv("NCCL_SET_THREAD_NAME"); return e && atoi(e) != 0; }();
  if (visible) {
    char shortName[16];
    snprintf(shortName, sizeof(shortName), "%s", tName);
    pthread_setname_np(pthread_self(), shortName);
  }
}

void debugLog(LogLevel level, uint64_t subsys, const char* file, int line, const char* fmt, ...) {
  std::call_once(gOnce, initOnce);
  if (level != LOG_WARN && (gLevel < (int)level || !(subsys & gMask))) return;   // nothing to format
  char msg[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  if (level == LOG_WARN) {
    std::lock_guard<std::mutex> g(gLock);
    snprintf(gLastError, sizeof(gLastError), "%s", msg);
  }
  if (gLevel < (int)level) return;
  if (level != LOG_WARN && !(subsys & gMask)) return;
  int dev = -1;
  // cudaGetDevice is cheap and never initialises a context; ignore errors on GPU-less hosts.
  if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); dev = -1; }
  long tid = syscall(SYS_gettid);
  char stamp[96];
  formatStamp((int)level, stamp, sizeof(stamp));
  const char* base = strrchr(file, '/');
  base = base ? base + 1 : file;
  std::lock_guard<std::mutex> g(gLock);
  if (level == LOG_WARN)
    fprintf(gFile, "\n%s%s:%d:%ld [%d] %s:%d NCCL WARN %s\n", stamp, gHost, gPid, tid, dev, base, line, msg);
  else if (level == LOG_INFO)
    fprintf(gFile, "%s%s:%d:%ld [%d] NCCL INFO %s\n", stamp, gHost, gPid, tid, dev, msg);
  else
    fprintf(gFile, "%s%s:%d:%ld [%d] %s:%d NCCL TRACE %s\n", stamp, gHost, gPid, tid, dev, base, line, msg);
  fflush(gFile);
}

}  // namespace b200

// Deprecated entry point of the reference's header (src/nccl.h.in:277): reload the logging settings.
extern "C" __attribute__((visibility("default"))) void ncclResetDebugInit() { b200::debugReload(); }
extern "C" __attribute__((visibility("default"))) void pncclResetDebugInit() { b200::debugReload(); }
