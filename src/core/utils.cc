// Small host utilities. Reference parity: src/misc/utils.cc (host hash with NCCL_HOSTID
// override :91-126, pid hash, bus-id conversion), src/include/collectives.h:44 (type sizes).
#include <stdio.h>
#include <time.h>
#include <unistd.h>

#include <random>

#include "core.h"

namespace b200 {

uint64_t hashBytes(const void* p, size_t n, uint64_t h) {
  const unsigned char* c = (const unsigned char*)p;
  for (size_t i = 0; i < n; ++i) { h ^= c[i]; h *= 0x100000001b3ull; }
  return h;
}

std::string hostName() {
  char buf[256] = {0};
  gethostname(buf, sizeof(buf) - 1);
  return buf;
}

uint64_t hostHash() {
  static uint64_t cached = 0;
  static bool done = false;
  if (done) return cached;
  std::string id;
  const char* forced = getEnv("NCCL_HOSTID");
  if (forced) {
    id = forced;
  } else {
    id = hostName();
    FILE* f = fopen("/proc/sys/kernel/random/boot_id", "r");
    if (f) {
      char b[128] = {0};
      if (fgets(b, sizeof(b), f)) id += b;
      fclose(f);
    }
  }
  cached = hashBytes(id.data(), id.size());
  done = true;
  return cached;
}

uint64_t pidHash() {
  char buf[256];
  // pid + pid namespace link, so that two containers with pid 1 differ.
  int n = snprintf(buf, sizeof(buf), "%ld", (long)getpid());
  ssize_t l = readlink("/proc/self/ns/pid", buf + n, sizeof(buf) - n - 1);
  if (l > 0) n += (int)l;
  return hashBytes(buf, n);
}

uint64_t nowNs() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + ts.tv_nsec;
}

uint64_t randomU64() {
  static thread_local std::mt19937_64 gen(std::random_device{}() ^ nowNs() ^ ((uint64_t)getpid() << 32));
  return gen();
}

int64_t busIdToInt64(const char* busId) {
  // "0000:1b:00.0" -> 0x00001b000 (hex digits only)
  int64_t v = 0;
  for (const char* p = busId; *p; ++p) {
    char c = *p;
    int d;
    if (c >= '0' && c <= '9') d = c - '0';
    else if (c >= 'a' && c <= 'f') d = c - 'a' + 10;
    else if (c >= 'A' && c <= 'F') d = c - 'A' + 10;
    else if (c == ':' || c == '.') continue;
    else break;
    v = (v << 4) | d;
  }
  return v;
}

void int64ToBusId(int64_t id, char* out) {
  snprintf(out, 16, "%04lx:%02lx:%02lx.%01lx", (long)((id >> 20) & 0xffff), (long)((id >> 12) & 0xff),
           (long)((id >> 4) & 0xff), (long)(id & 0xf));
}

size_t typeSize(ncclDataType_t t) {
  switch (t) {
    case ncclInt8: case ncclUint8: case ncclFloat8e4m3: case ncclFloat8e5m2: return 1;
    case ncclFloat16: case ncclBfloat16: return 2;
    case ncclInt32: case ncclUint32: case ncclFloat32: return 4;
    case ncclInt64: case ncclUint64: case ncclFloat64: return 8;
    default: return 0;
  }
}

const char* typeName(ncclDataType_t t) {
  static const char* n[] = {"int8", "uint8", "int32", "uint32", "int64", "uint64", "fp16", "fp32", "fp64",
                            "bf16", "fp8e4m3", "fp8e5m2"};
  return (int)t >= 0 && (int)t < ncclNumTypes ? n[t] : "unknown";
}

const char* opName(int op) {
  static const char* n[] = {"sum", "prod", "max", "min", "avg"};
  return op >= 0 && op < ncclNumOps ? n[op] : "premulsum";
}

}  // namespace b200
