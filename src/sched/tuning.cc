// Measured selection table: per collective and rank count, a list of (size limit, algorithm,
// copy mode, CTA count) rows produced by nccl_b200/utils/tune.py on the target machine. The first
// row whose limit covers the message decides the kernel; without rows for a rank count the
// threshold heuristics of the data plane apply.
// Reference parity: the role of src/graph/tuning.cc + src/sym_kernels.cc (cost models) and of the
// tuner plugin; here the table comes from measurement instead of a model.
#include <ctype.h>
#include <stdio.h>

#include "../comm/device_plane.h"
#include "tuning_defaults.h"

namespace b200 {

static int collIndex(const std::string& name) {
  if (name == "all_reduce") return 0;
  if (name == "all_gather") return 1;
  if (name == "reduce_scatter") return 2;
  if (name == "all_to_all") return 3;
  if (name == "broadcast") return 4;
  return -1;
}
int tuneCollOfFunc(int func) {
  switch (func) {
    case FUNC_ALLREDUCE: return 0;
    case FUNC_ALLGATHER: return 1;
    case FUNC_REDUCESCATTER: return 2;
    case FUNC_ALLTOALL: return 3;
    case FUNC_BROADCAST: return 4;
    default: return -1;
  }
}

// Grammar: { "<n>": { "<coll>": [ [upto, "ALGO", ctas], ... ], ... }, ..., "<switch>": number, ... }  with ALGO in
// LL, P2P, NVLS, NVLS1, PUSH, PULL, MC, BPUSH, BPULL, BMC, CE.
struct Cursor {
  const char* p;
  void ws() { while (*p && isspace((unsigned char)*p)) ++p; }
  bool eat(char c) { ws(); if (*p == c) { ++p; return true; } return false; }
  bool str(std::string* out) {
    ws();
    if (*p != '"') return false;
    ++p;
    out->clear();
    while (*p && *p != '"') out->push_back(*p++);
    if (*p != '"') return false;
    ++p;
    return true;
  }
  bool num(long long* v) {
    ws();
    char* end = nullptr;
    *v = strtoll(p, &end, 10);
    if (end == p) return false;
    p = end;
    return true;
  }
};

bool tuneParse(TuningTable* t, const std::string& json) {
  Cursor c{json.c_str()};
  if (!c.eat('{')) return false;
  while (true) {
    std::string nKey;
    if (!c.str(&nKey)) break;
    int n = atoi(nKey.c_str());
    if (!c.eat(':')) return false;
    if (!isdigit((unsigned char)nKey[0])) {
      // global switch: "llMcMin": 8, "barrierMcMin": 4, "ceMin": bytes
      long long v;
      if (!c.num(&v)) return false;
      if (nKey == "llMcMin") t->llMcMin = (int)v;
      else if (nKey == "barrierMcMin") t->barrierMcMin = (int)v;
      else if (nKey == "ceMin") t->ceMin = (size_t)v;
      if (!c.eat(',')) break;
      continue;
    }
    if (!c.eat('{')) return false;
    while (true) {
      std::string coll;
      if (!c.str(&coll)) break;
      int ci = collIndex(coll);
      if (!c.eat(':') || !c.eat('[')) return false;
      std::vector<TuneEntry> rows;
      while (c.eat('[')) {
        long long upto, ctas;
        std::string algo;
        if (!c.num(&upto) || !c.eat(',') || !c.str(&algo) || !c.eat(',') || !c.num(&ctas) || !c.eat(']')) return false;
        TuneEntry e{(size_t)upto, ALGO_P2P, -1, (int)ctas};
        if (algo == "LL") e.algo = ALGO_LL_ONESHOT;
        else if (algo == "NVLS") e.algo = ALGO_NVLS;
        else if (algo == "NVLS1") e.algo = ALGO_NVLS_ONESHOT;
        else if (algo == "MC") { e.algo = ALGO_NVLS; e.mode = MODE_MC; }
        else if (algo == "CE") e.algo = ALGO_CE;                      // copy engines: no SM at all
        else if (algo == "PUSH") e.mode = MODE_PUSH;
        else if (algo == "PULL") e.mode = MODE_PULL;
        else if (algo == "BPUSH") e.mode = MODE_PUSH | MODE_BULK;   // bulk-copy engines instead of threads
        else if (algo == "BPULL") e.mode = MODE_PULL | MODE_BULK;
        else if (algo == "BMC") { e.algo = ALGO_NVLS; e.mode = MODE_MC | MODE_BULK; }
        else if (algo == "SPLIT") e.mode = MODE_SPLIT;               // broadcast: the non-root ranks share the work
        rows.push_back(e);
        c.eat(',');
      }
      if (!c.eat(']')) return false;
      if (ci >= 0 && n >= 0 && n <= kMaxRanks) t->entries[ci][n] = rows;
      if (!c.eat(',')) break;
    }
    if (!c.eat('}')) return false;
    if (!c.eat(',')) break;
  }
  return c.eat('}');
}

void tuneLoadDefaults(TuningTable* t) {
  if (!tuneParse(t, kDefaultTuningJson)) WARN("built-in tuning table does not parse");
}

TunePick tunePick(const TuningTable& t, int func, int n, size_t bytes) {
  TunePick pk{false, ALGO_AUTO, -1, 0};
  int ci = tuneCollOfFunc(func);
  if (ci < 0 || n < 0 || n > kMaxRanks) return pk;
  const std::vector<TuneEntry>& rows = t.entries[ci][n];
  if (rows.empty()) return pk;
  const TuneEntry* e = &rows.back();
  for (auto& r : rows) if (bytes <= r.upto) { e = &r; break; }
  pk.valid = true;
  pk.algo = e->algo;
  pk.mode = e->mode;
  pk.ctas = e->ctas;
  return pk;
}

}  // namespace b200

// Parses a table given as text and looks one choice up: writes "<algo> <mode> <ctas>" (numbers as the data plane uses them)
// into out. Returns 0, 1 when the text does not parse, 2 when no row covers the request. For tests of the tuner's output.
extern "C" __attribute__((visibility("default"))) int b200TuningLookup(const char* json, int func, int nRanks, unsigned long long bytes, char* out, int outLen) {
  b200::TuningTable t;
  if (!json || !b200::tuneParse(&t, json)) return 1;
  b200::TunePick pk = b200::tunePick(t, func, nRanks, (size_t)bytes);
  if (!pk.valid) return 2;
  snprintf(out, outLen, "%d %d %d", pk.algo, pk.mode, pk.ctas);
  return 0;
}

// Parses the built-in table and returns the number of (collective, rank count) cells it fills, or -1 when it does
// not parse: lets a test without a GPU check the table that every GPU communicator loads.
extern "C" __attribute__((visibility("default"))) int b200TuningDefaultsCheck() {
  b200::TuningTable t;
  if (!b200::tuneParse(&t, b200::kDefaultTuningJson)) return -1;
  int cells = 0;
  for (auto& coll : t.entries)
    for (auto& rows : coll) {
      if (rows.empty()) continue;
      ++cells;
      size_t last = 0;
      for (auto& r : rows) {
        if (r.upto <= last || r.ctas < 0 || r.ctas > 148) return -2;   // thresholds ascend, CTA counts fit the device
        last = r.upto;
      }
    }
  return cells;
}
