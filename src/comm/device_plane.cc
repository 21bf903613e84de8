// GPU data plane: resource window set-up, per-call algorithm choice, kernel launches.
// Every collective is one kernel launch on the caller's stream (plus local copies when a user
// buffer is not inside a registered window and has to be staged through the resource window).
// Reference parity: src/enqueue.cc:1989-2180 (algorithm choice), :2479-2583 (reduction operator
// lowering), src/sym_kernels.cc:599-641 (kernel pick), src/scheduler/symmetric_sched.cc.
#include <mutex>

#include "device_plane.h"
#include "../plugin/plugin.h"

#include <math.h>
#include <stdio.h>

#include <algorithm>

#include "../host/hosttypes.h"

namespace b200 {

B200_PARAM(ScratchMb, "B200_SCRATCH_MB", 256, "Staging area of the resource window per rank (MiB)")
B200_PARAM(WaitTimeoutMs, "B200_WAIT_TIMEOUT_MS", 30000, "Budget of one device-side wait before the kernel gives up")
B200_PARAM(MaxCtas, "MAX_CTAS", 0, "Upper bound on CTAs per collective kernel (0 = from the tuning table)")
B200_PARAM(MinCtas, "MIN_CTAS", 0, "Lower bound on CTAs per collective kernel")
B200_PARAM(MaxNChannels, "MAX_NCHANNELS", 0, "Older name of NCCL_MAX_CTAS (used when that is not set)")
B200_PARAM(MinNChannels, "MIN_NCHANNELS", 0, "Older name of NCCL_MIN_CTAS (used when that is not set)")
B200_PARAM(MaxNRings, "MAX_NRINGS", 0, "Oldest name of NCCL_MAX_CTAS (used when neither that nor NCCL_MAX_NCHANNELS is set)")
B200_PARAM(MinNRings, "MIN_NRINGS", 0, "Oldest name of NCCL_MIN_CTAS (used when neither that nor NCCL_MIN_NCHANNELS is set)")
B200_PARAM(CtaPolicy, "CTA_POLICY", -1, "Overrides ncclConfig_t::CTAPolicy: 0 default, 1 efficiency (half the CTAs the table asks for), 2 zero (copy collectives on registered buffers use the copy engines: no SM)")
B200_PARAM(LLThreshold, "B200_LL_THRESHOLD", -1, "All-reduce payloads up to this many bytes use the one-shot flagged-line kernel")
B200_PARAM(NvlsThreshold, "B200_NVLS_THRESHOLD", -1, "All-reduce payloads from this many bytes use multimem")
B200_PARAM(P2pDisable, "P2P_DISABLE", 0, "Never map peer memory; GPU buffers are staged through host sockets")
B200_PARAM(CopyThreads, "B200_COPY_THREADS", 512, "Threads per CTA of the local copy kernel")
B200_PARAM(CopyUnroll, "B200_COPY_UNROLL", 4, "16-byte loads in flight per thread of the local copy kernel (4 or 8)")
B200_PARAM(CopyCtasPerSm, "B200_COPY_CTAS_PER_SM", 16, "Grid size of the local copy kernel in CTAs per SM")
B200_PARAM(LLMulticast, "B200_LL_MC_MIN_RANKS", -1, "Flagged-line all-reduce / all-gather publish each line with one multimem.st instead of one store per peer from this many ranks on (0 = never, -1 = from the selection table)")
B200_PARAM(CopyKernel, "B200_COPY_KERNEL", 0, "One-rank copy path: 0 = vector loads and stores, 1 = bulk-copy engines through shared memory (messages of 1 MiB and more)")
B200_PARAM(PreloadKernels, "B200_PRELOAD_KERNELS", 1, "Load every collective kernel when the first communicator of a device is created (with lazy module loading the first launch of a kernel can otherwise wait for kernels that are running, which may in turn be waiting for that launch on another rank)")
B200_PARAM(StagePipeline, "B200_STAGE_PIPELINE", 1, "Reductions on unregistered buffers overlap the copies through the staging area with the kernels (two halves, side stream)")
B200_PARAM(StagePipelineMin, "B200_STAGE_PIPELINE_MIN", 67108864, "Smallest message in bytes that is pipelined through the staging area")
B200_PARAM(P2pDirect, "B200_P2P_DIRECT", 1, "Large sends write straight into a receive buffer that lies in a registered window (rendezvous) instead of going through the mailbox")
B200_PARAM(LLCtas, "B200_LL_CTAS", 0, "CTAs of the flagged-line kernels (0: one per 512 lines, at most 64)")
B200_PARAM(LaunchPdl, "B200_PDL", 1, "Programmatic stream serialisation of collective launches (a kernel is scheduled while the previous one of the stream drains): 0 never, 1 yes, but for the flagged-line kernels only up to NCCL_B200_PDL_MAX_CTAS CTAs, 2 always")
B200_PARAM(LaunchPdlMaxCtas, "B200_PDL_MAX_CTAS", 4, "Largest grid of a flagged-line kernel that is launched with programmatic stream serialisation: measured between two such kernels, the gap is 1.5 us against 2.4 us without it for one CTA, about equal at four CTAs, and 3 to 3.5 us from eight CTAs on")
// Whether a launch of `ctas` CTAs asks for programmatic stream serialisation. The flagged-line kernels (`shortKernel`) last a few
// microseconds, so the gap to the next kernel is a large part of a call: there the attribute is dropped for the grids where it
// was measured to widen the gap. Kernels that run for tens of microseconds and more keep it as they were measured with it.
static inline bool pdlFor(int ctas, bool shortKernel) {
  if (paramLaunchPdl() == 2) return true;
  if (paramLaunchPdl() == 0) return false;
  return !shortKernel || ctas <= paramLaunchPdlMaxCtas();
}
B200_PARAM(BarrierMulticast, "B200_BARRIER_MC_MIN_RANKS", -1, "Cross-GPU barriers arrive with one multimem.red on a multicast alias of the flag page from this many ranks on (0 = never, -1 = from the selection table)")

// ------------------------------------------------------------------------------------ tuning
void tuningDefaults(TuningTable* t) {
  for (int n = 0; n <= kMaxRanks; ++n) {
    t->arLLMax[n] = n <= 2 ? (128 << 10) : n <= 4 ? (64 << 10) : (32 << 10);
    t->arNvlsMin[n] = 64 << 10;
    t->agMcMin[n] = 64 << 10;
    t->rsNvlsMin[n] = 64 << 10;
    t->rsLLMax[n] = 16 << 10;
    t->llCopyMax[n] = 16 << 10;
  }
  t->ceMin = 0;
  t->nvlsCtas = 32;
  t->p2pCtas = 64;
  t->copyCtas = 32;
  t->sendrecvCtas = 16;   // one CTA per mailbox slot of a pair: 32 measured half the bandwidth of 16 on messages beyond the mailbox size
  t->bytesPerCta = 128 << 10;
}

// Minimal reader for  {"arLLMax": {"2": 131072, ...}, "nvlsCtas": 32, ...}  files written by the sweep tool.
ncclResult_t tuningLoadFile(TuningTable* t, const char* path) {
  FILE* f = fopen(path, "r");
  if (!f) { WARN("tuning file %s: cannot open", path); return ncclInvalidArgument; }
  std::string s;
  char buf[4096];
  size_t r;
  while ((r = fread(buf, 1, sizeof(buf), f)) > 0) s.append(buf, r);
  fclose(f);
  if (s.find("\"all_reduce\"") != std::string::npos || s.find("\"all_gather\"") != std::string::npos) {
    if (!tuneParse(t, s)) { WARN("tuning file %s: malformed selection table", path); return ncclInvalidArgument; }
    INFO(SUB_TUNING, "selection table loaded from %s", path);
    return ncclSuccess;
  }
  auto scalar = [&](const char* key, long long* out) {
    size_t p = s.find(std::string("\"") + key + "\"");
    if (p == std::string::npos) return false;
    p = s.find(':', p);
    if (p == std::string::npos) return false;
    *out = strtoll(s.c_str() + p + 1, nullptr, 10);
    return true;
  };
  auto table = [&](const char* key, size_t* arr) {
    size_t p = s.find(std::string("\"") + key + "\"");
    if (p == std::string::npos) return;
    size_t b = s.find('{', p), e = s.find('}', p);
    if (b == std::string::npos || e == std::string::npos) return;
    for (int n = 2; n <= kMaxRanks; ++n) {
      std::string k = "\"" + std::to_string(n) + "\"";
      size_t q = s.find(k, b);
      if (q == std::string::npos || q > e) continue;
      q = s.find(':', q);
      arr[n] = (size_t)strtoll(s.c_str() + q + 1, nullptr, 10);
    }
  };
  table("arLLMax", t->arLLMax);
  table("arNvlsMin", t->arNvlsMin);
  table("agMcMin", t->agMcMin);
  table("rsNvlsMin", t->rsNvlsMin);
  table("rsLLMax", t->rsLLMax);
  table("llCopyMax", t->llCopyMax);
  long long v;
  if (scalar("ceMin", &v)) t->ceMin = (size_t)v;
  if (scalar("nvlsCtas", &v)) t->nvlsCtas = (int)v;
  if (scalar("p2pCtas", &v)) t->p2pCtas = (int)v;
  if (scalar("copyCtas", &v)) t->copyCtas = (int)v;
  if (scalar("sendrecvCtas", &v)) t->sendrecvCtas = (int)v;
  if (scalar("bytesPerCta", &v)) t->bytesPerCta = (size_t)v;
  INFO(SUB_TUNING, "tuning table loaded from %s", path);
  return ncclSuccess;
}

// ------------------------------------------------------------------------------------ set-up
// Queries the attributes of every kernel the data plane can launch, which loads it. Once per device and process.
// Reference parity: the loop over all kernels in ncclInitKernelsForDevice (src/enqueue.cc:60-125).
static void preloadKernels(int dev) {
  static std::mutex lock;
  static bool done[64] = {};
  std::lock_guard<std::mutex> g(lock);
  if (dev < 0 || dev >= 64 || done[dev] || !paramPreloadKernels()) return;
  done[dev] = true;
  cudaFuncAttributes attr;
  auto touch = [&](const void* fn) { if (fn && cudaFuncGetAttributes(&attr, fn) != cudaSuccess) (void)cudaGetLastError(); };
  for (const void* fn : {p2pKernelFn(), copyKernelFn(), copyBulkKernelFn(), llCopyKernelFn(), localCopyKernelFn(4), localCopyKernelFn(8), localBulkCopyKernelFn(),
                         signalKernelFn(), waitSignalKernelFn()})
    touch(fn);
  for (int t = 0; t < ncclNumTypes; ++t) {
    touch(scaleKernelFn((ncclDataType_t)t));
    for (int op = RED_SUM; op <= RED_MIN; ++op) {
      touch(reduceKernelFn(KERNEL_REDUCE_P2P, (ncclDataType_t)t, op));
      touch(reduceKernelFn(KERNEL_REDUCE_NVLS, (ncclDataType_t)t, op));
      touch(llReduceKernelFn((ncclDataType_t)t, op));
      touch(llReduceBatchKernelFn((ncclDataType_t)t, op));
      touch(ringKernelFn((ncclDataType_t)t, op));
      touch(treeKernelFn((ncclDataType_t)t, op));
    }
  }
}

ncclResult_t devPlaneCreate(ncclComm* comm) {
  DevicePlane* dp = new DevicePlane;
  comm->devPlane = dp;
  tuningDefaults(&dp->tune);
  tuneLoadDefaults(&dp->tune);
  const char* tf = getEnv("NCCL_TUNING_FILE");
  if (tf && *tf) tuningLoadFile(&dp->tune, tf);
  cudaDeviceProp prop;
  CUDACHECK(cudaGetDeviceProperties(&prop, comm->cudaDev));
  dp->smCount = prop.multiProcessorCount;
  dp->timeoutNs = (uint64_t)paramWaitTimeoutMs() * 1000000ull;
  dp->barrierMcMin = paramBarrierMulticast() >= 0 ? (int)paramBarrierMulticast() : dp->tune.barrierMcMin;
  dp->llMcMin = paramLLMulticast() >= 0 ? (int)paramLLMulticast() : dp->tune.llMcMin;
  CUDACHECK(cudaEventCreateWithFlags(&dp->lastEvent, cudaEventDisableTiming));
  CUDACHECK(cudaStreamCreateWithFlags(&dp->sideStream, cudaStreamNonBlocking));
  for (auto& e : dp->pipeEv) CUDACHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  // function attributes are per device: set with this communicator's device current
  CUDACHECK(cudaFuncSetAttribute(localBulkCopyKernelFn(), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)localBulkCopySmemBytes()));
  CUDACHECK(cudaFuncSetAttribute(copyBulkKernelFn(), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)copyBulkSmemBytes()));
  preloadKernels(comm->cudaDev);
  const size_t privWords = kPrivWords + 2 * kMaxRanks * kSignalsPerPeer;
  CUDACHECK(cudaMalloc(&dp->priv, privWords * sizeof(uint32_t)));
  CUDACHECK(cudaMemset(dp->priv, 0, privWords * sizeof(uint32_t)));
  dp->epochs = dp->priv;
  dp->llEpoch = dp->priv + kBarrierSlots;
  dp->p2pSeq = dp->llEpoch + 4;
  dp->sigSeen = (uint64_t*)(dp->priv + kPrivWords);
  memTrack(comm, dp->priv, privWords * sizeof(uint32_t), MEM_PERSIST, "epochs and sequence numbers");
  if (comm->nRanks == 1) return ncclSuccess;

  int usable = comm->lsaAll ? 1 : 0;
  if (usable) {
    NCCLCHECK(symInit(comm));
    dp->stageBytes = (size_t)paramScratchMb() << 20;
    dp->offLL = kSyncPageBytes;
    dp->offP2pLL = dp->offLL + kLLRegionBytes;
    dp->offMailbox = dp->offP2pLL + kP2pLLBytes;
    dp->offStage = alignUp(dp->offMailbox + kMailboxBytes, (size_t)(2 << 20));
    dp->resSize = dp->offStage + dp->stageBytes;
    ncclResult_t r = memAlloc(&dp->resBase, dp->resSize, comm->cudaDev);
    if (r == ncclSuccess) {
      // only the control part needs zeroing: flags, flagged lines
      if (cudaMemset(dp->resBase, 0, dp->offMailbox) != cudaSuccess) { (void)cudaGetLastError(); r = ncclUnhandledCudaError; }
      cudaDeviceSynchronize();
    }
    if (r == ncclSuccess) r = symWindowRegister(comm, dp->resBase, dp->resSize, &dp->resWin, NCCL_WIN_COLL_SYMMETRIC);
    if (r != ncclSuccess || !dp->resWin || !dp->resWin->symmetric) usable = 0;
    if (usable) {
      // the resource window is working memory: a suspend gives it back, a resume maps it again with clean flags
      // and restarts every epoch and sequence number that is compared against them
      memTrack(comm, dp->resBase, dp->resSize, MEM_SCRATCH, "resource window", &dp->resWin, NCCL_WIN_COLL_SYMMETRIC, dp->offMailbox, [comm] {
        DevicePlane* d = comm->devPlane;
        cudaMemset(d->priv, 0, (kPrivWords + 2 * kMaxRanks * kSignalsPerPeer) * sizeof(uint32_t));
        d->ceEpoch = 0;
      });
    }
  }
  // every rank must reach the same decision
  std::vector<int> oks(comm->nRanks, 0);
  oks[comm->rank] = usable;
  NCCLCHECK(bootstrapAllGather(comm->bootstrap, oks.data(), sizeof(int)));
  for (int v : oks) usable = usable && v;
  if (!usable) {
    if (comm->lsaAll) INFO(SUB_INIT, "peer mappings unavailable: GPU buffers will be staged through host sockets");
    comm->lsaAll = false;
    dp->hostStageBytes = 64 << 20;
    CUDACHECK(cudaHostAlloc(&dp->hostStage, dp->hostStageBytes, cudaHostAllocDefault));
    if (!comm->hostPlane) NCCLCHECK(hostPlaneCreate(comm));
  }
  NCCLCHECK(bootstrapBarrier(comm->bootstrap));
  return ncclSuccess;
}

void devPlaneDestroy(ncclComm* comm) {
  DevicePlane* dp = comm->devPlane;
  if (!dp) return;
  cudaDeviceSynchronize();
  (void)cudaGetLastError();
  if (comm->sym) symDestroy(comm);   // releases every window, the resource window included
  if (dp->resBase) memFree(dp->resBase);
  if (dp->priv) cudaFree(dp->priv);
  if (dp->reshardRuns) cudaFree(dp->reshardRuns);
  if (dp->lastEvent) cudaEventDestroy(dp->lastEvent);
  for (auto& e : dp->pipeEv) if (e) cudaEventDestroy(e);
  if (dp->sideStream) cudaStreamDestroy(dp->sideStream);
  if (dp->hostStage) cudaFreeHost(dp->hostStage);
  (void)cudaGetLastError();
  delete dp;
  comm->devPlane = nullptr;
}

ncclResult_t devPlaneCheckStatus(ncclComm* comm) {
  if (!comm->devStatus) return ncclSuccess;
  uint32_t code = comm->devStatus[0];
  if (code == DEV_OK) return ncclSuccess;
  static const char* kinds[] = {"?", "barrier", "flagged line", "mailbox ready flag", "mailbox ack flag", "signal", "tile flag"};
  uint32_t kind = comm->devStatus[1];
  WARN("rank %d: device-side wait on a %s of rank %u %s (expected value %u)", comm->rank, kind < 7 ? kinds[kind] : "?",
       comm->devStatus[2], code == DEV_TIMEOUT ? "timed out" : "was aborted", comm->devStatus[3]);
  return code == DEV_TIMEOUT ? ncclTimeout : ncclInternalError;
}

// ------------------------------------------------------------------------------------ helpers
struct DevOp {
  int red = RED_SUM;
  int scaleMode = SCALE_NONE;
  float scaleF = 1.f;
  double scaleD = 1.0;
  long long intDiv = 1;
  bool premul = false;
  unsigned long long premulBits = 0;
  const void* premulPtr = nullptr;
};

static bool isFloatType(ncclDataType_t t) {
  return t == ncclFloat16 || t == ncclFloat32 || t == ncclFloat64 || t == ncclBfloat16 || t == ncclFloat8e4m3 || t == ncclFloat8e5m2;
}

static ncclResult_t lowerOp(ncclComm* comm, const Task& t, DevOp* d) {
  switch (t.op) {
    case ncclSum: d->red = RED_SUM; return ncclSuccess;
    case ncclProd: d->red = RED_PROD; return ncclSuccess;
    case ncclMax: d->red = RED_MAX; return ncclSuccess;
    case ncclMin: d->red = RED_MIN; return ncclSuccess;
    case ncclAvg:
      d->red = RED_SUM;
      if (isFloatType(t.type)) { d->scaleMode = SCALE_MUL; d->scaleF = 1.0f / comm->nRanks; d->scaleD = 1.0 / comm->nRanks; }
      else { d->scaleMode = SCALE_INTDIV; d->intDiv = comm->nRanks; }
      return ncclSuccess;
    default: break;
  }
  int idx = t.op - ncclNumOps;
  if (idx < 0 || idx >= (int)comm->userOps.size() || !comm->userOps[idx].used) { WARN("invalid reduction operator %d", t.op); return ncclInvalidArgument; }
  const UserRedOp& u = comm->userOps[idx];
  if (u.type != t.type) { WARN("reduction operator was created for %s, used with %s", typeName(u.type), typeName(t.type)); return ncclInvalidArgument; }
  d->red = RED_SUM;
  d->premul = true;
  d->premulBits = u.scalarBits;
  d->premulPtr = u.residence == ncclScalarDevice ? u.devScalar : nullptr;
  return ncclSuccess;
}

static void fillSync(ncclComm* comm, SyncArgs* s) {
  DevicePlane* dp = comm->devPlane;
  memset(s, 0, sizeof(*s));
  for (int p = 0; p < comm->nRanks; ++p) s->inbox[p] = (uint32_t*)dp->resWin->host.peerPtr[p];
  s->epoch[comm->rank] = dp->epochs;
  s->status[comm->rank] = comm->devStatusDev;
  s->abortFlag = comm->abortFlagDev;
  s->timeoutNs = dp->timeoutNs;
  s->stamps = dp->curStamp;
  // every rank takes the same decision: the multicast alias exists on all ranks or on none
  if (dp->resWin->host.mcPtr && dp->barrierMcMin > 0 && comm->nRanks >= dp->barrierMcMin)
    s->mcArrive = (uint32_t*)((char*)dp->resWin->host.mcPtr + kOffMcBarrier);
}

static void baseArgs(ncclComm* comm, CollArgs* a, int func) {
  DevicePlane* dp = comm->devPlane;
  memset(a, 0, sizeof(*a));
  a->rank = comm->rank;
  a->nRanks = comm->nRanks;
  a->func = func;
  fillSync(comm, &a->sync);
  for (int p = 0; p < comm->nRanks; ++p) a->ll[p] = (char*)dp->resWin->host.peerPtr[p] + dp->offLL;
  a->llEpoch[comm->rank] = dp->llEpoch;
  if (dp->resWin->host.mcPtr && dp->llMcMin > 0 && comm->nRanks >= dp->llMcMin) a->llMc = (char*)dp->resWin->host.mcPtr + dp->offLL;
}

// Peer-visible aliases of `ptr` when it lies in a symmetric window (same offset on every rank).
struct Aliases {
  bool ok = false;
  void* peer[kMaxRanks] = {};
  void* mc = nullptr;
};
static Aliases aliasesOf(ncclComm* comm, const void* ptr, size_t bytes) {
  Aliases al;
  if (!ptr) return al;
  SymWindow* w = symFindWindow(comm, ptr, bytes ? bytes : 1);
  if (!w || !w->symmetric) return al;
  size_t off = (uintptr_t)ptr - (uintptr_t)w->host.userPtr;
  for (int p = 0; p < comm->nRanks; ++p) al.peer[p] = (char*)w->host.peerPtr[p] + off;
  if (w->host.mcPtr) al.mc = (char*)w->host.mcPtr + off;
  al.ok = true;
  return al;
}
static Aliases stageAliases(ncclComm* comm, size_t off) {
  DevicePlane* dp = comm->devPlane;
  Aliases al;
  for (int p = 0; p < comm->nRanks; ++p) al.peer[p] = (char*)dp->resWin->host.peerPtr[p] + dp->offStage + off;
  if (dp->resWin->host.mcPtr) al.mc = (char*)dp->resWin->host.mcPtr + dp->offStage + off;
  al.ok = true;
  return al;
}

static bool aligned16(const Aliases& al, int n) {
  for (int p = 0; p < n; ++p) if ((uintptr_t)al.peer[p] & 15) return false;
  return true;
}

static thread_local int tPickCtas = 0;   // CTA count of the measured row that chose this launch (0 = none)

static int clampCtas(ncclComm* comm, size_t bytes, int cap) {
  DevicePlane* dp = comm->devPlane;
  if (tPickCtas > 0) cap = tPickCtas;
  int64_t envMax = paramMaxCtas(), envMin = paramMinCtas();
  if (envMax <= 0) envMax = paramMaxNChannels();
  if (envMin <= 0) envMin = paramMinNChannels();
  if (envMax <= 0) envMax = paramMaxNRings();   // the oldest spelling
  if (envMin <= 0) envMin = paramMinNRings();
  const int policy = paramCtaPolicy() >= 0 ? (int)paramCtaPolicy() : comm->config.CTAPolicy;
  if ((policy & NCCL_CTA_POLICY_EFFICIENCY) && policy != NCCL_CONFIG_UNDEF_INT) { cap = std::max(1, cap / 2); if (tPickCtas > 0) tPickCtas = std::max(1, tPickCtas / 2); }
  if (comm->config.maxCTAs != NCCL_CONFIG_UNDEF_INT && comm->config.maxCTAs > 0) cap = std::min(cap, comm->config.maxCTAs);
  if (envMax > 0) cap = (int)std::min<int64_t>(cap, envMax);
  cap = std::min(cap, std::min(kMaxCtas, dp->smCount));
  int want = tPickCtas > 0 ? cap : (int)std::min<size_t>((bytes + dp->tune.bytesPerCta - 1) / dp->tune.bytesPerCta, (size_t)cap);
  int lo = 1;
  if (comm->config.minCTAs != NCCL_CONFIG_UNDEF_INT && comm->config.minCTAs > 0) lo = comm->config.minCTAs;
  if (envMin > 0) lo = (int)envMin;
  want = std::max(want, std::min(lo, cap));
  return std::max(want, 1);
}

static bool capturing(cudaStream_t s) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &st) != cudaSuccess) { (void)cudaGetLastError(); return false; }
  return st != cudaStreamCaptureStatusNone;
}

// Collectives of one communicator run one after the other even when issued on different streams.
ncclResult_t devPlaneOrderStreams(ncclComm* comm, cudaStream_t stream) {
  DevicePlane* dp = comm->devPlane;
  if (dp->hasLast && dp->lastStream != stream && !capturing(stream) && !capturing(dp->lastStream)) {
    CUDACHECK(cudaEventRecord(dp->lastEvent, dp->lastStream));
    CUDACHECK(cudaStreamWaitEvent(stream, dp->lastEvent, 0));
  }
  dp->lastStream = stream;
  dp->hasLast = true;
  return ncclSuccess;
}

// what the most recent launch of this thread ran (reported to profiler plugins)
static thread_local const char* tLastAlgo = "NONE";
static thread_local const char* tLastProto = "SIMPLE";
static thread_local int tLastCtas = 0;

static ncclResult_t launchColl(ncclComm* comm, const void* fn, CollArgs* a, int ctas, cudaStream_t stream, const char* algo = "P2P",
                               const char* proto = "SIMPLE", int threads = kCtaThreads, size_t smem = 0) {
  const bool shortKernel = proto && proto[0] == 'L';   // "LL": the flagged-line kernels
  if (!fn) { WARN("no kernel for this data type / operator"); return ncclInvalidUsage; }
  comm->devPlane->launches++;
  tLastAlgo = algo;
  tLastProto = proto;
  tLastCtas = ctas;
  return launchKernel(fn, dim3(ctas), dim3(threads), smem, a, stream, false, pdlFor(ctas, shortKernel));
}

static ncclResult_t scaleCopy(ncclComm* comm, ncclDataType_t type, const void* src, void* dst, size_t count, const DevOp& op,
                              cudaStream_t stream) {
  ScaleArgs sa{src, dst, count, op.premulBits, op.premulPtr};
  int ctas = (int)std::min<size_t>((count + 4095) / 4096, 1024);
  comm->devPlane->launches++;
  return launchKernel(scaleKernelFn(type), dim3(std::max(ctas, 1)), dim3(256), 0, &sa, stream, false);
}

void sliceEven(size_t count, size_t es, int n, size_t* begin, size_t* cnt) {
  const size_t unit = 16 / es;  // elements per 16 bytes
  size_t per = (count + n - 1) / n;
  per = (per + unit - 1) / unit * unit;
  for (int r = 0; r < n; ++r) {
    size_t b = std::min(count, (size_t)r * per);
    begin[r] = b;
    cnt[r] = std::min(per, count - b);
  }
}

// ------------------------------------------------------------------------------------ mesh-to-mesh reshard
ncclResult_t devPlaneRunReshard(ncclComm* comm, SymWindow* win, const ReshardRun* runs, int nRuns, const unsigned long long* tileOff, void* dst,
                                size_t totalBytes, cudaStream_t stream) {
  DevicePlane* dp = comm->devPlane;
  if (!dp || !dp->resWin || !win) return ncclInvalidUsage;
  NCCLCHECK(devPlaneOrderStreams(comm, stream));
  // the run list travels to device memory in stream order; the buffer grows as needed and lives as long as the communicator
  const size_t need = std::max<size_t>((size_t)nRuns, 1) * sizeof(ReshardRun);
  if (need > dp->reshardBytes) {
    if (dp->reshardRuns) { CUDACHECK(cudaStreamSynchronize(stream)); CUDACHECK(cudaFree(dp->reshardRuns)); dp->reshardRuns = nullptr; }
    dp->reshardBytes = std::max(need * 2, (size_t)4096);
    CUDACHECK(cudaMalloc(&dp->reshardRuns, dp->reshardBytes));
  }
  if (nRuns) CUDACHECK(cudaMemcpyAsync(dp->reshardRuns, runs, (size_t)nRuns * sizeof(ReshardRun), cudaMemcpyHostToDevice, stream));
  ReshardArgs a;
  memset(&a, 0, sizeof(a));
  a.rank = comm->rank;
  a.nRanks = comm->nRanks;
  a.nRuns = nRuns;
  a.runs = (const ReshardRun*)dp->reshardRuns;
  for (int p = 0; p < comm->nRanks; ++p) a.winPeer[p] = (const char*)win->host.peerPtr[p];
  a.tileOff = tileOff;
  a.dst = (char*)dst;
  fillSync(comm, &a.sync);
  // every rank launches the same number of CTAs (the barrier slots pair up CTA by CTA): sized from the largest tile a rank can
  // receive, which all ranks know
  int ctas = (int)std::min<size_t>(std::max<size_t>(totalBytes / ((size_t)256 << 10), 1), 32);
  dp->launches++;
  tLastAlgo = "PULL";
  tLastProto = "SIMPLE";
  tLastCtas = ctas;
  return launchKernel(reshardKernelFn(), dim3(ctas), dim3(kCtaThreads), 0, &a, stream, false, pdlFor(ctas, false));
}

// ------------------------------------------------------------------------------------ collectives
static thread_local int tForceAlgo = ALGO_AUTO, tForceMode = -1;
void devPlaneForce(int algo, int mode) { tForceAlgo = algo; tForceMode = mode; }

static int forcedAlgo() {
  if (tForceAlgo != ALGO_AUTO) return tForceAlgo;
  static const char* e = getEnv("NCCL_ALGO");
  if (!e || !*e) return ALGO_AUTO;
  if (!strcasecmp(e, "NVLS")) return ALGO_NVLS;
  if (!strcasecmp(e, "NVLS1") || !strcasecmp(e, "NVLSOneShot")) return ALGO_NVLS_ONESHOT;
  if (!strcasecmp(e, "P2P") || !strcasecmp(e, "TwoShot") || !strcasecmp(e, "Direct")) return ALGO_P2P;
  if (!strcasecmp(e, "LL") || !strcasecmp(e, "OneShot")) return ALGO_LL_ONESHOT;
  if (!strcasecmp(e, "Ring")) return ALGO_RING;
  if (!strcasecmp(e, "Tree")) return ALGO_TREE;
  if (!strcasecmp(e, "CE")) return ALGO_CE;
  return ALGO_AUTO;
}

ncclResult_t ringTreeRun(ncclComm* comm, const Task& t, int algo);   // ring / tree schedules over the staging area, further down in this file
ncclResult_t ceCollRun(ncclComm* comm, const Task& t, bool* handled); // sched/ce_coll.cc

static ncclResult_t runReduction(ncclComm* comm, const Task& t) {
  DevicePlane* dp = comm->devPlane;
  const int n = comm->nRanks, me = comm->rank;
  const size_t es = typeSize(t.type);
  DevOp op;
  NCCLCHECK(lowerOp(comm, t, &op));
  // element counts: `total` elements enter the reduction on every rank
  const size_t total = t.func == FUNC_REDUCESCATTER ? t.count * n : t.count;
  const size_t bytes = total * es;
  if (total == 0) return ncclSuccess;
  int forced = forcedAlgo();
  tPickCtas = 0;
  if (forced == ALGO_AUTO && comm->tuner) {
    int a = ALGO_AUTO, c = 0;
    if (tunerPick(comm, t.func, bytes, 1, symFindWindow(comm, t.recv, 1) != nullptr, &a, &c)) { forced = a; tPickCtas = c; }
  }
  if (forced == ALGO_AUTO && paramLLThreshold() < 0 && paramNvlsThreshold() < 0) {
    TunePick pk = tunePick(dp->tune, t.func, n, bytes);
    if (pk.valid) { forced = pk.algo; tPickCtas = pk.ctas; }
  }

  if ((forced == ALGO_RING || forced == ALGO_TREE) && !op.premul && t.func != FUNC_REDUCE) return ringTreeRun(comm, t, forced);

  // ---- small payloads: flagged lines, one NVLink crossing, no registration needed
  {
    int64_t llEnv = paramLLThreshold();
    const size_t recvBytes = t.count * es;   // what one receiver ends up with
    size_t llMax = llEnv >= 0 ? (size_t)llEnv : (t.func == FUNC_ALLREDUCE ? dp->tune.arLLMax[n] : dp->tune.rsLLMax[n]);
    llMax = std::min(llMax, kLLDataBytes);
    const bool llFits = recvBytes <= kLLDataBytes - 8;   // the last line of a region carries acknowledgements
    if (!op.premul && llFits && (forced == ALGO_LL_ONESHOT || (forced == ALGO_AUTO && recvBytes <= llMax))) {
      CollArgs a;
      baseArgs(comm, &a, t.func);
      a.count = t.count;
      a.root = t.root;
      a.lsend[me] = t.send;
      a.lrecv[me] = t.recv;
      a.scaleMode = op.scaleMode; a.scaleF = op.scaleF; a.scaleD = op.scaleD; a.intDiv = op.intDiv;
      size_t lines = (recvBytes + 7) / 8;
      int ctas = (int)std::min<size_t>((lines + kCtaThreads - 1) / kCtaThreads, 64);
      if (paramLLCtas() > 0) ctas = (int)std::min<int64_t>(paramLLCtas(), 64);
      return launchColl(comm, llReduceKernelFn(t.type, op.red), &a, std::max(ctas, 1), t.stream, "ONESHOT", "LL");
    }
  }

  // ---- one-shot through the switch: every rank reads the whole reduced vector with multimem.ld_reduce
  // and stores it locally. No second phase and no remote store, so the closing barrier carries no
  // release fence. The input must have a multicast alias; the output may be any local buffer, but not
  // the input itself (a rank would overwrite what its peers are still reading).
  // Reference parity: contrib/custom_algos/allreduce/oneshot_mc_allreduce_kernel.cuh.
  if (forced == ALGO_NVLS_ONESHOT && t.func == FUNC_ALLREDUCE && !op.premul && nvlsReduceSupported(t.type, op.red) && bytes % 16 == 0) {
    Aliases in = aliasesOf(comm, t.send, bytes);
    const bool disjoint = (const char*)t.recv + bytes <= (const char*)t.send || (const char*)t.send + bytes <= (const char*)t.recv;
    if (in.ok && in.mc && disjoint && aligned16(in, n) && ((uintptr_t)t.recv & 15) == 0) {
      CollArgs a;
      baseArgs(comm, &a, t.func);
      a.scaleMode = op.scaleMode; a.scaleF = op.scaleF; a.scaleD = op.scaleD; a.intDiv = op.intDiv;
      for (int r = 0; r < n; ++r) { a.sliceBegin[r] = 0; a.sliceCount[r] = total; a.dstOff[r] = 0; }
      a.dstAll = 0;
      a.sendMc = in.mc;
      a.lrecv[me] = t.recv;
      a.vec16 = 1;
      int ctas = clampCtas(comm, bytes, dp->tune.nvlsCtas);
      return launchColl(comm, reduceKernelFn(KERNEL_REDUCE_NVLS, t.type, op.red), &a, ctas, t.stream, "NVLS_ONESHOT");
    }
  }
  if (forced == ALGO_NVLS_ONESHOT) forced = ALGO_NVLS;

  // ---- large: every rank reduces one slice, inputs must be peer-visible
  Aliases sendAl = op.premul ? Aliases{} : aliasesOf(comm, t.send, bytes);
  const bool needRecvAll = t.func == FUNC_ALLREDUCE;
  Aliases recvAl = needRecvAll ? aliasesOf(comm, t.recv, bytes) : Aliases{};
  const bool direct = sendAl.ok && (!needRecvAll || recvAl.ok);

  // Work on buffers outside registered windows goes through the staging area of the resource window in
  // pieces. Large messages are pipelined over the two halves of the area: a side stream copies piece
  // k + 1 in (and piece k - 1 out) while the kernel of piece k runs, so the copies cost nothing but
  // the first and the last one. Each kernel opens with a barrier (every rank's piece is in place) and
  // closes with one (nobody reads this rank's half any more), which is all the cross-rank ordering
  // the reuse of a half needs; events order the two local streams.
  size_t pieceTotal = total;        // elements (over all slices) handled per launch
  bool pipelined = false;
  size_t halfBytes = 0;
  if (!direct) {
    const size_t stageElems = dp->stageBytes / es;
    size_t cap = stageElems / (16 * n) * (16 * n);   // reduce-scatter pieces stay divisible by n, slices by 16 bytes
    pipelined = paramStagePipeline() != 0 && bytes >= (size_t)paramStagePipelineMin() && dp->sideStream != nullptr;
    if (pipelined) {
      // at least four pieces, so that the copies of all but the first and the last one hide behind kernels, of 16 MiB or more
      halfBytes = dp->stageBytes / 2 / 4096 * 4096;
      const size_t unit = (size_t)16 * n;
      const size_t quarter = std::max<size_t>((total / 4 + unit - 1) / unit * unit, ((size_t)16 << 20) / es / unit * unit);
      cap = std::min(halfBytes / es / unit * unit, quarter);
    }
    if (pieceTotal > cap) pieceTotal = cap;
    if (pipelined && pieceTotal >= total) pipelined = false;
  }
  char* const stageBase = dp->resBase ? (char*)dp->resBase + dp->offStage : nullptr;
  cudaStream_t side = pipelined ? dp->sideStream : t.stream;
  // copy-in of the piece that starts at element `done` into the half `h` of the staging area
  auto copyIn = [&](size_t done, size_t cur, int h, cudaStream_t st) -> ncclResult_t {
    char* dstp = stageBase + (size_t)h * halfBytes;
    if (t.func == FUNC_REDUCESCATTER) {
      const size_t rsPiece = cur / n, rsDone = done / n;
      // rows of rsPiece elements, one per destination rank, gathered from a pitch of t.count
      if (op.premul) {
        for (int r = 0; r < n; ++r)
          NCCLCHECK(scaleCopy(comm, t.type, (const char*)t.send + ((size_t)r * t.count + rsDone) * es, dstp + (size_t)r * rsPiece * es, rsPiece, op, st));
      } else {
        // long rows go as one plain copy each (full copy bandwidth); a pitched copy only pays off for many short rows
        if (rsPiece * es >= ((size_t)1 << 20)) {
          for (int r = 0; r < n; ++r)
            CUDACHECK(cudaMemcpyAsync(dstp + (size_t)r * rsPiece * es, (const char*)t.send + ((size_t)r * t.count + rsDone) * es, rsPiece * es, cudaMemcpyDeviceToDevice, st));
        } else {
          CUDACHECK(cudaMemcpy2DAsync(dstp, rsPiece * es, (const char*)t.send + rsDone * es, t.count * es, rsPiece * es, n, cudaMemcpyDeviceToDevice, st));
        }
      }
    } else if (op.premul) {
      NCCLCHECK(scaleCopy(comm, t.type, (const char*)t.send + done * es, dstp, cur, op, st));
    } else {
      CUDACHECK(cudaMemcpyAsync(dstp, (const char*)t.send + done * es, cur * es, cudaMemcpyDeviceToDevice, st));
    }
    return ncclSuccess;
  };
  if (pipelined) {
    CUDACHECK(cudaEventRecord(dp->pipeEv[0], t.stream));          // fork: the side stream sees what the caller queued before
    CUDACHECK(cudaStreamWaitEvent(side, dp->pipeEv[0], 0));
    NCCLCHECK(copyIn(0, std::min(pieceTotal, total), 0, side));
    CUDACHECK(cudaEventRecord(dp->pipeEv[1], side));
  }
  int piece = 0;
  for (size_t done = 0; done < total; ++piece) {
    size_t cur = std::min(pieceTotal, total - done);   // all-reduce / reduce: elements; reduce-scatter: n * piece
    const int h = pipelined ? (piece & 1) : 0;
    CollArgs a;
    baseArgs(comm, &a, t.func);
    a.scaleMode = op.scaleMode; a.scaleF = op.scaleF; a.scaleD = op.scaleD; a.intDiv = op.intDiv;
    a.root = t.root;
    Aliases in, out;
    size_t rsPiece = 0, rsDone = 0;
    if (t.func == FUNC_REDUCESCATTER) { rsPiece = cur / n; rsDone = done / n; if (!direct && rsPiece == 0) rsPiece = t.count; }
    if (direct) {
      in = sendAl;
      out = recvAl;
      cur = total;
    } else {
      in = stageAliases(comm, (size_t)h * halfBytes);
      out = in;
      if (pipelined) {
        // next piece into the other half, once the kernel that last used that half (piece - 1) is done
        const size_t nextDone = done + cur;
        if (nextDone < total) {
          if (piece >= 1) CUDACHECK(cudaStreamWaitEvent(side, dp->pipeEv[3 + ((piece + 1) & 1)], 0));
          NCCLCHECK(copyIn(nextDone, std::min(pieceTotal, total - nextDone), (piece + 1) & 1, side));
          CUDACHECK(cudaEventRecord(dp->pipeEv[1 + ((piece + 1) & 1)], side));
        }
        CUDACHECK(cudaStreamWaitEvent(t.stream, dp->pipeEv[1 + h], 0));
      } else {
        NCCLCHECK(copyIn(done, cur, 0, t.stream));
      }
    }
    // slices
    if (t.func == FUNC_ALLREDUCE) {
      sliceEven(cur, es, n, a.sliceBegin, a.sliceCount);
      for (int r = 0; r < n; ++r) a.dstOff[r] = a.sliceBegin[r];
      a.dstAll = 1;
    } else if (t.func == FUNC_REDUCESCATTER) {
      size_t per = direct ? t.count : rsPiece;
      for (int r = 0; r < n; ++r) { a.sliceBegin[r] = (size_t)r * per; a.sliceCount[r] = per; a.dstOff[r] = 0; }
      a.dstAll = 0;
    } else {  // reduce: the root does all the work
      for (int r = 0; r < n; ++r) { a.sliceBegin[r] = 0; a.sliceCount[r] = r == t.root ? cur : 0; a.dstOff[r] = 0; }
      a.dstAll = 0;
    }
    for (int p = 0; p < n; ++p) { a.send[p] = in.peer[p]; a.recv[p] = out.peer[p]; }
    a.sendMc = in.mc;
    a.recvMc = out.mc;
    // local result pointer for reduce-scatter / reduce
    if (t.func == FUNC_REDUCESCATTER) a.lrecv[me] = (char*)t.recv + (direct ? 0 : rsDone * es);
    else if (t.func == FUNC_REDUCE) a.lrecv[me] = me == t.root ? (char*)t.recv + (direct ? 0 : done * es) : nullptr;
    const size_t curBytes = cur * es;
    bool v16 = aligned16(in, n) && (!a.dstAll || aligned16(out, n));
    if (!a.dstAll && a.lrecv[me] && ((uintptr_t)a.lrecv[me] & 15)) v16 = false;
    if (t.func == FUNC_REDUCESCATTER && (a.sliceCount[0] * es) % 16) v16 = false;
    a.vec16 = v16;
    // multimem needs whole 16-byte packs in every slice
    bool nvlsOk = in.mc && (!a.dstAll || out.mc) && v16 && nvlsReduceSupported(t.type, op.red) && (curBytes % 16 == 0) &&
                  (t.func != FUNC_REDUCESCATTER || (a.sliceCount[0] * es) % 16 == 0);
    int64_t nvEnv = paramNvlsThreshold();
    size_t nvMin = nvEnv >= 0 ? (size_t)nvEnv : (t.func == FUNC_ALLREDUCE ? dp->tune.arNvlsMin[n] : dp->tune.rsNvlsMin[n]);
    bool useNvls = nvlsOk && (forced == ALGO_NVLS || (forced == ALGO_AUTO && curBytes >= nvMin));
    if (forced == ALGO_P2P) useNvls = false;
    const size_t perRankBytes = t.func == FUNC_REDUCE ? curBytes : curBytes / n;
    int ctas = clampCtas(comm, perRankBytes, useNvls ? dp->tune.nvlsCtas : dp->tune.p2pCtas);
    NCCLCHECK(launchColl(comm, reduceKernelFn(useNvls ? KERNEL_REDUCE_NVLS : KERNEL_REDUCE_P2P, t.type, op.red), &a, ctas, t.stream, useNvls ? "NVLS" : "P2P"));
    if (direct) break;
    if (pipelined) CUDACHECK(cudaEventRecord(dp->pipeEv[3 + h], t.stream));   // kernel of this piece done: its half may be copied out / refilled
    // copy-out of the staged all-reduce
    if (t.func == FUNC_ALLREDUCE) {
      if (pipelined) CUDACHECK(cudaStreamWaitEvent(side, dp->pipeEv[3 + h], 0));
      CUDACHECK(cudaMemcpyAsync((char*)t.recv + done * es, stageBase + (size_t)h * halfBytes, cur * es, cudaMemcpyDeviceToDevice, side));
    }
    done += cur;
  }
  if (pipelined) {
    CUDACHECK(cudaEventRecord(dp->pipeEv[5], side));              // join: the caller's stream continues after the last copy
    CUDACHECK(cudaStreamWaitEvent(t.stream, dp->pipeEv[5], 0));
  }
  return ncclSuccess;
}

// ---- several small all-reduces of one group in one launch (flagged lines)
// A task can join a batch when it is an all-reduce with a built-in operator whose payload the
// selection table would send down the flagged-line path anyway.
static size_t llLimit(ncclComm* comm) {
  DevicePlane* dp = comm->devPlane;
  const int n = comm->nRanks;
  size_t lim = dp->tune.arLLMax[n];
  const std::vector<TuneEntry>& rows = dp->tune.entries[0][n];
  if (!rows.empty()) lim = rows[0].algo == ALGO_LL_ONESHOT ? rows[0].upto : 0;
  if (paramLLThreshold() >= 0) lim = (size_t)paramLLThreshold();
  return std::min(lim, kLLDataBytes / 2);
}

bool devPlaneBatchable(ncclComm* comm, const Task& t) {
  if (!comm->devPlane || comm->hostOnly || comm->nRanks < 2 || !comm->lsaAll || comm->tuner) return false;
  if (t.func != FUNC_ALLREDUCE || t.op >= ncclNumOps || t.count == 0) return false;
  const int forced = forcedAlgo();
  if (forced != ALGO_AUTO && forced != ALGO_LL_ONESHOT) return false;
  return t.count * typeSize(t.type) <= llLimit(comm);
}

// Tasks must be batchable, of one type, operator and stream. Returns how many of them went into the launch.
ncclResult_t devPlaneRunLLBatch(ncclComm* comm, const Task* tasks, int count, int* taken) {
  DevicePlane* dp = comm->devPlane;
  *taken = 0;
  NCCLCHECK(devPlaneCheckStatus(comm));
  int cur = -1;
  CUDACHECK(cudaGetDevice(&cur));
  if (cur != comm->cudaDev) CUDACHECK(cudaSetDevice(comm->cudaDev));
  const Task& t0 = tasks[0];
  const size_t es = typeSize(t0.type);
  DevOp op;
  NCCLCHECK(lowerOp(comm, t0, &op));
  LLBatchArgs b;
  baseArgs(comm, &b.c, FUNC_ALLREDUCE);
  b.c.scaleMode = op.scaleMode; b.c.scaleF = op.scaleF; b.c.scaleD = op.scaleD; b.c.intDiv = op.intDiv;
  const size_t cap = std::min(llLimit(comm) * 2, kLLDataBytes - 8) / 8;   // lines
  uint32_t lines = 0;
  int k = 0;
  for (; k < count && k < kMaxLLItems; ++k) {
    const size_t nl = (tasks[k].count * es + 7) / 8;
    if (lines + nl > cap) break;
    b.items[k] = LLItem{(long long)(uintptr_t)tasks[k].send, (long long)(uintptr_t)tasks[k].recv, (uint32_t)tasks[k].count, lines};
    lines += (uint32_t)nl;
  }
  if (k == 0) return ncclInternalError;
  b.nItems = k;
  b.totalLines = lines;
  NCCLCHECK(devPlaneOrderStreams(comm, t0.stream));
  const int ctas = (int)std::min<size_t>(((size_t)lines + kCtaThreads - 1) / kCtaThreads, 64);
  dp->launches++;
  ncclResult_t r = launchKernel(llReduceBatchKernelFn(t0.type, op.red), dim3(std::max(ctas, 1)), dim3(kCtaThreads), 0, &b, t0.stream, false, pdlFor(std::max(ctas, 1), true));
  if (cur != comm->cudaDev && cur >= 0) cudaSetDevice(cur);
  *taken = k;
  return r;
}

static ncclResult_t runCopyColl(ncclComm* comm, const Task& t) {
  DevicePlane* dp = comm->devPlane;
  const int n = comm->nRanks, me = comm->rank;
  const size_t es = typeSize(t.type);
  const size_t B = t.count * es;   // bytes per segment
  if (B == 0) return ncclSuccess;
  int forced = forcedAlgo();
  int modeForce = tForceMode;
  bool bulk = false;
  tPickCtas = 0;
  if (forced == ALGO_AUTO && modeForce < 0 && comm->tuner) {
    int a = ALGO_AUTO, c = 0;
    if (tunerPick(comm, t.func, B * (t.func == FUNC_ALLGATHER ? n : 1), 1, symFindWindow(comm, t.recv, 1) != nullptr, &a, &c)) {
      forced = a == ALGO_TREE ? ALGO_AUTO : a;   // copy collectives have no tree form
      tPickCtas = c;
    }
  }
  if (forced == ALGO_AUTO && modeForce < 0) {
    size_t key = (t.func == FUNC_ALLGATHER || t.func == FUNC_ALLTOALL) ? B * n : B;
    TunePick pk = tunePick(dp->tune, t.func, n, key);
    if (pk.valid) { forced = pk.algo; modeForce = pk.mode; tPickCtas = pk.ctas; }
  }
  const bool wantSplit = modeForce == MODE_SPLIT;
  if (wantSplit) modeForce = -1;
  if (modeForce >= 0 && (modeForce & MODE_BULK)) { bulk = true; modeForce &= ~MODE_BULK; }
  if (forced == ALGO_RING && t.func == FUNC_ALLGATHER) return ringTreeRun(comm, t, forced);
  const int ctaPolicy = paramCtaPolicy() >= 0 ? (int)paramCtaPolicy() : comm->config.CTAPolicy;
  const bool zeroSm = ctaPolicy != NCCL_CONFIG_UNDEF_INT && (ctaPolicy & NCCL_CTA_POLICY_ZERO) && forced == ALGO_AUTO && B >= ((size_t)1 << 20);
  if (forced == ALGO_CE || zeroSm || (forced == ALGO_AUTO && dp->tune.ceMin && B >= dp->tune.ceMin)) {
    bool handled = false;
    NCCLCHECK(ceCollRun(comm, t, &handled));
    if (handled) return ncclSuccess;
  }
  // ---- small blocks: flagged lines
  if (B <= kLLDataBytes - 8 && (forced == ALGO_LL_ONESHOT || (forced == ALGO_AUTO && B <= dp->tune.llCopyMax[n]))) {
    CollArgs a;
    baseArgs(comm, &a, t.func);
    a.root = t.root;
    a.count = B;
    a.sendStride = B;
    a.recvStride = B;
    a.lsend[me] = t.send;
    a.lrecv[me] = t.recv;
    size_t items = ((B + 7) / 8) * (size_t)(n - 1);
    int ctas = (int)std::min<size_t>((items + kCtaThreads - 1) / kCtaThreads, 64);
    if (paramLLCtas() > 0) ctas = (int)std::min<int64_t>(paramLLCtas(), 64);
    return launchColl(comm, llCopyKernelFn(), &a, std::max(ctas, 1), t.stream, "ONESHOT", "LL");
  }
  size_t sendBytes = B, recvBytes = B;
  if (t.func == FUNC_ALLGATHER || t.func == FUNC_GATHER) recvBytes = B * n;
  if (t.func == FUNC_ALLTOALL) { sendBytes = B * n; recvBytes = B * n; }
  if (t.func == FUNC_SCATTER) sendBytes = B * n;
  // which side is significant on this rank
  const bool recvEverywhere = t.func != FUNC_GATHER;
  const bool sendEverywhere = t.func != FUNC_BROADCAST && t.func != FUNC_SCATTER;
  Aliases recvAl = recvEverywhere ? aliasesOf(comm, t.recv, recvBytes) : Aliases{};
  Aliases sendAl = sendEverywhere ? aliasesOf(comm, t.send, sendBytes) : Aliases{};
  // registration must be agreed upon: a buffer counts as symmetric only if its window is (collective property)
  int mode;
  bool staged = false;
  if (recvAl.ok && !(modeForce == MODE_PULL && sendAl.ok)) mode = MODE_PUSH;
  else if (sendAl.ok) mode = MODE_PULL;
  else { mode = MODE_PULL; staged = true; }

  // ---- broadcast with the work shared out among the non-root ranks (see copyCollKernel). Every rank takes this decision
  // from what all ranks know: the output windows (symmetric offsets) and the size. Whether the root's input can be pulled
  // is the root's knowledge; it tells the others from inside the kernel.
  if (wantSplit && t.func == FUNC_BROADCAST && n >= 3 && recvAl.ok && B % 16 == 0 && aligned16(recvAl, n) && comm->sym && comm->sym->winTableDev) {
    CollArgs a;
    baseArgs(comm, &a, t.func);
    a.root = t.root;
    a.count = B;
    a.sendStride = a.recvStride = B;
    a.mode = MODE_SPLIT;
    a.lsend[me] = t.send;
    a.lrecv[me] = t.recv;
    for (int p = 0; p < n; ++p) a.recv[p] = recvAl.peer[p];
    a.winTable = (void* const*)comm->sym->winTableDev;
    a.vec16 = 1;
    if (me == t.root) {
      SymWindow* w = symFindWindow(comm, t.send, B);
      if (w && w->symmetric && w->slot >= 0 && ((uintptr_t)t.send & 15) == 0) {
        a.bcastSlot = w->slot + 1;
        a.bcastOff = (uintptr_t)t.send - (uintptr_t)w->host.userPtr;
      } else if ((uintptr_t)t.send & 15) {
        a.vec16 = 0;   // the root pushes everything itself, byte by byte where it has to
      }
    }
    int ctas = clampCtas(comm, B, dp->tune.copyCtas);
    return launchColl(comm, copyKernelFn(), &a, ctas, t.stream, "SPLIT");
  }

  // pieces that fit the staging area
  const size_t segsStaged = (t.func == FUNC_ALLTOALL || t.func == FUNC_SCATTER) ? n : 1;
  size_t piece = B;
  if (staged) {
    size_t cap = dp->stageBytes / segsStaged / 16 * 16;
    piece = std::min(B, cap);
  }
  for (size_t done = 0; done < B; done += piece) {
    const size_t cur = std::min(piece, B - done);
    CollArgs a;
    baseArgs(comm, &a, t.func);
    a.root = t.root;
    a.count = cur;
    a.sendStride = staged ? cur : B;
    a.recvStride = B;
    a.mode = mode;
    Aliases in = sendAl, out = recvAl;
    a.lsend[me] = (const char*)t.send + done;
    a.lrecv[me] = (char*)t.recv + done;
    if (staged) {
      in = stageAliases(comm, 0);
      char* st = (char*)dp->resBase + dp->offStage;
      const bool iSend = sendEverywhere || me == t.root;
      if (iSend) {
        if (segsStaged > 1) {
          CUDACHECK(cudaMemcpy2DAsync(st, cur, (const char*)t.send + done, B, cur, n, cudaMemcpyDeviceToDevice, t.stream));
        } else {
          CUDACHECK(cudaMemcpyAsync(st, (const char*)t.send + done, cur, cudaMemcpyDeviceToDevice, t.stream));
        }
      }
      a.lsend[me] = st;
    } else if (cur != B) {
      return ncclInternalError;
    }
    for (int p = 0; p < n; ++p) { a.send[p] = in.peer[p]; a.recv[p] = out.peer[p]; }
    bool v16 = (cur % 16 == 0) && (((uintptr_t)a.lsend[me] | (uintptr_t)a.lrecv[me]) & 15) == 0;
    if (mode == MODE_PUSH) v16 = v16 && aligned16(out, n); else v16 = v16 && aligned16(in, n);
    if (B % 16) v16 = false;
    a.vec16 = v16;
    if (mode == MODE_PUSH && out.mc && v16 && (t.func == FUNC_ALLGATHER || t.func == FUNC_BROADCAST) &&
        modeForce != MODE_PUSH && (forced == ALGO_NVLS || modeForce == MODE_MC || (forced == ALGO_AUTO && cur >= dp->tune.agMcMin[n]))) {
      a.mode = MODE_MC;
      a.recvMc = out.mc;
    }
    // offsets of this piece inside peer buffers
    if (done) {
      for (int p = 0; p < n; ++p) {
        if (a.send[p] && !staged) a.send[p] = (const char*)a.send[p] + done;
        if (a.recv[p]) a.recv[p] = (char*)a.recv[p] + done;
      }
      if (a.recvMc) a.recvMc = (char*)a.recvMc + done;
    }
    size_t moved = cur * ((t.func == FUNC_BROADCAST && mode != MODE_PUSH) ? 1 : (a.mode == MODE_MC ? 1 : n));
    int ctas = clampCtas(comm, moved, dp->tune.copyCtas);
    const char* algoName = a.mode == MODE_MC ? "NVLS" : a.mode == MODE_PULL ? "P2P_PULL" : "P2P_PUSH";
    if (bulk && v16 && cur % 16 == 0) {
      NCCLCHECK(launchColl(comm, copyBulkKernelFn(), &a, ctas, t.stream, algoName, "BULK", 32, copyBulkSmemBytes()));
    } else {
      NCCLCHECK(launchColl(comm, copyKernelFn(), &a, ctas, t.stream, algoName));
    }
  }
  return ncclSuccess;
}

static ncclResult_t runOneRank(ncclComm* comm, const Task& t) {
  const size_t es = typeSize(t.type);
  size_t bytes = t.count * es;
  const void* src = t.send;
  void* dst = t.recv;
  switch (t.func) {
    case FUNC_SEND: case FUNC_RECV:
      WARN("send/recv to self must be grouped");
      return ncclInvalidUsage;
    default: break;
  }
  if (bytes == 0) return ncclSuccess;
  bool reduces = t.func == FUNC_ALLREDUCE || t.func == FUNC_REDUCE || t.func == FUNC_REDUCESCATTER;
  if (reduces && t.op >= ncclNumOps) {
    DevOp op;
    NCCLCHECK(lowerOp(comm, t, &op));
    return scaleCopy(comm, t.type, src, dst, t.count, op, t.stream);
  }
  if (src != dst) {
    ScaleArgs ca{src, dst, bytes, 0, nullptr};
    if (paramCopyKernel() == 1 && bytes >= (1u << 20) && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
      comm->devPlane->launches++;
      return launchKernel(localBulkCopyKernelFn(), dim3(comm->devPlane->smCount), dim3(32), localBulkCopySmemBytes(), &ca, t.stream, false);
    }
    const int threads = (int)paramCopyThreads(), unroll = (int)paramCopyUnroll();
    size_t perCta = (size_t)threads * unroll * 16;
    int ctas = (int)std::min<size_t>((bytes + perCta - 1) / perCta, (size_t)comm->devPlane->smCount * paramCopyCtasPerSm());
    comm->devPlane->launches++;
    NCCLCHECK(launchKernel(localCopyKernelFn(unroll), dim3(std::max(ctas, 1)), dim3(threads), 0, &ca, t.stream, false));
  }
  return ncclSuccess;
}

// GPU buffers, ranks that cannot map each other: stage through pinned host memory and sockets.
static ncclResult_t runViaHost(ncclComm* comm, const Task& t) {
  const int n = comm->nRanks;
  const size_t es = typeSize(t.type);
  size_t sendBytes = t.count * es, recvBytes = t.count * es;
  switch (t.func) {
    case FUNC_ALLGATHER: recvBytes *= n; break;
    case FUNC_REDUCESCATTER: sendBytes *= n; break;
    case FUNC_ALLTOALL: sendBytes *= n; recvBytes *= n; break;
    case FUNC_GATHER: recvBytes *= n; break;
    case FUNC_SCATTER: sendBytes *= n; break;
    default: break;
  }
  std::vector<char> hs(t.send ? sendBytes : 0), hr(t.recv ? recvBytes : 0);
  CUDACHECK(cudaStreamSynchronize(t.stream));
  if (t.send && t.func != FUNC_RECV) CUDACHECK(cudaMemcpy(hs.data(), t.send, sendBytes, cudaMemcpyDeviceToHost));
  Task ht = t;
  ht.send = hs.data();
  ht.recv = hr.data();
  NCCLCHECK(hostPlaneRun(comm, ht));
  bool wroteRecv = t.recv && !(t.func == FUNC_SEND) && !((t.func == FUNC_REDUCE || t.func == FUNC_GATHER) && comm->rank != t.root);
  if (wroteRecv) CUDACHECK(cudaMemcpy(t.recv, hr.data(), recvBytes, cudaMemcpyHostToDevice));
  return ncclSuccess;
}

ncclResult_t signalRun(ncclComm* comm, const Task& t);  // sched/rma.cc

ncclResult_t devPlaneRun(ncclComm* comm, const Task& t, ncclSimInfo_t* sim) {
  (void)sim;
  DevicePlane* dp = comm->devPlane;
  if (!dp) return ncclInternalError;
  NCCLCHECK(devPlaneCheckStatus(comm));
  int cur = -1;
  CUDACHECK(cudaGetDevice(&cur));
  if (cur != comm->cudaDev) CUDACHECK(cudaSetDevice(comm->cudaDev));
  ncclResult_t r = ncclSuccess;
  void* prof = comm->profiler ? profilerTaskStart(comm, t) : nullptr;
  tLastAlgo = comm->nRanks == 1 ? "ONERANK" : comm->lsaAll ? "P2P" : "HOST";
  tLastProto = "SIMPLE";
  tLastCtas = 0;
  if (t.func == FUNC_PUTSIGNAL || t.func == FUNC_SIGNAL || t.func == FUNC_WAITSIGNAL) {
    r = devPlaneOrderStreams(comm, t.stream);
    if (r == ncclSuccess) r = signalRun(comm, t);
  } else if (comm->nRanks == 1) {
    r = runOneRank(comm, t);
  } else if (!comm->lsaAll) {
    r = runViaHost(comm, t);
  } else {
    r = devPlaneOrderStreams(comm, t.stream);
    if (r == ncclSuccess) {
      switch (t.func) {
        case FUNC_ALLREDUCE: case FUNC_REDUCESCATTER: case FUNC_REDUCE: r = runReduction(comm, t); break;
        case FUNC_ALLGATHER: case FUNC_BROADCAST: case FUNC_ALLTOALL: case FUNC_GATHER: case FUNC_SCATTER: r = runCopyColl(comm, t); break;
        default: WARN("unexpected function %d", t.func); r = ncclInternalError;
      }
    }
  }
  if (prof) profilerTaskStop(comm, t, prof, tLastAlgo, tLastProto, tLastCtas);
  if (cur != comm->cudaDev && cur >= 0) cudaSetDevice(cur);
  return r;
}

ncclResult_t devPlaneRunP2pGroup(ncclComm* comm, const std::vector<Task>& tasks) {
  DevicePlane* dp = comm->devPlane;
  if (!dp) return ncclInternalError;
  if (tasks.empty()) return ncclSuccess;
  NCCLCHECK(devPlaneCheckStatus(comm));
  cudaStream_t stream = tasks[0].stream;
  int cur = -1;
  CUDACHECK(cudaGetDevice(&cur));
  if (cur != comm->cudaDev) CUDACHECK(cudaSetDevice(comm->cudaDev));
  ncclResult_t res = ncclSuccess;
  // sends and receives addressed to myself pair up in posting order and become local copies
  std::vector<const Task*> selfS, selfR;
  std::vector<const Task*> remote;
  for (auto& t : tasks) {
    if (t.root == comm->rank) (t.func == FUNC_SEND ? selfS : selfR).push_back(&t);
    else remote.push_back(&t);
  }
  if (selfS.size() != selfR.size()) { WARN("send/recv to self: %zu sends but %zu receives in the group", selfS.size(), selfR.size()); return ncclInvalidUsage; }
  for (size_t i = 0; i < selfS.size(); ++i) {
    size_t sb = selfS[i]->count * typeSize(selfS[i]->type), rb = selfR[i]->count * typeSize(selfR[i]->type);
    if (sb > rb) { WARN("send to self is larger than the matching receive"); return ncclInvalidArgument; }
    if (sb && selfS[i]->send != selfR[i]->recv) CUDACHECK(cudaMemcpyAsync(selfR[i]->recv, selfS[i]->send, sb, cudaMemcpyDeviceToDevice, stream));
  }
  if (remote.empty()) goto out;
  if (!comm->lsaAll) {
    CUDACHECK(cudaStreamSynchronize(stream));
    std::vector<Task> ht;
    std::vector<std::vector<char>> bufs(remote.size());
    for (size_t i = 0; i < remote.size(); ++i) {
      const Task& t = *remote[i];
      size_t b = t.count * typeSize(t.type);
      bufs[i].resize(b);
      Task h = t;
      if (t.func == FUNC_SEND) { CUDACHECK(cudaMemcpy(bufs[i].data(), t.send, b, cudaMemcpyDeviceToHost)); h.send = bufs[i].data(); }
      else h.recv = bufs[i].data();
      ht.push_back(h);
    }
    res = hostPlaneRunP2pGroup(comm, ht);
    if (res == ncclSuccess)
      for (size_t i = 0; i < remote.size(); ++i)
        if (remote[i]->func == FUNC_RECV) CUDACHECK(cudaMemcpy(remote[i]->recv, bufs[i].data(), bufs[i].size(), cudaMemcpyHostToDevice));
    goto out;
  }
  res = devPlaneOrderStreams(comm, stream);
  for (size_t first = 0; first < remote.size() && res == ncclSuccess; first += kMaxP2pOps) {
    size_t nOps = std::min<size_t>(kMaxP2pOps, remote.size() - first);
    P2pArgs a;
    memset(&a, 0, sizeof(a));
    a.rank = comm->rank;
    a.nRanks = comm->nRanks;
    fillSync(comm, &a.sync);
    for (int p = 0; p < comm->nRanks; ++p) {
      char* base = (char*)dp->resWin->host.peerPtr[p];
      a.mailbox[p] = base + dp->offMailbox;
      a.llbox[p] = base + dp->offP2pLL;
      a.ready[p] = (uint32_t*)(base + kOffP2pReady);
      a.ack[p] = (uint32_t*)(base + kOffP2pAck);
    }
    a.seq[comm->rank] = dp->p2pSeq;
    a.nOps[comm->rank] = (int)nOps;
    a.opBase[comm->rank] = 0;
    for (int p = 0; p < comm->nRanks; ++p) a.rdv[p] = (void*)((char*)dp->resWin->host.peerPtr[p] + kOffP2pRdv);
    a.opDone[comm->rank] = dp->priv + kPrivP2pDone;
    a.winTable = paramP2pDirect() && comm->sym ? (void* const*)comm->sym->winTableDev : nullptr;
    int cta = 0;
    int perOpCap = std::max(1, std::min(dp->tune.sendrecvCtas, (int)(std::min(kMaxCtas, dp->smCount) / (int)nOps)));
    uint32_t posted[2][kMaxRanks] = {};   // chunks of earlier ops of this launch per direction and peer
    int large[2][kMaxRanks] = {};         // large operations so far per direction and peer: their rendezvous line
    for (size_t i = 0; i < nOps; ++i) {
      const Task& t = *remote[first + i];
      P2pOp& o = a.ops[i];
      o.peer = t.root;
      o.isSend = t.func == FUNC_SEND;
      o.buf = o.isSend ? (void*)t.send : t.recv;
      o.bytes = t.count * typeSize(t.type);
      const size_t cb = p2pChunkOf(o.bytes);
      size_t chunks = (o.bytes + cb - 1) / cb;
      o.ctaCount = (int)std::max<size_t>(1, std::min<size_t>(chunks, (size_t)perOpCap));
      o.rdvLine = -1;
      o.winSlot = -1;
      o.winOff = 0;
      if (a.winTable && o.bytes >= kP2pDirectMin) {
        // both sides count the pair's large operations of this launch the same way (operations match in posting order)
        int& ord = large[o.isSend ? 0 : 1][o.peer];
        if (ord < kP2pRdvLines) o.rdvLine = ord;
        ++ord;
        if (o.rdvLine >= 0 && !o.isSend) {
          SymWindow* w = symFindWindow(comm, o.buf, o.bytes);
          if (w && w->symmetric && w->slot >= 0) {
            o.winSlot = w->slot;
            o.winOff = (uintptr_t)o.buf - (uintptr_t)w->host.userPtr;
            o.ctaCount = 1;   // only waits: the sender writes straight into the buffer
          }
        }
      }
      o.ctaBegin = cta;
      cta += o.ctaCount;
      o.seqOffset = posted[o.isSend ? 0 : 1][o.peer];
      posted[o.isSend ? 0 : 1][o.peer] += (uint32_t)chunks;
    }
    dp->launches++;
    res = launchKernel(p2pKernelFn(), dim3(cta), dim3(kCtaThreads), 0, &a, stream, false, pdlFor(cta, false));
  }
out:
  if (cur != comm->cudaDev && cur >= 0) cudaSetDevice(cur);
  return res;
}

// Ring / tree schedules (NCCL_ALGO=Ring|Tree): always run in place on the staging area, which is
// symmetric, so any user buffer works; the copies in and out ride on the same stream.
ncclResult_t ringTreeRun(ncclComm* comm, const Task& t, int algo) {
  DevicePlane* dp = comm->devPlane;
  const int n = comm->nRanks, me = comm->rank;
  const size_t es = typeSize(t.type);
  DevOp op;
  NCCLCHECK(lowerOp(comm, t, &op));
  if (op.premul) return ncclInvalidUsage;
  if (algo == ALGO_TREE && t.func != FUNC_ALLREDUCE) algo = ALGO_RING;
  char* st = (char*)dp->resBase + dp->offStage;
  const bool blocks = t.func != FUNC_ALLREDUCE;          // stage holds n blocks of `piece` elements
  size_t cap = dp->stageBytes / es / (blocks ? n : 1);
  cap = cap / 64 * 64;
  for (size_t done = 0; done < t.count; done += cap) {
    const size_t cur = std::min(cap, t.count - done);
    if (t.func == FUNC_ALLREDUCE) {
      CUDACHECK(cudaMemcpyAsync(st, (const char*)t.send + done * es, cur * es, cudaMemcpyDeviceToDevice, t.stream));
    } else if (t.func == FUNC_REDUCESCATTER) {
      CUDACHECK(cudaMemcpy2DAsync(st, cur * es, (const char*)t.send + done * es, t.count * es, cur * es, n, cudaMemcpyDeviceToDevice, t.stream));
    } else {
      CUDACHECK(cudaMemcpyAsync(st + (size_t)me * cur * es, (const char*)t.send + done * es, cur * es, cudaMemcpyDeviceToDevice, t.stream));
    }
    CollArgs a;
    baseArgs(comm, &a, t.func);
    a.count = cur;
    a.scaleMode = op.scaleMode; a.scaleF = op.scaleF; a.scaleD = op.scaleD; a.intDiv = op.intDiv;
    Aliases W = stageAliases(comm, 0);
    for (int p = 0; p < n; ++p) a.recv[p] = W.peer[p];
    a.vec16 = !blocks || (cur * es) % 16 == 0;
    int ctas = clampCtas(comm, cur * es, dp->tune.p2pCtas);
    const void* fn = algo == ALGO_TREE ? treeKernelFn(t.type, op.red) : ringKernelFn(t.type, op.red);
    NCCLCHECK(launchColl(comm, fn, &a, ctas, t.stream, algo == ALGO_TREE ? "TREE" : "RING"));
    if (t.func == FUNC_ALLREDUCE) {
      CUDACHECK(cudaMemcpyAsync((char*)t.recv + done * es, st, cur * es, cudaMemcpyDeviceToDevice, t.stream));
    } else if (t.func == FUNC_REDUCESCATTER) {
      CUDACHECK(cudaMemcpyAsync((char*)t.recv + done * es, st + (size_t)me * cur * es, cur * es, cudaMemcpyDeviceToDevice, t.stream));
    } else {
      CUDACHECK(cudaMemcpy2DAsync((char*)t.recv + done * es, t.count * es, st, cur * es, cur * es, n, cudaMemcpyDeviceToDevice, t.stream));
    }
  }
  return ncclSuccess;
}

// Latency/bandwidth model used only for ncclGroupSimulateEnd (microseconds).
float devPlaneEstimateUs(ncclComm* comm, const Task& t) {
  const int n = comm->nRanks;
  const double bytes = (double)t.count * typeSize(t.type);
  if (n == 1) return (float)(2.0 + bytes / 3.0e6);
  const double linkGBs = comm->lsaAll ? 700.0 : 5.0;   // NVLink 5 through NVSwitch vs host sockets
  double lat = comm->lsaAll ? 6.0 : 60.0, moved = bytes;
  switch (t.func) {
    case FUNC_ALLREDUCE: moved = 2.0 * bytes * (n - 1) / n; lat = bytes <= 32768 ? 4.0 : 9.0; break;
    case FUNC_ALLGATHER: case FUNC_ALLTOALL: case FUNC_GATHER: moved = bytes * (n - 1); break;
    case FUNC_REDUCESCATTER: moved = bytes * (n - 1); break;
    default: break;
  }
  return (float)(lat + moved / (linkGBs * 1e3));
}

}  // namespace b200
