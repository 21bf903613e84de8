// Host side of expert-parallel dispatch / combine: groups (symmetric landing zones), handles
// (routing of one batch), launches, and a single-GPU emulation used by the unit tests.
// Reference parity: contrib/nccl_ep/nccl_ep.cc (ncclEpCreateGroup :1223, handles :1904-2408,
// ncclEpDispatch :2410, ncclEpCombine :2984, ncclEpComplete :3413, error API :3430-3545).
#include "nccl_ep.h"

#include <algorithm>

#include "../comm/device_plane.h"
#include "ep_kernels.cuh"

using namespace b200;

struct ncclEpGroup {
  ncclComm* comm = nullptr;
  ncclEpGroupConfig_t cfg;
  int n = 1, E = 0, El = 0, H = 0, maxTokens = 0, K = 0;
  size_t slotBytes = 0, zoneBytes = 0, combZoneBytes = 0;
  char* recvZone = nullptr;           // 2 zones (epoch parity)
  SymWindow* recvWin = nullptr;
  char* ctl = nullptr;                // counts [2][El][n] u64, combine flags [n] u64
  SymWindow* ctlWin = nullptr;
  char* combZone = nullptr;           // 2 zones, allocated with the first handle (needs top-k)
  SymWindow* combWin = nullptr;
  uint32_t* state = nullptr;
  uint32_t* mask = nullptr;           // [n] device words: non-zero = that rank is left out of dispatch / combine
  int smCount = 0;
  int lastError = 0;
  int layoutClass = 0;                // 0 none yet, 1 expert-major, 2 per-rank (rank-major / flat)
};

// Buffers that only this rank touches come from the group's allocator hooks when the configuration gives them
// (ncclEpGroupConfig_t::alloc); memory that peers map stays with the library's own allocator, which makes it exportable.
static cudaError_t epAlloc(const ncclEpAllocConfig_t& a, void** p, size_t bytes) {
  if (a.alloc_fn) return a.alloc_fn(p, bytes, a.context);
  return cudaMalloc(p, bytes);
}
static void epFree(const ncclEpAllocConfig_t& a, void* p) {
  if (!p) return;
  if (a.alloc_fn) a.free_fn(p, a.context);
  else cudaFree(p);
}

struct ncclEpHandle {
  ncclEpGroup* g = nullptr;
  ncclEpLayout_t layout;
  int K = 0, T = 0;
  int outSlots = 0;                   // flat layout: rows of the last dispatch's outputs
  const int64_t* topkIdx = nullptr;
  const float* topkW = nullptr;
  int2* srcInfo = nullptr;
  int* expertCount = nullptr;
  ncclEpAllocConfig_t alloc = {};     // the group's hooks, kept here so that a handle can outlive its group's record
  // a send_only call leaves its receiving half to ncclEpComplete
  int pending = 0;                    // 0 nothing, 1 dispatch, 2 combine
  EpArgs pendingArgs;
  int pendingCtas = 0;
  size_t pendingSmem = 0;
  void* pendingCounters = nullptr;    // layout_info->expert_counters of the pending dispatch
};

static bool cfgOk(const void* p) {
  const unsigned int* u = (const unsigned int*)p;
  return p && u[1] == NCCL_EP_MAGIC;
}
static bool tensorOk(const ncclEpTensor_t* t, unsigned ndim) {
  return t && t->magic == NCCL_EP_TENSOR_MAGIC && t->ndim == ndim && t->data && t->sizes;
}

static size_t ctlBytes(int El, int n) { return ((size_t)2 * El * n + n) * sizeof(unsigned long long); }

static void fillEpArgs(ncclEpGroup* g, EpArgs* a) {
  memset(a, 0, sizeof(*a));
  ncclComm* comm = g->comm;
  a->rank = comm->rank;
  a->nRanks = g->n;
  a->numExperts = g->E;
  a->expertsPerRank = g->El;
  a->hidden = g->H;
  a->maxTokens = g->maxTokens;
  for (int p = 0; p < g->n; ++p) {
    char* rz = g->n > 1 ? (char*)g->recvWin->host.peerPtr[p] : g->recvZone;
    char* cz = g->n > 1 ? (char*)g->ctlWin->host.peerPtr[p] : g->ctl;
    a->recvBuf[p] = rz;
    a->recvCount[p] = (unsigned long long*)cz;
    a->combFlag[p] = (unsigned long long*)cz + (size_t)2 * g->El * g->n;
    if (g->combZone) a->combBuf[p] = g->n > 1 ? (char*)g->combWin->host.peerPtr[p] : g->combZone;
  }
  a->state[comm->rank] = g->state;
  a->mask[comm->rank] = g->mask;
  a->enableMask = g->cfg.enable_mask ? 1 : 0;
  a->phases = 3;
  a->sync.status[comm->rank] = comm->devStatusDev;
  a->sync.abortFlag = comm->abortFlagDev;
  a->sync.timeoutNs = g->cfg.timeout_ns ? g->cfg.timeout_ns : (comm->devPlane ? comm->devPlane->timeoutNs : 5000000000ull);
}

static ncclResult_t launchEp(const void* fn, EpArgs* a, int ctas, int ranksY, size_t smem, cudaStream_t stream, bool coop) {
  // the attribute is per device and cheap to set: no process-wide "done once" flag
  if (smem > 40000) CUDACHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  return launchKernel(fn, dim3(ctas, ranksY), dim3(512), smem, a, stream, coop);
}

B200_PARAM(EpBulk, "B200_EP_BULK", 1, "Expert-parallel dispatch hands the packed tokens to the bulk-copy engines (a ring of shared-memory stages per CTA) instead of storing them with the warps: 0 never, 1 for the expert-major layout, 2 for every layout")

// Dynamic shared memory of the dispatch kernel: one packed token, or the ring of stages of the bulk form.
static size_t dispatchSmem(int H, int fp8, int bulkStages = 0) {
  if (bulkStages > 0) return 128 + (size_t)bulkStages * epStageBytes(H, fp8);
  return 128 + (fp8 ? (size_t)H + (size_t)(H / 128) * 4 + 16 : (size_t)H * 2);
}

extern "C" {

ncclResult_t ncclEpGetVersion(int* version) {
  if (!version) return ncclInvalidArgument;
  *version = NCCL_EP_VERSION_CODE;
  return ncclSuccess;
}

ncclResult_t ncclEpTensorAlloc(ncclEpTensor_t** tensor, unsigned int ndim, ncclDataType_t datatype, const size_t* sizes, const ncclEpTensorAllocConfig_t* config) {
  if (!tensor || !sizes || ndim == 0 || ndim > 8) return ncclInvalidArgument;
  if (config && !cfgOk(config)) return ncclInvalidArgument;
  ncclEpTensor_t* t = new ncclEpTensor_t;
  t->size = sizeof(*t);
  t->magic = NCCL_EP_TENSOR_MAGIC;
  t->ndim = ndim;
  t->datatype = datatype;
  t->win_hdl = nullptr;
  t->win_offset = 0;
  t->sizes = new size_t[ndim];
  size_t bytes = typeSize(datatype);
  for (unsigned i = 0; i < ndim; ++i) { t->sizes[i] = sizes[i]; bytes *= sizes[i]; }
  t->data = nullptr;
  if (cudaMalloc(&t->data, std::max<size_t>(bytes, 16)) != cudaSuccess) { (void)cudaGetLastError(); delete[] t->sizes; delete t; return ncclUnhandledCudaError; }
  *tensor = t;
  return ncclSuccess;
}

ncclResult_t ncclEpTensorDestroy(ncclEpTensor_t* t) {
  if (!t) return ncclSuccess;
  if (t->magic != NCCL_EP_TENSOR_MAGIC) return ncclInvalidArgument;
  if (t->data) cudaFree(t->data);
  delete[] t->sizes;
  delete t;
  return ncclSuccess;
}

ncclResult_t ncclEpCreateGroup(ncclEpGroup_t* out, ncclComm_t comm, const ncclEpGroupConfig_t* cfg) {
  if (!out) return ncclInvalidArgument;
  *out = nullptr;
  if (!commValid(comm) || comm->hostOnly) { WARN("ncclEpCreateGroup needs a GPU communicator"); return ncclInvalidArgument; }
  if (!cfgOk(cfg)) { WARN("ncclEpCreateGroup: configuration was not initialised"); return ncclInvalidArgument; }
  NCCLCHECK(commEnsureReady(comm));
  const int n = comm->nRanks;
  if (n > 1 && !comm->lsaAll) { WARN("ncclEpCreateGroup: ranks must be able to map each other's memory"); return ncclInvalidUsage; }
  if (cfg->num_experts == 0 || cfg->num_experts % n) { WARN("ncclEpCreateGroup: %u experts do not divide over %d ranks", cfg->num_experts, n); return ncclInvalidArgument; }
  if (cfg->max_token_bytes == 0 || (cfg->max_token_bytes / 2) % 128) { WARN("ncclEpCreateGroup: hidden size must be a multiple of 128"); return ncclInvalidArgument; }
  if (cfg->max_dispatch_tokens_per_rank == 0) return ncclInvalidArgument;
  if ((cfg->alloc.alloc_fn == nullptr) != (cfg->alloc.free_fn == nullptr)) { WARN("ncclEpCreateGroup: alloc_fn and free_fn come as a pair"); return ncclInvalidArgument; }
  if ((int)cfg->num_experts / n > kEpMaxLocalExperts) { WARN("ncclEpCreateGroup: at most %d experts per rank", kEpMaxLocalExperts); return ncclInvalidArgument; }
  ncclEpGroup* g = new ncclEpGroup;
  g->comm = comm;
  g->cfg = *cfg;
  g->n = n;
  g->E = (int)cfg->num_experts;
  g->El = g->E / n;
  g->H = (int)cfg->max_token_bytes / 2;
  g->maxTokens = (int)cfg->max_dispatch_tokens_per_rank;
  g->slotBytes = epSlotBytes(g->H, 0);   // sized for the larger (bf16) payload
  // one zone holds either layout: per expert and source (expert-major) or per source with the routing row appended (rank-major, flat)
  g->zoneBytes = (size_t)n * g->maxTokens * std::max((size_t)g->El * g->slotBytes, g->slotBytes + epMetaBytes(16));
  int cur = -1;
  CUDACHECK(cudaGetDevice(&cur));
  if (cur != comm->cudaDev) CUDACHECK(cudaSetDevice(comm->cudaDev));
  CUDACHECK(cudaDeviceGetAttribute(&g->smCount, cudaDevAttrMultiProcessorCount, comm->cudaDev));
  NCCLCHECK(memAlloc((void**)&g->recvZone, 2 * g->zoneBytes, comm->cudaDev));
  NCCLCHECK(memAlloc((void**)&g->ctl, ctlBytes(g->El, n), comm->cudaDev));
  CUDACHECK(cudaMemset(g->ctl, 0, ctlBytes(g->El, n)));
  CUDACHECK(cudaMemset(g->recvZone, 0, 2 * g->zoneBytes));   // rank-major rows are recognised by the epoch in their header: none is valid yet
  CUDACHECK(epAlloc(g->cfg.alloc, (void**)&g->state, (8 + g->E) * sizeof(uint32_t)));
  CUDACHECK(cudaMemset(g->state, 0, (8 + g->E) * sizeof(uint32_t)));
  CUDACHECK(epAlloc(g->cfg.alloc, (void**)&g->mask, kMaxRanks * sizeof(uint32_t)));
  CUDACHECK(cudaMemset(g->mask, 0, kMaxRanks * sizeof(uint32_t)));
  CUDACHECK(cudaDeviceSynchronize());
  if (n > 1) {
    NCCLCHECK(symWindowRegister(comm, g->recvZone, 2 * g->zoneBytes, &g->recvWin, NCCL_WIN_COLL_SYMMETRIC));
    NCCLCHECK(symWindowRegister(comm, g->ctl, ctlBytes(g->El, n), &g->ctlWin, NCCL_WIN_COLL_SYMMETRIC));
    if (!g->recvWin->symmetric || !g->ctlWin->symmetric) { WARN("ncclEpCreateGroup: windows could not be mapped by the peers"); return ncclInternalError; }
    NCCLCHECK(bootstrapBarrier(comm->bootstrap));
  }
  // landing zones and flags are working memory: a suspended communicator gives them back; flags and epochs restart together
  memTrack(comm, g->recvZone, 2 * g->zoneBytes, MEM_SCRATCH, "expert-parallel landing zones", n > 1 ? &g->recvWin : nullptr, NCCL_WIN_COLL_SYMMETRIC,
           2 * g->zoneBytes);
  memTrack(comm, g->ctl, ctlBytes(g->El, n), MEM_SCRATCH, "expert-parallel counts and flags", n > 1 ? &g->ctlWin : nullptr, NCCL_WIN_COLL_SYMMETRIC,
           ctlBytes(g->El, n), [g] { cudaMemset(g->state, 0, (8 + g->E) * sizeof(uint32_t)); });
  memTrack(comm, g->state, (8 + g->E) * sizeof(uint32_t), MEM_PERSIST, "expert-parallel epochs");
  if (cur != comm->cudaDev) cudaSetDevice(cur);
  *out = g;
  return ncclSuccess;
}

ncclResult_t ncclEpGroupDestroy(ncclEpGroup_t g) {
  if (!g) return ncclSuccess;
  cudaDeviceSynchronize();
  memUntrack(g->comm, g->recvZone);
  memUntrack(g->comm, g->ctl);
  memUntrack(g->comm, g->state);
  if (g->combZone) memUntrack(g->comm, g->combZone);
  if (g->recvWin) symWindowDeregister(g->comm, g->recvWin);
  if (g->ctlWin) symWindowDeregister(g->comm, g->ctlWin);
  if (g->combWin) symWindowDeregister(g->comm, g->combWin);
  if (g->recvZone) memFree(g->recvZone);
  if (g->ctl) memFree(g->ctl);
  if (g->combZone) memFree(g->combZone);
  epFree(g->cfg.alloc, g->state);
  epFree(g->cfg.alloc, g->mask);
  delete g;
  return ncclSuccess;
}

ncclResult_t ncclEpHandleMemSize(ncclEpGroup_t g, ncclEpLayout_t, const ncclEpHandleConfig_t*, size_t* size_out, int) {
  if (!g || !size_out) return ncclInvalidArgument;
  *size_out = (size_t)g->El * g->n * g->maxTokens * sizeof(int2) + (size_t)g->El * sizeof(int);
  return ncclSuccess;
}

ncclResult_t ncclEpInitHandle(ncclEpHandle_t* out, ncclEpGroup_t g, ncclEpLayout_t layout, const ncclEpHandleConfig_t* config, int num_topk, const ncclEpTensor_t*) {
  if (!out || !g || num_topk <= 0 || num_topk > 16) return ncclInvalidArgument;
  if (config && !cfgOk(config)) return ncclInvalidArgument;
  if (layout == NCCL_EP_LAYOUT_UNSET) layout = NCCL_EP_LAYOUT_EXPERT_MAJOR;
  if (layout != NCCL_EP_LAYOUT_EXPERT_MAJOR && layout != NCCL_EP_LAYOUT_RANK_MAJOR && layout != NCCL_EP_LAYOUT_FLAT) return ncclInvalidArgument;
  // The landing zones are laid out per layout class, and the per-rank layouts recognise a used row by the epoch in its
  // header: rows of the other class left in the zone could be mistaken for one. One class per group.
  const int cls = layout == NCCL_EP_LAYOUT_EXPERT_MAJOR ? 1 : 2;
  if (g->layoutClass && g->layoutClass != cls) {
    WARN("ncclEp: a group serves either expert-major handles or rank-major / flat handles, not both (create a second group)");
    return ncclInvalidUsage;
  }
  g->layoutClass = cls;
  if (g->K == 0) {
    // first handle: the combine landing zones depend on top-k (collective, like every handle creation); a row per
    // selected expert (expert-major) or per rank (rank-major, flat), whichever is more
    g->K = num_topk;
    g->combZoneBytes = (size_t)g->maxTokens * std::max(num_topk, g->n) * g->H * 2;
    NCCLCHECK(memAlloc((void**)&g->combZone, 2 * g->combZoneBytes, g->comm->cudaDev));
    if (g->n > 1) {
      NCCLCHECK(symWindowRegister(g->comm, g->combZone, 2 * g->combZoneBytes, &g->combWin, NCCL_WIN_COLL_SYMMETRIC));
      if (!g->combWin->symmetric) return ncclInternalError;
    }
    memTrack(g->comm, g->combZone, 2 * g->combZoneBytes, MEM_SCRATCH, "expert-parallel combine zones", g->n > 1 ? &g->combWin : nullptr, NCCL_WIN_COLL_SYMMETRIC);
  } else if (g->K != num_topk) {
    WARN("ncclEp: all handles of a group must use the same top-k (%d, got %d)", g->K, num_topk);
    return ncclInvalidUsage;
  }
  ncclEpHandle* h = new ncclEpHandle;
  h->g = g;
  h->layout = layout;
  h->K = num_topk;
  h->alloc = g->cfg.alloc;
  const size_t cap = (size_t)g->n * g->maxTokens;
  CUDACHECK(epAlloc(h->alloc, (void**)&h->srcInfo, (size_t)g->El * cap * sizeof(int2)));
  CUDACHECK(epAlloc(h->alloc, (void**)&h->expertCount, (size_t)g->El * sizeof(int)));
  CUDACHECK(cudaMemset(h->expertCount, 0, (size_t)g->El * sizeof(int)));
  *out = h;
  return ncclSuccess;
}

ncclResult_t ncclEpUpdateHandle(ncclEpHandle_t h, const ncclEpTensor_t* topk_idx, const ncclEpLayoutInfo_t*, cudaStream_t) {
  if (!h || !tensorOk(topk_idx, 2)) return ncclInvalidArgument;
  if (topk_idx->datatype != ncclInt64) { WARN("ncclEp: topk_idx must be int64"); return ncclInvalidArgument; }
  if ((int)topk_idx->sizes[1] != h->K) { WARN("ncclEp: topk_idx has %zu columns, the handle was made for top-%d", topk_idx->sizes[1], h->K); return ncclInvalidArgument; }
  if ((int)topk_idx->sizes[0] > h->g->maxTokens) { WARN("ncclEp: %zu tokens exceed max_dispatch_tokens_per_rank", topk_idx->sizes[0]); return ncclInvalidArgument; }
  h->T = (int)topk_idx->sizes[0];
  h->topkIdx = (const int64_t*)topk_idx->data;
  return ncclSuccess;
}

ncclResult_t ncclEpCreateHandle(ncclEpHandle_t* out, ncclEpGroup_t g, ncclEpLayout_t layout, const ncclEpTensor_t* topk_idx, const ncclEpLayoutInfo_t* li,
                                const ncclEpHandleConfig_t* config, cudaStream_t stream) {
  if (!tensorOk(topk_idx, 2)) return ncclInvalidArgument;
  NCCLCHECK(ncclEpInitHandle(out, g, layout, config, (int)topk_idx->sizes[1], nullptr));
  return ncclEpUpdateHandle(*out, topk_idx, li, stream);
}

ncclResult_t ncclEpHandleDestroy(ncclEpHandle_t h) {
  if (!h) return ncclSuccess;
  cudaDeviceSynchronize();
  epFree(h->alloc, h->srcInfo);
  epFree(h->alloc, h->expertCount);
  delete h;
  return ncclSuccess;
}

ncclResult_t ncclEpDispatch(ncclEpHandle_t h, const ncclEpDispatchInputs_t* in, const ncclEpDispatchOutputs_t* out, const ncclEpLayoutInfo_t* li,
                            const ncclEpDispatchConfig_t* config, cudaStream_t stream) {
  if (!h || !cfgOk(in) || !cfgOk(out)) return ncclInvalidArgument;
  if (config && !cfgOk(config)) return ncclInvalidArgument;
  ncclEpGroup* g = h->g;
  NCCLCHECK(devPlaneCheckStatus(g->comm));
  if (!h->topkIdx) { WARN("ncclEpDispatch: the handle has no routing (ncclEpUpdateHandle)"); return ncclInvalidUsage; }
  if (!tensorOk(in->tokens, 2) || in->tokens->datatype != ncclBfloat16 || (int)in->tokens->sizes[1] != g->H || (int)in->tokens->sizes[0] != h->T) {
    WARN("ncclEpDispatch: input tokens must be bf16 [%d, %d]", h->T, g->H);
    return ncclInvalidArgument;
  }
  const bool fp8 = out->scales != nullptr;
  const size_t cap = (size_t)g->n * g->maxTokens;
  const ncclDataType_t tokType = fp8 ? ncclFloat8e4m3 : ncclBfloat16;
  size_t outRows = cap;
  if (h->layout == NCCL_EP_LAYOUT_EXPERT_MAJOR) {
    if (!tensorOk(out->tokens, 3) || (int)out->tokens->sizes[0] != g->El || out->tokens->sizes[1] != cap || (int)out->tokens->sizes[2] != g->H || out->tokens->datatype != tokType) {
      WARN("ncclEpDispatch: output tokens must be %s [%d, %zu, %d] (local experts, capacity, hidden)", fp8 ? "fp8 e4m3" : "bf16", g->El, cap, g->H);
      return ncclInvalidArgument;
    }
  } else if (h->layout == NCCL_EP_LAYOUT_RANK_MAJOR) {
    if (!tensorOk(out->tokens, 3) || (int)out->tokens->sizes[0] != g->n || (int)out->tokens->sizes[1] != g->maxTokens || (int)out->tokens->sizes[2] != g->H || out->tokens->datatype != tokType) {
      WARN("ncclEpDispatch: output tokens must be %s [%d, %d, %d] (ranks, max tokens per rank, hidden)", fp8 ? "fp8 e4m3" : "bf16", g->n, g->maxTokens, g->H);
      return ncclInvalidArgument;
    }
  } else {
    if (!tensorOk(out->tokens, 2) || out->tokens->sizes[0] == 0 || (int)out->tokens->sizes[1] != g->H || out->tokens->datatype != tokType) {
      WARN("ncclEpDispatch: output tokens must be %s [receive slots, %d]", fp8 ? "fp8 e4m3" : "bf16", g->H);
      return ncclInvalidArgument;
    }
    outRows = std::min(cap, out->tokens->sizes[0]);
  }
  long long* outIdx = nullptr;
  float* outW = nullptr;
  if (h->layout != NCCL_EP_LAYOUT_EXPERT_MAJOR) {
    // the routing row of every received token comes with it: [rows, top-k] (rank-major: [ranks, max tokens, top-k])
    const unsigned nd = h->layout == NCCL_EP_LAYOUT_RANK_MAJOR ? 3 : 2;
    auto rowsOf = [&](const ncclEpTensor_t* t) { return nd == 3 ? t->sizes[0] * t->sizes[1] : t->sizes[0]; };
    if (!tensorOk(out->topk_idx, nd) || out->topk_idx->datatype != ncclInt64 || rowsOf(out->topk_idx) < outRows || (int)out->topk_idx->sizes[nd - 1] != h->K) {
      WARN("ncclEpDispatch: this layout needs an int64 topk_idx output with %zu rows of %d", outRows, h->K);
      return ncclInvalidArgument;
    }
    outIdx = (long long*)out->topk_idx->data;
    if (out->topk_weights) {
      if (!tensorOk(out->topk_weights, nd) || out->topk_weights->datatype != ncclFloat32 || rowsOf(out->topk_weights) < outRows || (int)out->topk_weights->sizes[nd - 1] != h->K) return ncclInvalidArgument;
      outW = (float*)out->topk_weights->data;
    }
  }
  if (fp8 && (!out->scales || out->scales->magic != NCCL_EP_TENSOR_MAGIC || !out->scales->data || out->scales->datatype != ncclFloat32)) return ncclInvalidArgument;
  if (in->topk_weights) {
    if (!tensorOk(in->topk_weights, 2) || in->topk_weights->datatype != ncclFloat32) return ncclInvalidArgument;
    h->topkW = (const float*)in->topk_weights->data;
  }
  EpArgs a;
  fillEpArgs(g, &a);
  const int me = g->comm->rank;
  a.topk = h->K;
  a.fp8 = fp8;
  a.numTokens[me] = h->T;
  a.x[me] = (const __nv_bfloat16*)in->tokens->data;
  a.topkIdx[me] = h->topkIdx;
  a.topkW[me] = h->topkW;
  a.outTokens[me] = out->tokens->data;
  a.outScales[me] = fp8 ? (float*)out->scales->data : nullptr;
  a.expertCount[me] = h->expertCount;
  a.srcInfo[me] = h->srcInfo;
  a.layout = h->layout == NCCL_EP_LAYOUT_RANK_MAJOR ? EP_RANK_MAJOR : h->layout == NCCL_EP_LAYOUT_FLAT ? EP_FLAT : EP_EXPERT_MAJOR;
  // the rank-major / flat forms measured slower through the bulk engines (one lane per destination writes the routing rows)
  a.bulkStages = (paramEpBulk() == 1 && a.layout == EP_EXPERT_MAJOR) || paramEpBulk() == 2 ? kEpBulkStages : 0;
  a.outSlots = (int)outRows;
  a.outTopkIdx[me] = outIdx;
  a.outTopkW[me] = outW;
  a.recvTotal[me] = (li && li->recv_total_counter && li->recv_total_counter->data) ? (int*)li->recv_total_counter->data : nullptr;
  h->outSlots = (int)outRows;
  int ctas = g->cfg.max_num_sms ? (int)std::min<unsigned>(g->cfg.max_num_sms, (unsigned)g->smCount) : g->smCount;
  if (h->pending) { WARN("ncclEpDispatch: a send_only call on this handle is still waiting for ncclEpComplete"); return ncclInvalidUsage; }
  const bool sendOnly = config && config->send_only;
  if (sendOnly) a.phases = 1;
  // the per-rank layouts count the tokens of every local expert with atomics while they unpack: start from zero
  if (a.layout != EP_EXPERT_MAJOR && !sendOnly) CUDACHECK(cudaMemsetAsync(h->expertCount, 0, (size_t)g->El * sizeof(int), stream));
  NCCLCHECK(launchEp(epDispatchKernelFn(), &a, ctas, 1, dispatchSmem(g->H, fp8, a.bulkStages), stream, false));
  if (g->comm->devPlane) g->comm->devPlane->launches++;
  void* counters = (li && li->expert_counters && li->expert_counters->data) ? li->expert_counters->data : nullptr;
  if (sendOnly) {
    // tokens and counts are on their way; the receiving half (wait, pack) runs when ncclEpComplete is called
    h->pending = 1;
    h->pendingArgs = a;
    h->pendingArgs.phases = 2;
    h->pendingCtas = ctas;
    h->pendingSmem = dispatchSmem(g->H, fp8, a.bulkStages);
    h->pendingCounters = counters;
    return ncclSuccess;
  }
  if (counters) CUDACHECK(cudaMemcpyAsync(counters, h->expertCount, (size_t)g->El * sizeof(int), cudaMemcpyDeviceToDevice, stream));
  return ncclSuccess;
}

ncclResult_t ncclEpCombine(ncclEpHandle_t h, const ncclEpCombineInputs_t* in, const ncclEpCombineOutputs_t* out, const ncclEpCombineConfig_t* config, cudaStream_t stream) {
  if (!h || !cfgOk(in) || !cfgOk(out)) return ncclInvalidArgument;
  if (config && !cfgOk(config)) return ncclInvalidArgument;
  ncclEpGroup* g = h->g;
  NCCLCHECK(devPlaneCheckStatus(g->comm));
  const size_t cap = (size_t)g->n * g->maxTokens;
  if (h->layout == NCCL_EP_LAYOUT_EXPERT_MAJOR) {
    if (!tensorOk(in->tokens, 3) || in->tokens->datatype != ncclBfloat16 || (int)in->tokens->sizes[0] != g->El || in->tokens->sizes[1] != cap || (int)in->tokens->sizes[2] != g->H) {
      WARN("ncclEpCombine: input tokens must be bf16 [%d, %zu, %d]", g->El, cap, g->H);
      return ncclInvalidArgument;
    }
  } else if (h->layout == NCCL_EP_LAYOUT_RANK_MAJOR) {
    if (!tensorOk(in->tokens, 3) || in->tokens->datatype != ncclBfloat16 || (int)in->tokens->sizes[0] != g->n || (int)in->tokens->sizes[1] != g->maxTokens || (int)in->tokens->sizes[2] != g->H) {
      WARN("ncclEpCombine: input tokens must be bf16 [%d, %d, %d]", g->n, g->maxTokens, g->H);
      return ncclInvalidArgument;
    }
  } else {
    if (!tensorOk(in->tokens, 2) || in->tokens->datatype != ncclBfloat16 || (int)in->tokens->sizes[0] < h->outSlots || (int)in->tokens->sizes[1] != g->H) {
      WARN("ncclEpCombine: input tokens must be bf16 [>= %d, %d] (the rows of the dispatch output)", h->outSlots, g->H);
      return ncclInvalidArgument;
    }
  }
  if (!tensorOk(out->tokens, 2) || out->tokens->datatype != ncclBfloat16 || (int)out->tokens->sizes[0] != h->T || (int)out->tokens->sizes[1] != g->H) {
    WARN("ncclEpCombine: output tokens must be bf16 [%d, %d]", h->T, g->H);
    return ncclInvalidArgument;
  }
  const float* weights = h->topkW;
  if (in->topk_weights && in->topk_weights->data) weights = (const float*)in->topk_weights->data;
  // the per-rank layouts return rows that the caller has already weighted
  if (!weights && h->layout == NCCL_EP_LAYOUT_EXPERT_MAJOR) { WARN("ncclEpCombine: no top-k weights were given (dispatch inputs or combine inputs)"); return ncclInvalidUsage; }
  EpArgs a;
  fillEpArgs(g, &a);
  const int me = g->comm->rank;
  a.topk = h->K;
  a.numTokens[me] = h->T;
  a.x[me] = (const __nv_bfloat16*)in->tokens->data;
  a.topkIdx[me] = h->topkIdx;
  a.topkW[me] = weights;
  a.outTokens[me] = out->tokens->data;
  a.expertCount[me] = h->expertCount;
  a.srcInfo[me] = h->srcInfo;
  a.layout = h->layout == NCCL_EP_LAYOUT_RANK_MAJOR ? EP_RANK_MAJOR : h->layout == NCCL_EP_LAYOUT_FLAT ? EP_FLAT : EP_EXPERT_MAJOR;
  a.outSlots = h->outSlots;
  int ctas = g->cfg.max_num_sms ? (int)std::min<unsigned>(g->cfg.max_num_sms, (unsigned)g->smCount) : g->smCount;
  if (h->pending) { WARN("ncclEpCombine: a send_only call on this handle is still waiting for ncclEpComplete"); return ncclInvalidUsage; }
  const bool sendOnly = config && config->send_only;
  if (sendOnly) a.phases = 1;
  NCCLCHECK(launchEp(epCombineKernelFn(), &a, ctas, 1, 0, stream, false));
  if (g->comm->devPlane) g->comm->devPlane->launches++;
  if (sendOnly) {
    h->pending = 2;
    h->pendingArgs = a;
    h->pendingArgs.phases = 2;
    h->pendingCtas = ctas;
    h->pendingSmem = 0;
  }
  return ncclSuccess;
}

// Runs the receiving half that a send_only dispatch / combine left open: the sends were issued by the earlier
// call, so whatever the caller queued in between (for example the previous layer's expert GEMMs) overlapped them.
// Reference parity: contrib/nccl_ep/nccl_ep.cc:3413.
ncclResult_t ncclEpComplete(ncclEpHandle_t h, const ncclEpCompleteConfig_t* config, cudaStream_t stream) {
  if (!h) return ncclInvalidArgument;
  if (config && !cfgOk(config)) return ncclInvalidArgument;
  if (!h->pending) return ncclSuccess;
  ncclEpGroup* g = h->g;
  NCCLCHECK(devPlaneCheckStatus(g->comm));
  const void* fn = h->pending == 1 ? epDispatchKernelFn() : epCombineKernelFn();
  if (h->pending == 1 && h->pendingArgs.layout != EP_EXPERT_MAJOR) CUDACHECK(cudaMemsetAsync(h->expertCount, 0, (size_t)g->El * sizeof(int), stream));
  NCCLCHECK(launchEp(fn, &h->pendingArgs, h->pendingCtas, 1, h->pendingSmem, stream, false));
  if (g->comm->devPlane) g->comm->devPlane->launches++;
  if (h->pending == 1 && h->pendingCounters)
    CUDACHECK(cudaMemcpyAsync(h->pendingCounters, h->expertCount, (size_t)g->El * sizeof(int), cudaMemcpyDeviceToDevice, stream));
  h->pending = 0;
  return ncclSuccess;
}

// Rank masks: a masked rank receives nothing and nobody waits for it. With enable_mask in the group
// configuration a wait on a rank that runs out (timeout_ns) sets that rank's mask word on the waiting rank
// instead of failing the call; ncclEpMaskQuery shows the words, ncclEpMaskUpdate sets them (for example after a
// health check excluded a rank everywhere), ncclEpMaskClean clears them.
// Reference parity: contrib/nccl_ep/nccl_ep.cc:3430-3545.
ncclResult_t ncclEpMaskQuery(ncclEpGroup_t g, int* mask_status, cudaStream_t stream) {
  if (!g || !mask_status) return ncclInvalidArgument;
  uint32_t host[kMaxRanks] = {};
  CUDACHECK(cudaMemcpyAsync(host, g->mask, g->n * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
  CUDACHECK(cudaStreamSynchronize(stream));
  for (int r = 0; r < g->n; ++r) mask_status[r] = host[r] ? 1 : 0;
  return ncclSuccess;
}
ncclResult_t ncclEpMaskUpdate(ncclEpGroup_t g, const int* mask, cudaStream_t stream) {
  if (!g || !mask) return ncclInvalidArgument;
  if (mask[g->comm->rank]) { WARN("ncclEpMaskUpdate: a rank cannot leave itself out"); return ncclInvalidArgument; }
  uint32_t host[kMaxRanks] = {};
  for (int r = 0; r < g->n; ++r) host[r] = mask[r] ? 1u : 0u;
  CUDACHECK(cudaMemcpyAsync(g->mask, host, g->n * sizeof(uint32_t), cudaMemcpyHostToDevice, stream));
  CUDACHECK(cudaStreamSynchronize(stream));   // `host` is on this stack frame
  return ncclSuccess;
}
ncclResult_t ncclEpMaskClean(ncclEpGroup_t g, cudaStream_t stream) {
  if (!g) return ncclInvalidArgument;
  CUDACHECK(cudaMemsetAsync(g->mask, 0, kMaxRanks * sizeof(uint32_t), stream));
  return ncclSuccess;
}

ncclResult_t ncclEpGetAsyncError(ncclEpGroup_t g, int* error_out) {
  if (!g || !error_out) return ncclInvalidArgument;
  ncclResult_t r = devPlaneCheckStatus(g->comm);
  if (r != ncclSuccess) g->lastError = (int)r;
  *error_out = g->lastError;
  return ncclSuccess;
}
ncclResult_t ncclEpErrorClear(ncclEpGroup_t g) {
  if (!g) return ncclInvalidArgument;
  g->lastError = 0;
  if (g->comm->devStatus) for (int i = 0; i < 4; ++i) g->comm->devStatus[i] = 0;
  return ncclSuccess;
}

// --------------------------------------------------------------------------- single-GPU emulation
struct EpEmu {
  int n, E, El, K, H, maxTokens;
  char* recv[kMaxRanks];
  char* ctl[kMaxRanks];
  char* comb[kMaxRanks];
  uint32_t* state[kMaxRanks];
  uint32_t* status[kMaxRanks];
  int2* srcInfo[kMaxRanks];
  int* counts[kMaxRanks];
  uint32_t* mask[kMaxRanks];
  int phases = 3, enableMask = 0;
  int layout = 0;
  int bulk = -1;                      // -1: as the parameter says
  long long* outIdx[kMaxRanks];
  float* outW[kMaxRanks];
  const float* inW[kMaxRanks];
  unsigned absent = 0;
  unsigned long long timeoutNs = 3000000000ull;
};

void* b200EpEmuCreate(int n, int E, int K, int H, int maxTokens) {
  if (n < 1 || n > kMaxRanks || E % n || H % 128 || E / n > kEpMaxLocalExperts) return nullptr;
  EpEmu* e = new EpEmu;
  memset(e, 0, sizeof(*e));
  e->n = n; e->E = E; e->El = E / n; e->K = K; e->H = H; e->maxTokens = maxTokens;
  e->phases = 3;
  e->bulk = -1;
  e->timeoutNs = 3000000000ull;
  size_t zone = (size_t)n * maxTokens * std::max((size_t)e->El * epSlotBytes(H, 0), epSlotBytes(H, 0) + epMetaBytes(16));
  size_t comb = (size_t)maxTokens * std::max(K, n) * H * 2;
  for (int r = 0; r < n; ++r) {
    bool ok = cudaMalloc(&e->recv[r], 2 * zone) == cudaSuccess && cudaMalloc(&e->ctl[r], ctlBytes(e->El, n)) == cudaSuccess &&
              cudaMalloc(&e->comb[r], 2 * comb) == cudaSuccess && cudaMalloc(&e->state[r], (8 + E) * 4) == cudaSuccess &&
              cudaMalloc(&e->status[r], 16) == cudaSuccess && cudaMalloc(&e->srcInfo[r], (size_t)e->El * n * maxTokens * sizeof(int2)) == cudaSuccess &&
              cudaMalloc(&e->counts[r], e->El * sizeof(int)) == cudaSuccess && cudaMalloc(&e->mask[r], kMaxRanks * 4) == cudaSuccess;
    if (!ok) return nullptr;
    cudaMemset(e->recv[r], 0, 2 * zone);
    cudaMemset(e->mask[r], 0, kMaxRanks * 4);
    cudaMemset(e->counts[r], 0, e->El * sizeof(int));
    cudaMemset(e->ctl[r], 0, ctlBytes(e->El, n));
    cudaMemset(e->state[r], 0, (8 + E) * 4);
    cudaMemset(e->status[r], 0, 16);
  }
  cudaDeviceSynchronize();
  return e;
}
void b200EpEmuDestroy(void* ctx) {
  EpEmu* e = (EpEmu*)ctx;
  if (!e) return;
  for (int r = 0; r < e->n; ++r) { cudaFree(e->recv[r]); cudaFree(e->ctl[r]); cudaFree(e->comb[r]); cudaFree(e->state[r]); cudaFree(e->status[r]); cudaFree(e->srcInfo[r]); cudaFree(e->counts[r]); cudaFree(e->mask[r]); }
  delete e;
}
static void emuArgs(EpEmu* e, EpArgs* a) {
  memset(a, 0, sizeof(*a));
  a->nRanks = e->n; a->emu = 1; a->numExperts = e->E; a->expertsPerRank = e->El; a->topk = e->K; a->hidden = e->H; a->maxTokens = e->maxTokens;
  for (int r = 0; r < e->n; ++r) {
    a->recvBuf[r] = e->recv[r];
    a->recvCount[r] = (unsigned long long*)e->ctl[r];
    a->combFlag[r] = (unsigned long long*)e->ctl[r] + (size_t)2 * e->El * e->n;
    a->combBuf[r] = e->comb[r];
    a->state[r] = e->state[r];
    a->sync.status[r] = e->status[r];
    a->srcInfo[r] = e->srcInfo[r];
    a->expertCount[r] = e->counts[r];
    a->mask[r] = e->mask[r];
  }
  a->phases = e->phases;
  a->enableMask = e->enableMask;
  a->absent = e->absent;
  a->layout = e->layout;
  a->bulkStages = (e->bulk < 0 ? ((paramEpBulk() == 1 && e->layout == EP_EXPERT_MAJOR) || paramEpBulk() == 2) : e->bulk != 0) ? kEpBulkStages : 0;
  a->outSlots = e->n * e->maxTokens;
  for (int r = 0; r < e->n; ++r) { a->outTopkIdx[r] = e->outIdx[r]; a->outTopkW[r] = e->outW[r]; a->topkW[r] = e->inW[r]; }
  a->sync.timeoutNs = e->timeoutNs;
}
// Settings of the following emulated calls: which halves run (1 send, 2 receive, 3 both), which ranks never show up
// (bit mask), whether waits that run out mask the rank instead of failing, and the budget of one wait.
int b200EpEmuSet(void* ctx, int phases, unsigned absent, int enableMask, unsigned long long timeoutMs) {
  EpEmu* e = (EpEmu*)ctx;
  if (!e || phases < 1 || phases > 3) return ncclInvalidArgument;
  e->phases = phases;
  e->absent = absent;
  e->enableMask = enableMask;
  if (timeoutMs) e->timeoutNs = timeoutMs * 1000000ull;
  return 0;
}
// Layout of the following emulated calls (0 expert-major, 1 rank-major, 2 flat) with, for the per-rank layouts, every
// rank's outputs for the routing rows ([rows, top-k] int64 and fp32) and the weights that travel with the tokens.
int b200EpEmuLayout(void* ctx, int layout, void** outIdx, void** outW, void** inW) {
  EpEmu* e = (EpEmu*)ctx;
  if (!e || layout < 0 || layout > 2) return ncclInvalidArgument;
  e->layout = layout;
  for (int r = 0; r < e->n; ++r) {
    e->outIdx[r] = outIdx ? (long long*)outIdx[r] : nullptr;
    e->outW[r] = outW ? (float*)outW[r] : nullptr;
    e->inW[r] = inW ? (const float*)inW[r] : nullptr;
  }
  return 0;
}
// 1 / 0: the following emulated dispatches use / do not use the bulk-copy engines; -1: as NCCL_B200_EP_BULK says.
int b200EpEmuBulk(void* ctx, int bulk) {
  EpEmu* e = (EpEmu*)ctx;
  if (!e) return ncclInvalidArgument;
  e->bulk = bulk;
  return 0;
}
int b200EpEmuMask(void* ctx, int rank, unsigned int* out) {
  EpEmu* e = (EpEmu*)ctx;
  return cudaMemcpy(out, e->mask[rank], e->n * 4, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : 1;
}
int b200EpEmuClear(void* ctx) {
  EpEmu* e = (EpEmu*)ctx;
  for (int r = 0; r < e->n; ++r) { cudaMemset(e->mask[r], 0, kMaxRanks * 4); cudaMemset(e->status[r], 0, 16); }
  return 0;
}
int b200EpEmuDispatch(void* ctx, int fp8, const int* numTokens, void** x, void** idx, void** outTokens, void** outScales, int** countsOut, int ctas) {
  EpEmu* e = (EpEmu*)ctx;
  EpArgs a;
  emuArgs(e, &a);
  a.fp8 = fp8;
  for (int r = 0; r < e->n; ++r) {
    a.numTokens[r] = numTokens[r];
    a.x[r] = (const __nv_bfloat16*)x[r];
    a.topkIdx[r] = (const int64_t*)idx[r];
    a.outTokens[r] = outTokens[r];
    a.outScales[r] = outScales ? (float*)outScales[r] : nullptr;
  }
  if (a.layout != EP_EXPERT_MAJOR && (a.phases & 2))
    for (int r = 0; r < e->n; ++r) cudaMemset(e->counts[r], 0, e->El * sizeof(int));
  ncclResult_t res = launchEp(epDispatchKernelFn(), &a, ctas, e->n, dispatchSmem(e->H, fp8, a.bulkStages), 0, true);
  if (res != ncclSuccess) return res;
  if (cudaDeviceSynchronize() != cudaSuccess) return ncclUnhandledCudaError;
  for (int r = 0; r < e->n; ++r) cudaMemcpy(countsOut[r], e->counts[r], e->El * sizeof(int), cudaMemcpyDeviceToHost);
  uint32_t st = 0;
  for (int r = 0; r < e->n; ++r) { cudaMemcpy(&st, e->status[r], 4, cudaMemcpyDeviceToHost); if (st) return ncclTimeout; }
  return 0;
}
int b200EpEmuCombine(void* ctx, const int* numTokens, void** y, void** idx, void** weights, void** out, int ctas) {
  EpEmu* e = (EpEmu*)ctx;
  EpArgs a;
  emuArgs(e, &a);
  for (int r = 0; r < e->n; ++r) {
    a.numTokens[r] = numTokens[r];
    a.x[r] = (const __nv_bfloat16*)y[r];
    a.topkIdx[r] = (const int64_t*)idx[r];
    a.topkW[r] = weights ? (const float*)weights[r] : nullptr;
    a.outTokens[r] = out[r];
  }
  ncclResult_t res = launchEp(epCombineKernelFn(), &a, ctas, e->n, 0, 0, true);
  if (res != ncclSuccess) return res;
  if (cudaDeviceSynchronize() != cudaSuccess) return ncclUnhandledCudaError;
  uint32_t st = 0;
  for (int r = 0; r < e->n; ++r) { cudaMemcpy(&st, e->status[r], 4, cudaMemcpyDeviceToHost); if (st) return ncclTimeout; }
  return 0;
}

}  // extern "C"
