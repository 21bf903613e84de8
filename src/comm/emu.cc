// Single-GPU emulation of a multi-rank communicator, for unit tests of the kernels.
// One cooperative grid plays every rank (rank = blockIdx.y): the CTAs of all "ranks" are
// co-resident, so the cross-rank barriers, flagged lines and mailboxes run exactly the code of
// a real multi-GPU launch while every buffer lives on one device. (Separate launches per rank
// on one GPU would wait on each other without any guarantee of running at the same time.)
#include <algorithm>

#include "device_plane.h"

namespace b200 {

void sliceEven(size_t count, size_t es, int n, size_t* begin, size_t* cnt);

struct EmuCtx {
  int n = 0;
  char* sync[kMaxRanks] = {};      // per-rank sync page
  char* ll[kMaxRanks] = {};
  char* mailbox[kMaxRanks] = {};
  char* llbox[kMaxRanks] = {};
  uint32_t* priv[kMaxRanks] = {};  // epochs | llEpoch(4) | p2pSeq(2*kMaxRanks+4)
  uint32_t* status[kMaxRanks] = {};
  uint64_t timeoutNs = 5000000000ull;
};

static void fillSyncEmu(EmuCtx* e, SyncArgs* s) {
  memset(s, 0, sizeof(*s));
  for (int p = 0; p < e->n; ++p) {
    s->inbox[p] = (uint32_t*)e->sync[p];
    s->epoch[p] = e->priv[p];
    s->status[p] = e->status[p];
  }
  s->abortFlag = nullptr;
  s->timeoutNs = e->timeoutNs;
}

static int coopLaunch(const void* fn, int ctas, int n, void* args, int threads = kCtaThreads, size_t smem = 0) {
  if (!fn) return ncclInvalidUsage;
  int dev = 0, sms = 0, perSm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, fn, threads, smem);
  if (ctas * n > sms * std::max(perSm, 1)) { WARN("emulation: %d x %d CTAs cannot be co-resident", ctas, n); return ncclInvalidArgument; }
  ncclResult_t r = launchKernel(fn, dim3(ctas, n), dim3(threads), smem, args, 0, true);
  if (r != ncclSuccess) return r;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { WARN("emulation kernel failed: %s", cudaGetErrorString(e)); return ncclUnhandledCudaError; }
  return ncclSuccess;
}

}  // namespace b200

using namespace b200;

extern "C" {

void* b200EmuCreate(int nRanks, unsigned long long timeoutMs) {
  if (nRanks < 1 || nRanks > kMaxRanks) return nullptr;
  EmuCtx* e = new EmuCtx;
  e->n = nRanks;
  if (timeoutMs) e->timeoutNs = timeoutMs * 1000000ull;
  const size_t privWords = kPrivWords;
  for (int p = 0; p < nRanks; ++p) {
    bool ok = cudaMalloc(&e->sync[p], kSyncPageBytes) == cudaSuccess && cudaMalloc(&e->ll[p], kLLRegionBytes) == cudaSuccess &&
              cudaMalloc(&e->mailbox[p], kMailboxBytes) == cudaSuccess && cudaMalloc(&e->llbox[p], kP2pLLBytes) == cudaSuccess && cudaMalloc(&e->priv[p], privWords * 4) == cudaSuccess &&
              cudaMalloc(&e->status[p], 16) == cudaSuccess;
    if (!ok) { WARN("emulation: out of memory"); return nullptr; }
    cudaMemset(e->sync[p], 0, kSyncPageBytes);
    cudaMemset(e->ll[p], 0, kLLRegionBytes);
    cudaMemset(e->llbox[p], 0, kP2pLLBytes);
    cudaMemset(e->priv[p], 0, privWords * 4);
    cudaMemset(e->status[p], 0, 16);
  }
  cudaDeviceSynchronize();
  return e;
}

void b200EmuDestroy(void* ctx) {
  EmuCtx* e = (EmuCtx*)ctx;
  if (!e) return;
  for (int p = 0; p < e->n; ++p) { cudaFree(e->sync[p]); cudaFree(e->ll[p]); cudaFree(e->mailbox[p]); cudaFree(e->llbox[p]); cudaFree(e->priv[p]); cudaFree(e->status[p]); }
  delete e;
}

int b200EmuStatus(void* ctx, int rank, unsigned int* out4) {
  EmuCtx* e = (EmuCtx*)ctx;
  return cudaMemcpy(out4, e->status[rank], 16, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : 1;
}
int b200EmuClearStatus(void* ctx) {
  EmuCtx* e = (EmuCtx*)ctx;
  for (int p = 0; p < e->n; ++p) cudaMemset(e->status[p], 0, 16);
  return 0;
}

// kernel: KERNEL_REDUCE_P2P or KERNEL_ALLREDUCE_LL. func: all-reduce, reduce-scatter or reduce.
// op: ncclRedOp_t (sum, prod, max, min, avg). count: as in the public API of `func`.
int b200EmuReduce(void* ctx, int kernel, int func, int type, int op, size_t count, const void** send, void** recv, int root, int ctas) {
  EmuCtx* e = (EmuCtx*)ctx;
  const int n = e->n;
  const size_t es = typeSize((ncclDataType_t)type);
  CollArgs a;
  memset(&a, 0, sizeof(a));
  a.nRanks = n;
  a.emu = 1;
  a.func = func;
  a.root = root;
  fillSyncEmu(e, &a.sync);
  int red = op == ncclAvg ? RED_SUM : op;
  if (op == ncclAvg) {
    bool fl = type == ncclFloat16 || type == ncclFloat32 || type == ncclFloat64 || type == ncclBfloat16 || type == ncclFloat8e4m3 || type == ncclFloat8e5m2;
    if (fl) { a.scaleMode = SCALE_MUL; a.scaleF = 1.0f / n; a.scaleD = 1.0 / n; } else { a.scaleMode = SCALE_INTDIV; a.intDiv = n; }
  }
  bool v16 = true;
  for (int p = 0; p < n; ++p) {
    a.send[p] = send[p];
    a.recv[p] = recv[p];
    a.lsend[p] = send[p];
    a.lrecv[p] = recv[p];
    a.ll[p] = e->ll[p];
    a.llEpoch[p] = e->priv[p] + kBarrierSlots;
    if (((uintptr_t)send[p] & 15) || (recv[p] && ((uintptr_t)recv[p] & 15))) v16 = false;
  }
  if (kernel == KERNEL_ALLREDUCE_LL) {
    a.count = count;
  } else if (func == FUNC_ALLREDUCE) {
    sliceEven(count, es, n, a.sliceBegin, a.sliceCount);
    for (int r = 0; r < n; ++r) a.dstOff[r] = a.sliceBegin[r];
    a.dstAll = 1;
  } else if (func == FUNC_REDUCESCATTER) {
    for (int r = 0; r < n; ++r) { a.sliceBegin[r] = (size_t)r * count; a.sliceCount[r] = count; }
    if ((count * es) % 16) v16 = false;
  } else {
    for (int r = 0; r < n; ++r) a.sliceCount[r] = r == root ? count : 0;
  }
  a.vec16 = v16;
  return coopLaunch(reduceKernelFn(kernel, (ncclDataType_t)type, red), ctas, n, &a);
}

// Several all-reduces in one launch of the flagged-line kernel: item i reduces counts[i] elements found at byte offset
// sendOff[i] of every rank's sendBase and writes them at recvOff[i] of every rank's recvBase.
int b200EmuReduceBatch(void* ctx, int type, int op, int nItems, const size_t* counts, const size_t* sendOff, const size_t* recvOff,
                       const void** sendBase, void** recvBase, int ctas) {
  EmuCtx* e = (EmuCtx*)ctx;
  const int n = e->n;
  if (nItems < 1 || nItems > kMaxLLItems) return ncclInvalidArgument;
  const size_t es = typeSize((ncclDataType_t)type);
  LLBatchArgs b;
  memset(&b, 0, sizeof(b));
  CollArgs& a = b.c;
  a.nRanks = n;
  a.emu = 1;
  a.func = FUNC_ALLREDUCE;
  fillSyncEmu(e, &a.sync);
  int red = op == ncclAvg ? RED_SUM : op;
  if (op == ncclAvg) { a.scaleMode = SCALE_MUL; a.scaleF = 1.0f / n; a.scaleD = 1.0 / n; }
  for (int p = 0; p < n; ++p) {
    a.lsend[p] = sendBase[p];
    a.lrecv[p] = recvBase[p];
    a.ll[p] = e->ll[p];
    a.llEpoch[p] = e->priv[p] + kBarrierSlots;
  }
  uint32_t lines = 0;
  for (int i = 0; i < nItems; ++i) {
    b.items[i] = LLItem{(long long)sendOff[i], (long long)recvOff[i], (uint32_t)counts[i], lines};
    lines += (uint32_t)((counts[i] * es + 7) / 8);
  }
  if (lines > kLLLines - 1) return ncclInvalidArgument;
  b.nItems = nItems;
  b.totalLines = lines;
  return coopLaunch(llReduceBatchKernelFn((ncclDataType_t)type, red), ctas, n, &b);
}

// Copy collectives; bytes = size of one block (all-gather: per-rank contribution, ...).
int b200EmuCopy(void* ctx, int func, int mode, size_t bytes, const void** send, void** recv, int root, int ctas) {
  EmuCtx* e = (EmuCtx*)ctx;
  const int n = e->n;
  CollArgs a;
  memset(&a, 0, sizeof(a));
  a.nRanks = n;
  a.emu = 1;
  a.func = func;
  a.root = root;
  const bool bulk = mode >= 0 && mode != 3 && mode != 8 && (mode & MODE_BULK);
  a.mode = mode == 8 ? MODE_SPLIT : bulk ? (mode & ~MODE_BULK) : mode;   // 8: broadcast shared out among the non-root ranks
  a.count = bytes;
  a.sendStride = bytes;
  a.recvStride = bytes;
  fillSyncEmu(e, &a.sync);
  bool v16 = bytes % 16 == 0;
  for (int p = 0; p < n; ++p) {
    a.send[p] = send[p];
    a.recv[p] = recv[p];
    a.lsend[p] = send[p];
    a.lrecv[p] = recv[p];
    if (((uintptr_t)send[p] & 15) || ((uintptr_t)recv[p] & 15)) v16 = false;
  }
  a.vec16 = v16;
  if (mode == 3) {  // flagged lines
    for (int p = 0; p < n; ++p) { a.ll[p] = e->ll[p]; a.llEpoch[p] = e->priv[p] + kBarrierSlots; }
    return coopLaunch(llCopyKernelFn(), ctas, n, &a);
  }
  if (bulk) {
    if (!v16) return ncclInvalidArgument;
    if (cudaFuncSetAttribute(copyBulkKernelFn(), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)copyBulkSmemBytes()) != cudaSuccess) return ncclUnhandledCudaError;
    return coopLaunch(copyBulkKernelFn(), ctas, n, &a, 32, copyBulkSmemBytes());
  }
  return coopLaunch(copyKernelFn(), ctas, n, &a);
}

// Grouped send/recv: op i belongs to rank opRank[i]; ops of one rank must be listed together.
int b200EmuP2p(void* ctx, int nOps, const int* opRank, const int* peer, const int* isSend, void** buf, const size_t* bytes, int ctasPerOp) {
  EmuCtx* e = (EmuCtx*)ctx;
  const int n = e->n;
  if (nOps > kMaxP2pOps) return ncclInvalidArgument;
  P2pArgs a;
  memset(&a, 0, sizeof(a));
  a.nRanks = n;
  a.emu = 1;
  fillSyncEmu(e, &a.sync);
  for (int p = 0; p < n; ++p) {
    a.mailbox[p] = e->mailbox[p];
    a.llbox[p] = e->llbox[p];
    a.ready[p] = (uint32_t*)(e->sync[p] + kOffP2pReady);
    a.ack[p] = (uint32_t*)(e->sync[p] + kOffP2pAck);
    a.seq[p] = e->priv[p] + kBarrierSlots + 4;
    a.rdv[p] = (void*)(e->sync[p] + kOffP2pRdv);
    a.opDone[p] = e->priv[p] + kPrivP2pDone;
    a.opBase[p] = -1;
  }
  int maxCtas = 1;
  std::vector<int> nextCta(n, 0);
  std::vector<uint32_t> posted((size_t)n * 2 * kMaxRanks, 0);   // [rank][direction][peer] chunks so far
  for (int i = 0; i < nOps; ++i) {
    int r = opRank[i];
    if (a.opBase[r] < 0) a.opBase[r] = i;
    a.nOps[r]++;
    uint32_t& before = posted[((size_t)r * 2 + (isSend[i] ? 0 : 1)) * kMaxRanks + peer[i]];
    a.ops[i] = P2pOp{peer[i], isSend[i], buf[i], bytes[i], nextCta[r], ctasPerOp, before, -1, -1, 0};
    before += (uint32_t)((bytes[i] + p2pChunkOf(bytes[i]) - 1) / p2pChunkOf(bytes[i]));
    nextCta[r] += ctasPerOp;
    maxCtas = std::max(maxCtas, nextCta[r]);
  }
  for (int p = 0; p < n; ++p) if (a.opBase[p] < 0) a.opBase[p] = 0;
  return coopLaunch(p2pKernelFn(), maxCtas, n, &a);
}

}  // extern "C"

// Introspection used by the benchmarks and tests.
extern "C" unsigned long long b200CommLaunchCount(ncclComm_t comm) {
  return (commValid(comm) && comm->devPlane) ? comm->devPlane->launches : 0;
}
extern "C" int b200CommIsSymmetric(ncclComm_t comm) { return commValid(comm) && comm->lsaAll ? 1 : 0; }
extern "C" int b200CommHasMulticast(ncclComm_t comm) { return commValid(comm) && comm->sym && comm->sym->mcUsable ? 1 : 0; }

// Live tuning (sweeps): name is a TuningTable field; n selects the rank-count column of tables.
extern "C" int b200CommSetTuning(ncclComm_t comm, const char* name, int n, long long value) {
  if (!commValid(comm) || !comm->devPlane || n < 0 || n > kMaxRanks) return 1;
  TuningTable& t = comm->devPlane->tune;
  std::string k(name);
  if (k == "arLLMax") t.arLLMax[n] = (size_t)value;
  else if (k == "arNvlsMin") t.arNvlsMin[n] = (size_t)value;
  else if (k == "agMcMin") t.agMcMin[n] = (size_t)value;
  else if (k == "rsNvlsMin") t.rsNvlsMin[n] = (size_t)value;
  else if (k == "rsLLMax") t.rsLLMax[n] = (size_t)value;
  else if (k == "llCopyMax") t.llCopyMax[n] = (size_t)value;
  else if (k == "ceMin") t.ceMin = (size_t)value;
  else if (k == "nvlsCtas") t.nvlsCtas = (int)value;
  else if (k == "p2pCtas") t.p2pCtas = (int)value;
  else if (k == "copyCtas") t.copyCtas = (int)value;
  else if (k == "sendrecvCtas") t.sendrecvCtas = (int)value;
  else if (k == "bytesPerCta") t.bytesPerCta = (size_t)value;
  else if (k == "barrierMcMin") comm->devPlane->barrierMcMin = (int)value;
  else if (k == "llMcMin") comm->devPlane->llMcMin = (int)value;
  else return 2;
  return 0;
}
extern "C" void b200ForceAlgo(int algo, int mode) { devPlaneForce(algo, mode); }
