// Window registration: exchange of allocation handles between the ranks of one host, peer
// mappings, multicast objects.
// Reference parity: src/dev_runtime.cc:212-479,545-951 (handle export/import over the proxy's
// Unix socket, LSA mappings, cuMulticast* team objects), src/transport/p2p.cc:220-324 (legacy
// cudaIpc import for memory that does not come from the virtual-memory API).
#include "symmetric.h"

#include <unistd.h>

#include <algorithm>

namespace b200 {

B200_PARAM(IpcTimeoutMs, "B200_IPC_TIMEOUT_MS", 60000, "Give up waiting for a peer's memory handle after this long")

struct RegDesc {
  int kind;
  int dev;
  uint64_t base;          // owner's address of the allocation (identifies the segment)
  uint64_t allocSize;
  uint64_t offset;        // window offset inside the allocation
  uint64_t winSize;
  uint64_t pidHash;
  cudaIpcMemHandle_t ipc;
};

ncclResult_t symInit(ncclComm* comm) {
  SymRuntime* s = new SymRuntime;
  s->comm = comm;
  const BootstrapRingData* peers = bootstrapPeers(comm->bootstrap);
  ncclResult_t r = ipcOpen(&s->ipc, peers[comm->rank].peerUDS);
  if (r != ncclSuccess) { delete s; return r; }
  bool mc = true, vmm = true;
  for (auto& p : comm->peers) { mc = mc && p.mcSupport; vmm = vmm && p.vmmSupport; }
  s->vmmUsable = vmm && comm->lsaAll;
  s->fabric = comm->mnnvl;   // the ranks span hosts: descriptors cannot travel over UNIX sockets, fabric handles are plain bytes
  s->mcUsable = mc && s->vmmUsable && comm->nRanks > 1;
  if (cudaMalloc(&s->winTableDev, (size_t)kMaxWinSlots * kMaxRanks * sizeof(void*)) != cudaSuccess ||
      cudaMemset(s->winTableDev, 0, (size_t)kMaxWinSlots * kMaxRanks * sizeof(void*)) != cudaSuccess) {
    (void)cudaGetLastError();
    s->winTableDev = nullptr;   // rendezvous send / receive stays off; everything else works
  }
  comm->sym = s;
  INFO(SUB_INIT, "symmetric runtime: vmm %d multicast %d", (int)s->vmmUsable, (int)s->mcUsable);
  return ncclSuccess;
}

static void releaseSegment(ncclComm* comm, SymSegment* seg) {
  const CuApi* cu = cuApi();
  int n = comm->nRanks, me = comm->rank;
  if (seg->mcBase && cu) {
    cu->cuMemUnmap((CUdeviceptr)seg->mcBase, seg->mcSize);
    cu->cuMemAddressFree((CUdeviceptr)seg->mcBase, seg->mcSize);
  }
  if (seg->mcHandle && cu) {
    if (seg->mcBound) {
      CUdevice d;
      if (cu->cuDeviceGet(&d, comm->cudaDev) == CUDA_SUCCESS) cu->cuMulticastUnbind(seg->mcHandle, d, 0, seg->mcSize);
    }
    cu->cuMemRelease(seg->mcHandle);
  }
  for (int p = 0; p < n; ++p) {
    if (p == me || !seg->peerBase[p]) continue;
    if (seg->kind == SEG_VMM && cu) {
      if (seg->peerHandle[p]) {
        cu->cuMemUnmap((CUdeviceptr)seg->peerBase[p], seg->peerSize[p]);
        cu->cuMemAddressFree((CUdeviceptr)seg->peerBase[p], seg->peerSize[p]);
        cu->cuMemRelease(seg->peerHandle[p]);
      }
    } else if (seg->kind == SEG_IPC && seg->peerIpcOpened[p]) {
      cudaIpcCloseMemHandle(seg->peerBase[p]);
    }
  }
  if (seg->ownHandleRetained && cu) cu->cuMemRelease(seg->ownHandle);
  delete seg;
}

void symDestroy(ncclComm* comm) {
  SymRuntime* s = comm->sym;
  if (!s) return;
  for (auto* w : s->windows) {
    symWindowUnpublishHandle(w);
    if (w->host.devSelf) cudaFree(w->host.devSelf);
    delete w;
  }
  for (auto* seg : s->segments) releaseSegment(comm, seg);
  if (s->winTableDev) cudaFree(s->winTableDev);
  ipcClose(&s->ipc);
  delete s;
  comm->sym = nullptr;
}

// A shareable form of an allocation handle: a file descriptor (one host; travels over UNIX sockets) or a fabric handle
// (64 plain bytes; travels over the bootstrap network, valid on every host of the NVLink fabric).
struct ShareHandle {
  int fd = -1;
  CUmemFabricHandle fabric = {};
};
static CUmemAllocationHandleType shareType(const SymRuntime* s) { return s->fabric ? CU_MEM_HANDLE_TYPE_FABRIC : CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR; }
static CUresult exportHandle(const SymRuntime* s, CUmemGenericAllocationHandle h, ShareHandle* out) {
  const CuApi* cu = cuApi();
  if (s->fabric) return cu->cuMemExportToShareableHandle(&out->fabric, h, CU_MEM_HANDLE_TYPE_FABRIC, 0);
  return cu->cuMemExportToShareableHandle(&out->fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
}
static CUresult importHandle(const SymRuntime* s, CUmemGenericAllocationHandle* h, const ShareHandle* in) {
  const CuApi* cu = cuApi();
  if (s->fabric) return cu->cuMemImportFromShareableHandle(h, (void*)&in->fabric, CU_MEM_HANDLE_TYPE_FABRIC);
  return cu->cuMemImportFromShareableHandle(h, (void*)(uintptr_t)in->fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
}
static void closeHandle(const SymRuntime* s, ShareHandle* h) {
  if (!s->fabric && h->fd >= 0) close(h->fd);
  h->fd = -1;
}

// Describes the allocation behind `buff` for the other ranks.
static void describeLocal(ncclComm* comm, void* buff, size_t size, RegDesc* d, CUmemGenericAllocationHandle* handle,
                          bool* retained) {
  memset(d, 0, sizeof(*d));
  d->dev = comm->cudaDev;
  d->winSize = size;
  d->pidHash = pidHash();
  *retained = false;
  const CuApi* cu = cuApi();
  MemAlloc m;
  if (memLookup(buff, &m)) {
    d->base = (uint64_t)m.ptr;
    d->allocSize = m.size;
    d->offset = (uintptr_t)buff - (uintptr_t)m.ptr;
    if (m.vmm && comm->sym->vmmUsable && m.handleType == (int)shareType(comm->sym)) {
      d->kind = SEG_VMM;
      *handle = m.handle;
      return;
    }
  } else if (cu) {
    CUdeviceptr base = 0;
    size_t asz = 0;
    if (cu->cuMemGetAddressRange(&base, &asz, (CUdeviceptr)buff) != CUDA_SUCCESS) return;
    d->base = base;
    d->allocSize = asz;
    d->offset = (uintptr_t)buff - (uintptr_t)base;
    // Memory created by somebody else's cuMemCreate can be shared when it carries a POSIX-fd handle
    // type; exporting tells (memory of cudaMalloc has no generic handle at all).
    if (comm->sym->vmmUsable && cu->cuMemRetainAllocationHandle(handle, (void*)base) == CUDA_SUCCESS) {
      ShareHandle sh;
      if (exportHandle(comm->sym, *handle, &sh) == CUDA_SUCCESS) {
        closeHandle(comm->sym, &sh);
        d->kind = SEG_VMM;
        *retained = true;
        return;
      }
      cu->cuMemRelease(*handle);
    }
  }
  if (!d->base || d->offset + size > d->allocSize) return;
  if (comm->sym->fabric) return;   // legacy handles do not cross hosts
  // legacy inter-process handle: works for cudaMalloc memory
  if (cudaIpcGetMemHandle(&d->ipc, (void*)d->base) == cudaSuccess) d->kind = SEG_IPC;
  else (void)cudaGetLastError();
}

static ncclResult_t mapPeerVmm(ncclComm* comm, SymSegment* seg, int p, const ShareHandle* sh, size_t allocSize) {
  const CuApi* cu = cuApi();
  CUmemGenericAllocationHandle h;
  CUCHECK(importHandle(comm->sym, &h, sh));
  size_t gran = shareableGranularity(comm->cudaDev);
  size_t mapSize = alignUp(allocSize, (size_t)(2 << 20));
  CUdeviceptr va = 0;
  CUresult r = cu->cuMemAddressReserve(&va, mapSize, gran, 0, 0);
  if (r != CUDA_SUCCESS) { cu->cuMemRelease(h); WARN("reserve for peer %d: %s", p, cuErrStr(r)); return ncclUnhandledCudaError; }
  r = cu->cuMemMap(va, allocSize, 0, h, 0);
  if (r != CUDA_SUCCESS) { cu->cuMemAddressFree(va, mapSize); cu->cuMemRelease(h); WARN("map peer %d: %s", p, cuErrStr(r)); return ncclUnhandledCudaError; }
  CUmemAccessDesc ad = {};
  ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  ad.location.id = comm->cudaDev;
  ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = cu->cuMemSetAccess(va, allocSize, &ad, 1);
  if (r != CUDA_SUCCESS) {
    cu->cuMemUnmap(va, allocSize); cu->cuMemAddressFree(va, mapSize); cu->cuMemRelease(h);
    WARN("access to peer %d memory: %s", p, cuErrStr(r));
    return ncclUnhandledCudaError;
  }
  seg->peerBase[p] = (void*)va;
  seg->peerSize[p] = allocSize;
  seg->peerHandle[p] = h;
  return ncclSuccess;
}

// Receives the next datagram carrying `tag`; datagrams of other stages that arrive early
// (a fast peer already sent its multicast handle) are parked.
static ncclResult_t recvTagged(ncclComm* comm, int tag, int* fd, IpcMsg* msg) {
  SymRuntime* s = comm->sym;
  for (size_t i = 0; i < s->stash.size(); ++i) {
    if (s->stash[i].first.tag == tag) {
      *msg = s->stash[i].first;
      *fd = s->stash[i].second;
      s->stash.erase(s->stash.begin() + i);
      return ncclSuccess;
    }
  }
  for (;;) {
    NCCLCHECK(ipcRecvFd(&s->ipc, fd, msg, comm->abortFlag, (int)paramIpcTimeoutMs()));
    if (msg->tag == tag) return ncclSuccess;
    s->stash.push_back({*msg, *fd});
  }
}

// Sends `fd` to every peer and collects one descriptor from each (any arrival order).
static ncclResult_t exchangeFds(ncclComm* comm, int tag, int myFd, uint64_t a, int* fds /* [nRanks] */) {
  SymRuntime* s = comm->sym;
  const BootstrapRingData* peers = bootstrapPeers(comm->bootstrap);
  int n = comm->nRanks, me = comm->rank;
  for (int p = 0; p < n; ++p) fds[p] = -1;
  for (int step = 1; step < n; ++step) {
    int to = (me + step) % n;
    NCCLCHECK(ipcSendFd(&s->ipc, peers[to].peerUDS, myFd, IpcMsg{me, tag, a, 0}));
  }
  for (int got = 0; got < n - 1; ++got) {
    IpcMsg msg;
    int fd = -1;
    NCCLCHECK(recvTagged(comm, tag, &fd, &msg));
    if (msg.srcRank < 0 || msg.srcRank >= n || fd < 0 || fds[msg.srcRank] >= 0) {
      WARN("symmetric: unexpected handle message (tag %d/%d from %d)", msg.tag, tag, msg.srcRank);
      if (fd >= 0) close(fd);
      return ncclInternalError;
    }
    fds[msg.srcRank] = fd;
  }
  return ncclSuccess;
}

// Every rank's shareable handle of its allocation, at every rank.
static ncclResult_t exchangeHandles(ncclComm* comm, int tag, const ShareHandle* mine, uint64_t a, ShareHandle* all /* [nRanks] */) {
  const int n = comm->nRanks, me = comm->rank;
  if (comm->sym->fabric) {
    std::vector<CUmemFabricHandle> fh(n);
    fh[me] = mine->fabric;
    NCCLCHECK(bootstrapAllGather(comm->bootstrap, fh.data(), sizeof(CUmemFabricHandle)));
    for (int p = 0; p < n; ++p) { all[p].fd = -1; all[p].fabric = fh[p]; }
    return ncclSuccess;
  }
  std::vector<int> fds(n, -1);
  NCCLCHECK(exchangeFds(comm, tag, mine->fd, a, fds.data()));
  for (int p = 0; p < n; ++p) all[p].fd = fds[p];
  return ncclSuccess;
}

static ncclResult_t setupMulticast(ncclComm* comm, SymSegment* seg, const RegDesc* all, int tag) {
  const CuApi* cu = cuApi();
  SymRuntime* s = comm->sym;
  const BootstrapRingData* peers = bootstrapPeers(comm->bootstrap);
  int n = comm->nRanks, me = comm->rank;
  size_t common = all[0].allocSize;
  for (int p = 1; p < n; ++p) common = std::min<size_t>(common, all[p].allocSize);
  CUmulticastObjectProp mp = {};
  mp.numDevices = n;
  mp.handleTypes = shareType(s);
  mp.size = common;
  size_t mg = 0;
  if (cu->cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) != CUDA_SUCCESS || mg == 0) return ncclSuccess;
  // all ranks take the same decision from the same gathered sizes
  if (common % mg != 0) { INFO(SUB_NVLS, "multicast skipped: common size %zu is not a multiple of %zu", common, mg); return ncclSuccess; }
  mp.size = common;
  int okLocal = 1;
  if (s->fabric) {
    // the object's fabric handle is plain bytes: rank 0's copy reaches everybody through one gather
    struct McMsg { int ok; CUmemFabricHandle h; };
    std::vector<McMsg> msgs(n);
    memset(msgs.data(), 0, n * sizeof(McMsg));
    if (me == 0) {
      CUresult r = cu->cuMulticastCreate(&seg->mcHandle, &mp);
      if (r == CUDA_SUCCESS) r = cu->cuMemExportToShareableHandle(&msgs[0].h, seg->mcHandle, CU_MEM_HANDLE_TYPE_FABRIC, 0);
      if (r != CUDA_SUCCESS) { INFO(SUB_NVLS, "multicast object creation failed: %s", cuErrStr(r)); okLocal = 0; }
      msgs[0].ok = okLocal;
    }
    NCCLCHECK(bootstrapAllGather(comm->bootstrap, msgs.data(), sizeof(McMsg)));
    if (me != 0) {
      if (!msgs[0].ok) okLocal = 0;
      else if (cu->cuMemImportFromShareableHandle(&seg->mcHandle, (void*)&msgs[0].h, CU_MEM_HANDLE_TYPE_FABRIC) != CUDA_SUCCESS) okLocal = 0;
    }
  } else if (me == 0) {
    CUresult r = cu->cuMulticastCreate(&seg->mcHandle, &mp);
    int fd = -1;
    if (r == CUDA_SUCCESS) r = cu->cuMemExportToShareableHandle(&fd, seg->mcHandle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) { INFO(SUB_NVLS, "multicast object creation failed: %s", cuErrStr(r)); okLocal = 0; }
    for (int p = 1; p < n; ++p) NCCLCHECK(ipcSendFd(&s->ipc, peers[p].peerUDS, okLocal ? fd : -1, IpcMsg{me, tag, (uint64_t)okLocal, 0}));
    if (fd >= 0) close(fd);
  } else {
    IpcMsg msg;
    int fd = -1;
    NCCLCHECK(recvTagged(comm, tag, &fd, &msg));
    if (msg.srcRank != 0) { WARN("symmetric: unexpected multicast message"); if (fd >= 0) close(fd); return ncclInternalError; }
    if (!msg.a || fd < 0) okLocal = 0;
    else if (cu->cuMemImportFromShareableHandle(&seg->mcHandle, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS) okLocal = 0;
    if (fd >= 0) close(fd);
  }
  CUdevice dev;
  CUCHECK(cu->cuDeviceGet(&dev, comm->cudaDev));
  if (okLocal && cu->cuMulticastAddDevice(seg->mcHandle, dev) != CUDA_SUCCESS) okLocal = 0;
  // every device must have joined before anyone binds memory; also agree on success
  std::vector<int> oks(n, 0);
  oks[me] = okLocal;
  NCCLCHECK(bootstrapAllGather(comm->bootstrap, oks.data(), sizeof(int)));
  bool allOk = true;
  for (int v : oks) allOk = allOk && v;
  if (allOk) {
    CUresult r = cu->cuMulticastBindMem(seg->mcHandle, 0, seg->ownHandle, 0, common, 0);
    if (r != CUDA_SUCCESS) { INFO(SUB_NVLS, "cuMulticastBindMem failed: %s", cuErrStr(r)); okLocal = 0; }
    else seg->mcBound = true;
    if (okLocal) {
      CUdeviceptr va = 0;
      size_t gran = std::max(mg, shareableGranularity(comm->cudaDev));
      r = cu->cuMemAddressReserve(&va, common, gran, 0, 0);
      if (r == CUDA_SUCCESS) {
        r = cu->cuMemMap(va, common, 0, seg->mcHandle, 0);
        if (r == CUDA_SUCCESS) {
          CUmemAccessDesc ad = {};
          ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
          ad.location.id = comm->cudaDev;
          ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
          r = cu->cuMemSetAccess(va, common, &ad, 1);
        }
        if (r != CUDA_SUCCESS) { cu->cuMemAddressFree(va, common); va = 0; }
      }
      if (r != CUDA_SUCCESS || !va) { INFO(SUB_NVLS, "multicast mapping failed: %s", cuErrStr(r)); okLocal = 0; }
      else { seg->mcBase = (void*)va; seg->mcSize = common; }
    }
    oks[me] = okLocal;
    NCCLCHECK(bootstrapAllGather(comm->bootstrap, oks.data(), sizeof(int)));
    for (int v : oks) allOk = allOk && v;
  }
  if (!allOk) {
    // somebody failed: nobody uses the multicast alias of this segment
    if (seg->mcBase) { cu->cuMemUnmap((CUdeviceptr)seg->mcBase, seg->mcSize); cu->cuMemAddressFree((CUdeviceptr)seg->mcBase, seg->mcSize); seg->mcBase = nullptr; }
    if (seg->mcHandle) {
      if (seg->mcBound) cu->cuMulticastUnbind(seg->mcHandle, dev, 0, common);
      cu->cuMemRelease(seg->mcHandle);
      seg->mcHandle = 0;
      seg->mcBound = false;
    }
    seg->mcSize = 0;
  } else {
    INFO(SUB_NVLS, "multicast alias of %zu bytes at %p", seg->mcSize, seg->mcBase);
  }
  return ncclSuccess;
}

ncclResult_t symWindowRegister(ncclComm* comm, void* buff, size_t size, SymWindow** out, int flags) {
  SymRuntime* s = comm->sym;
  if (!s) return ncclInvalidUsage;
  const int n = comm->nRanks, me = comm->rank;
  std::lock_guard<std::mutex> g(s->lock);
  RegDesc mine;
  CUmemGenericAllocationHandle myHandle = 0;
  bool retained = false;
  describeLocal(comm, buff, size, &mine, &myHandle, &retained);
  if (!comm->lsaAll) mine.kind = SEG_NONE;
  std::vector<RegDesc> all(n);
  all[me] = mine;
  NCCLCHECK(bootstrapAllGather(comm->bootstrap, all.data(), sizeof(RegDesc)));
  int kind = all[0].kind;
  for (int p = 0; p < n; ++p) if (all[p].kind != kind) kind = SEG_NONE;   // mixed kinds: local-only
  const int tag = ++s->regSeq;

  SymWindow* w = new SymWindow;
  w->flags = flags;
  w->offset = mine.offset;
  memset(&w->host, 0, sizeof(w->host));
  w->host.size = size;
  w->host.rank = me;
  w->host.nRanks = n;
  w->host.userPtr = buff;
  w->host.magic = kWindowMagic;
  w->host.hostState = w;
  w->host.peerPtr[me] = buff;

  if (kind != SEG_NONE && n > 1) {
    // reuse the mapping of this allocation when every rank presents the same allocation as before
    SymSegment* seg = nullptr;
    for (auto* c : s->segments) {
      bool same = c->kind == kind;
      for (int p = 0; p < n && same; ++p) same = c->peerBaseId[p] == all[p].base && c->peerSize[p] == all[p].allocSize;
      if (same) { seg = c; break; }
    }
    if (!seg) {
      seg = new SymSegment;
      seg->kind = kind;
      seg->base = mine.base;
      seg->size = mine.allocSize;
      seg->ownHandle = myHandle;
      seg->ownHandleRetained = retained;
      for (int p = 0; p < n; ++p) { seg->peerBaseId[p] = all[p].base; seg->peerSize[p] = all[p].allocSize; }
      seg->peerBase[me] = (void*)mine.base;
      ncclResult_t res = ncclSuccess;
      if (kind == SEG_VMM) {
        ShareHandle mySh;
        CUresult r = exportHandle(s, myHandle, &mySh);
        if (r != CUDA_SUCCESS) { WARN("export of window memory failed: %s", cuErrStr(r)); res = ncclUnhandledCudaError; }
        std::vector<ShareHandle> shs(n);
        // every rank takes part in the exchange even after a failed export (an invalid handle fails at the importer)
        if (res == ncclSuccess || s->fabric) { ncclResult_t xr = exchangeHandles(comm, 2 * tag, &mySh, mine.allocSize, shs.data()); if (res == ncclSuccess) res = xr; }
        closeHandle(s, &mySh);
        for (int p = 0; p < n; ++p) {
          if (p == me) continue;
          if (!s->fabric && shs[p].fd < 0) continue;
          if (res == ncclSuccess) res = mapPeerVmm(comm, seg, p, &shs[p], all[p].allocSize);
          closeHandle(s, &shs[p]);
        }
        if (res == ncclSuccess && s->mcUsable) res = setupMulticast(comm, seg, all.data(), 2 * tag + 1);
      } else {
        for (int p = 0; p < n && res == ncclSuccess; ++p) {
          if (p == me) continue;
          if (all[p].pidHash == mine.pidHash) {
            // same process: the pointer is valid here once peer access is on
            int cur = comm->cudaDev;
            cudaError_t e = cudaDeviceEnablePeerAccess(all[p].dev, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { WARN("peer access %d->%d: %s", cur, all[p].dev, cudaGetErrorString(e)); res = ncclUnhandledCudaError; }
            (void)cudaGetLastError();
            seg->peerBase[p] = (void*)all[p].base;
          } else {
            void* ptr = nullptr;
            cudaError_t e = cudaIpcOpenMemHandle(&ptr, all[p].ipc, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) { (void)cudaGetLastError(); WARN("cudaIpcOpenMemHandle(rank %d): %s", p, cudaGetErrorString(e)); res = ncclUnhandledCudaError; }
            else { seg->peerBase[p] = ptr; seg->peerIpcOpened[p] = true; }
          }
        }
      }
      if (res != ncclSuccess) { releaseSegment(comm, seg); delete w; return res; }
      s->segments.push_back(seg);
    } else if (retained) {
      cuApi()->cuMemRelease(myHandle);  // the cached segment already holds one reference
    }
    seg->refs++;
    w->seg = seg;
    w->symmetric = true;
    bool sameOffsets = true;
    for (int p = 0; p < n; ++p) {
      w->host.peerPtr[p] = (char*)seg->peerBase[p] + all[p].offset;
      sameOffsets = sameOffsets && all[p].offset == mine.offset;
    }
    w->host.peerPtr[me] = buff;
    if (seg->mcBase && sameOffsets && mine.offset + size <= seg->mcSize) w->host.mcPtr = (char*)seg->mcBase + mine.offset;
  } else if (retained) {
    cuApi()->cuMemRelease(myHandle);
  }
  // device copy for kernels that take a window handle
  ncclWindow_vidmem* dev = nullptr;
  if (cudaMalloc(&dev, sizeof(ncclWindow_vidmem)) != cudaSuccess) { (void)cudaGetLastError(); delete w; return ncclUnhandledCudaError; }
  w->host.devSelf = dev;
  cudaMemcpy(dev, &w->host, sizeof(ncclWindow_vidmem), cudaMemcpyHostToDevice);
  symWindowPublishHandle(w);
  s->windows.push_back(w);
  if (w->symmetric && s->winTableDev) {
    for (int i = 0; i < kMaxWinSlots; ++i)
      if (!s->slotUsed[i]) { w->slot = i; s->slotUsed[i] = true; break; }
    if (w->slot >= 0) {
      void* row[kMaxRanks] = {};
      for (int p = 0; p < n; ++p) row[p] = w->host.peerPtr[p];
      if (cudaMemcpy(s->winTableDev + (size_t)w->slot * kMaxRanks, row, sizeof(row), cudaMemcpyHostToDevice) != cudaSuccess) {
        (void)cudaGetLastError();
        s->slotUsed[w->slot] = false;
        w->slot = -1;
      }
    }
  }
  INFO(SUB_REG, "window %p size %zu: %s%s", buff, size, w->symmetric ? (kind == SEG_VMM ? "symmetric (vmm)" : "symmetric (ipc)") : "local only",
       w->host.mcPtr ? " + multicast" : "");
  *out = w;
  return ncclSuccess;
}

void symWindowPublishHandle(SymWindow* w) {
  int dev = 0, same = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&same, cudaDevAttrCanUseHostPointerForRegisteredMem, dev) != cudaSuccess || !same) {
    (void)cudaGetLastError();
    return;
  }
  if (cudaHostRegister(&w->host, sizeof(w->host), cudaHostRegisterPortable | cudaHostRegisterMapped) == cudaSuccess) w->hostMapped = true;
  else (void)cudaGetLastError();   // the host handle then works on the host only; kernels use devSelf
}

void symWindowUnpublishHandle(SymWindow* w) {
  if (!w->hostMapped) return;
  if (cudaHostUnregister(&w->host) != cudaSuccess) (void)cudaGetLastError();
  w->hostMapped = false;
}

ncclResult_t symWindowDeregister(ncclComm* comm, SymWindow* win) {
  SymRuntime* s = comm->sym;
  if (!s || !win) return ncclInvalidArgument;
  std::lock_guard<std::mutex> g(s->lock);
  auto it = std::find(s->windows.begin(), s->windows.end(), win);
  if (it == s->windows.end()) return ncclInvalidArgument;
  s->windows.erase(it);
  if (win->slot >= 0) {
    cudaDeviceSynchronize();   // no kernel may still resolve addresses through this row
    cudaMemset(s->winTableDev + (size_t)win->slot * kMaxRanks, 0, kMaxRanks * sizeof(void*));
    s->slotUsed[win->slot] = false;
    win->slot = -1;
  }
  if (win->seg && --win->seg->refs == 0) {
    auto sit = std::find(s->segments.begin(), s->segments.end(), win->seg);
    if (sit != s->segments.end()) s->segments.erase(sit);
    // peers may still be reading through their own mappings; those are theirs to release
    cudaDeviceSynchronize();
    releaseSegment(comm, win->seg);
  }
  symWindowUnpublishHandle(win);
  if (win->host.devSelf) cudaFree(win->host.devSelf);
  delete win;
  return ncclSuccess;
}

SymWindow* symFindWindow(ncclComm* comm, const void* ptr, size_t bytes) {
  SymRuntime* s = comm->sym;
  if (!s) return nullptr;
  std::lock_guard<std::mutex> g(s->lock);
  for (auto* w : s->windows) {
    uintptr_t b = (uintptr_t)w->host.userPtr;
    if ((uintptr_t)ptr >= b && (uintptr_t)ptr + bytes <= b + w->host.size) return w;
  }
  return nullptr;
}

}  // namespace b200
