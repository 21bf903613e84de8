// User-buffer registration entry points and memory accounting.
//   ncclCommWindowRegister / Deregister / ncclWinGetUserPtr : symmetric windows (collective calls)
//   ncclCommRegister / Deregister : registration handle for buffers used repeatedly; here it is a
//       window registration as well, so later collectives on the buffer run without staging
//   ncclCommSuspend / Resume / MemStats : release and re-create the communicator's own device
//       memory (the resource window) around idle periods; user windows stay mapped
// Reference parity: src/dev_runtime.cc:1333-1401 (window API), src/register/register.cc
// (ncclCommRegister), src/mem_manager.cc:926-1010 (suspend / resume / stats).
#include "../comm/device_plane.h"
#include "symmetric.h"

using namespace b200;

static ncclResult_t gpuComm(ncclComm_t comm, const char* what) {
  if (!commValid(comm)) { WARN("%s : invalid communicator", what); return ncclInvalidArgument; }
  ncclResult_t r = commEnsureReady(comm);
  if (r != ncclSuccess) return r;
  if (comm->hostOnly) { WARN("%s : not available on host-memory communicators", what); return ncclInvalidUsage; }
  return ncclSuccess;
}

B200_PARAM(WinEnable, "WIN_ENABLE", 1, "0: ncclCommWindowRegister called by the application registers nothing and returns a null window (its buffers are then staged)")

namespace b200 {
// Window registration for the library's own needs (device communicators, ncclCommRegister): not subject to NCCL_WIN_ENABLE.
ncclResult_t windowRegister(ncclComm_t comm, void* buff, size_t size, ncclWindow_t* win, int winFlags);
}

extern "C" {

ncclResult_t ncclCommWindowRegister(ncclComm_t comm, void* buff, size_t size, ncclWindow_t* win, int winFlags) {
  if (!win) return ncclInvalidArgument;
  *win = nullptr;
  if (!paramWinEnable()) {
    NCCLCHECK(gpuComm(comm, "ncclCommWindowRegister"));
    return ncclSuccess;
  }
  return b200::windowRegister(comm, buff, size, win, winFlags);
}

}  // extern "C"

ncclResult_t b200::windowRegister(ncclComm_t comm, void* buff, size_t size, ncclWindow_t* win, int winFlags) {
  if (!win) return ncclInvalidArgument;
  *win = nullptr;
  NCCLCHECK(gpuComm(comm, "ncclCommWindowRegister"));
  if (!buff || size == 0) return ncclSuccess;   // a rank may contribute nothing
  if ((uintptr_t)buff % NCCL_WIN_REQUIRED_ALIGNMENT) { WARN("ncclCommWindowRegister : buffer %p is not %d-byte aligned", buff, NCCL_WIN_REQUIRED_ALIGNMENT); return ncclInvalidArgument; }
  if (comm->nRanks == 1 || !comm->sym) {
    // nothing to map: keep a local record so that the handle API still works
    SymWindow* w = new SymWindow;
    memset(&w->host, 0, sizeof(w->host));
    w->host.size = size;
    w->host.rank = comm->rank;
    w->host.nRanks = comm->nRanks;
    w->host.userPtr = buff;
    w->host.peerPtr[comm->rank % kMaxRanks] = buff;
    w->host.magic = kWindowMagic;
    w->host.hostState = w;
    w->flags = winFlags;
    ncclWindow_vidmem* dev = nullptr;
    CUDACHECK(cudaMalloc(&dev, sizeof(*dev)));
    w->host.devSelf = dev;
    CUDACHECK(cudaMemcpy(dev, &w->host, sizeof(*dev), cudaMemcpyHostToDevice));
    symWindowPublishHandle(w);
    *win = &w->host;
    return ncclSuccess;
  }
  int cur = -1;
  CUDACHECK(cudaGetDevice(&cur));
  if (cur != comm->cudaDev) CUDACHECK(cudaSetDevice(comm->cudaDev));
  SymWindow* w = nullptr;
  ncclResult_t r = symWindowRegister(comm, buff, size, &w, winFlags);
  if (cur != comm->cudaDev) cudaSetDevice(cur);
  NCCLCHECK(r);
  *win = &w->host;
  return ncclSuccess;
}

extern "C" {

ncclResult_t ncclCommWindowDeregister(ncclComm_t comm, ncclWindow_t win) {
  if (!win) return ncclSuccess;
  if (!commValid(comm)) return ncclInvalidArgument;
  if (win->magic != kWindowMagic) { WARN("ncclCommWindowDeregister : not a window handle"); return ncclInvalidArgument; }
  SymWindow* w = (SymWindow*)win->hostState;
  if (comm->nRanks == 1 || !comm->sym) {
    symWindowUnpublishHandle(w);
    if (w->host.devSelf) cudaFree(w->host.devSelf);
    delete w;
    return ncclSuccess;
  }
  return symWindowDeregister(comm, w);
}

ncclResult_t ncclWinGetUserPtr(ncclComm_t comm, ncclWindow_t win, void** outUserPtr) {
  if (!commValid(comm) || !outUserPtr) return ncclInvalidArgument;
  if (!win) { *outUserPtr = nullptr; return ncclSuccess; }
  if (win->magic != kWindowMagic) return ncclInvalidArgument;
  *outUserPtr = win->userPtr;
  return ncclSuccess;
}

ncclResult_t ncclCommRegister(const ncclComm_t comm, void* buff, size_t size, void** handle) {
  if (!handle) return ncclInvalidArgument;
  *handle = nullptr;
  NCCLCHECK(gpuComm(comm, "ncclCommRegister"));
  if (!buff || size == 0) return ncclSuccess;
  ncclWindow_t win = nullptr;
  // Registration is collective here as well: every rank registers its buffer in the same order,
  // which is how symmetric use of registered buffers is written anyway.
  uintptr_t base = (uintptr_t)buff & ~(uintptr_t)(NCCL_WIN_REQUIRED_ALIGNMENT - 1);
  NCCLCHECK(b200::windowRegister(comm, (void*)base, size + ((uintptr_t)buff - base), &win, NCCL_WIN_DEFAULT));
  *handle = win;
  return ncclSuccess;
}

ncclResult_t ncclCommDeregister(const ncclComm_t comm, void* handle) {
  if (!handle) return ncclSuccess;
  return ncclCommWindowDeregister(comm, (ncclWindow_t)handle);
}

ncclResult_t ncclCommSuspend(ncclComm_t comm, int flags) {
  NCCLCHECK(gpuComm(comm, "ncclCommSuspend"));
  if (!(flags & NCCL_SUSPEND_MEM)) { WARN("ncclCommSuspend : no known flag set"); return ncclInvalidArgument; }
  return memSuspend(comm);
}
ncclResult_t ncclCommResume(ncclComm_t comm) {
  NCCLCHECK(gpuComm(comm, "ncclCommResume"));
  return memResume(comm);
}
ncclResult_t ncclCommMemStats(ncclComm_t comm, ncclCommMemStat_t stat, uint64_t* value) {
  if (!commValid(comm) || !value) return ncclInvalidArgument;
  return memStats(comm, (int)stat, value);
}

ncclResult_t pncclCommWindowRegister(ncclComm_t c, void* b, size_t s, ncclWindow_t* w, int f) { return ncclCommWindowRegister(c, b, s, w, f); }
ncclResult_t pncclCommWindowDeregister(ncclComm_t c, ncclWindow_t w) { return ncclCommWindowDeregister(c, w); }
ncclResult_t pncclWinGetUserPtr(ncclComm_t c, ncclWindow_t w, void** p) { return ncclWinGetUserPtr(c, w, p); }
ncclResult_t pncclCommRegister(const ncclComm_t c, void* b, size_t s, void** h) { return ncclCommRegister(c, b, s, h); }
ncclResult_t pncclCommDeregister(const ncclComm_t c, void* h) { return ncclCommDeregister(c, h); }
ncclResult_t pncclCommSuspend(ncclComm_t c, int f) { return ncclCommSuspend(c, f); }
ncclResult_t pncclCommResume(ncclComm_t c) { return ncclCommResume(c); }
ncclResult_t pncclCommMemStats(ncclComm_t c, ncclCommMemStat_t s, uint64_t* v) { return ncclCommMemStats(c, s, v); }

}  // extern "C"
