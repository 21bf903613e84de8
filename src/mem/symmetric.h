// Symmetric-memory runtime: registered windows whose memory every rank of the load/store domain
// can address (peer mappings) and, when the fabric supports it, a multicast alias that reaches
// all ranks with one multimem instruction.
// Reference parity: src/dev_runtime.cc (symMemoryObtain :545-656, symMemoryMapLsaTeam :294-340,
// multicast team :342-479, symWindowCreate :712-789), src/register/register.cc.
#pragma once
#include "../comm/comm.h"
#include "../core/ipcsocket.h"
#include "../kernels/args.h"
#include "allocator.h"

// ncclWindow_vidmem (what ncclWindow_t points to, on the host and on the device) is part of the public device API.
#include "nccl_device/core.h"
static_assert(NCCL_DEVICE_MAX_LSA == b200::kMaxRanks, "window peer table and kernel rank limit must agree");

namespace b200 {

constexpr unsigned long long kWindowMagic = 0x57494e42323030ull;

enum SegKind : int { SEG_NONE = 0, SEG_VMM = 1, SEG_IPC = 2 };

struct SymSegment {
  int kind = SEG_NONE;
  uintptr_t base = 0;
  size_t size = 0;
  CUmemGenericAllocationHandle ownHandle = 0;
  bool ownHandleRetained = false;
  uintptr_t peerBaseId[kMaxRanks] = {};         // peers' own base addresses (cache key)
  void* peerBase[kMaxRanks] = {};               // local mapping of peer p's allocation
  size_t peerSize[kMaxRanks] = {};
  CUmemGenericAllocationHandle peerHandle[kMaxRanks] = {};
  bool peerIpcOpened[kMaxRanks] = {};
  void* mcBase = nullptr;
  size_t mcSize = 0;
  CUmemGenericAllocationHandle mcHandle = 0;
  bool mcBound = false;
  int refs = 0;
};

// Page-aligned and page-sized so that `host` can be pinned and mapped for device access on its own:
// the handle ncclCommWindowRegister returns (&host) is then valid inside kernels too, as the
// reference's window handles are; host.devSelf is the copy in device memory that kernels read faster.
struct alignas(4096) SymWindow {
  ncclWindow_vidmem host;          // host mirror (host.devSelf = device copy)
  bool hostMapped = false;         // `host` is registered with the CUDA driver (cudaHostRegister)
  SymSegment* seg = nullptr;
  size_t offset = 0;               // offset of the window inside my allocation
  int flags = 0;
  bool symmetric = false;          // peers are mapped; false = local-only registration
  int slot = -1;                   // row of this window in the device-side table of peer mappings (same on every rank), -1: none
};

void symWindowPublishHandle(SymWindow* w);     // after `host` is complete: make &w->host readable from kernels
void symWindowUnpublishHandle(SymWindow* w);   // before the object is freed

struct SymRuntime {
  ncclComm* comm = nullptr;
  IpcSocket ipc;
  bool mcUsable = false;           // every rank supports multicast
  bool vmmUsable = false;
  bool fabric = false;             // handles are fabric handles exchanged over the bootstrap network (multi-node NVLink)
  int regSeq = 0;
  std::vector<SymSegment*> segments;
  std::vector<SymWindow*> windows;
  std::vector<std::pair<IpcMsg, int>> stash;   // early datagrams of a later stage
  std::mutex lock;
  // Device-side table [kMaxWinSlots][kMaxRanks] of where every symmetric window is mapped on this rank: kernels that learn
  // "window slot, offset" from a peer (send / receive rendezvous) turn it into an address here. Registration is collective and
  // slots are handed out lowest-free-first, so a window has the same slot on every rank.
  void** winTableDev = nullptr;
  bool slotUsed[kMaxWinSlots] = {};
};

ncclResult_t symInit(ncclComm* comm);
void symDestroy(ncclComm* comm);
// Collective over the communicator.
ncclResult_t symWindowRegister(ncclComm* comm, void* buff, size_t size, SymWindow** out, int flags);
ncclResult_t symWindowDeregister(ncclComm* comm, SymWindow* win);
// Window of `comm` that contains [ptr, ptr+bytes), or null.
SymWindow* symFindWindow(ncclComm* comm, const void* ptr, size_t bytes);

}  // namespace b200
