/*
 * GPU-initiated one-sided surface of the device API: put, signal, wait. The reference routes these
 * through a network backend (GDAKI / proxy); this build serves one NVLink domain, so for peers inside
 * the load/store team the operations are peer stores, `red.add` on signal words of the target's
 * resource window and bounded polls. Peers outside the team report ncclInvalidUsage (no RDMA
 * backend is linked).
 * Proxy mode (ncclDevCommRequirements_t::ginConnectionType > 0, ginForceEnable, or NCCL_GIN_TYPE=PROXY): put and signal
 * do not touch the peer from the kernel; one thread queues a descriptor for a host thread, which runs the copy on the
 * copy engines and the signal / counter updates behind it in stream order (the way a network proxy would post them),
 * and flush() waits until everything queued so far has completed. The SMs then only pay for the descriptor.
 *   put(peer, dst, src, bytes [, signal])   copy, then optionally bump a signal on the peer
 *   signal(peer, id)                        bump signal `id` on the peer (release ordering)
 *   waitSignal(id, value) / readSignal(id)  bounded wait on / read of a local signal
 *   flush()                                 make earlier puts visible before what follows
 * Reference parity: src/include/nccl_device/gin.h:21-333 (ncclGin: put, signal, flush, wait*,
 * read*, reset*), impl/gin__funcs.h (abort-aware waits :774-1000).
 */
#ifndef NCCL_DEVICE_GIN_H_
#define NCCL_DEVICE_GIN_H_
#include "core.h"
#include "coop.h"
#include "utility.h"
#if defined(__CUDACC__)
#include <cuda/atomic>
/* ---- the reference's spellings of "what else to do with a put": a signal on the peer (by id, or a 64-bit word
 * at an offset of a window: "VA" signals), a completion counter on this rank. Strong and weak variants differ in
 * what a network must settle first; with peer stores both are a release-ordered add after the data. */
typedef uint32_t ncclGinSignal_t;
typedef uint32_t ncclGinCounter_t;
struct ncclGin_None {};
struct ncclGin_SignalInc { ncclGinSignal_t signal; };
struct ncclGin_StrongSignalInc { ncclGinSignal_t signal; };
struct ncclGin_WeakSignalInc { ncclGinSignal_t signal; };
struct ncclGin_SignalAdd { ncclGinSignal_t signal; uint64_t value; };
struct ncclGin_StrongSignalAdd { ncclGinSignal_t signal; uint64_t value; };
struct ncclGin_WeakSignalAdd { ncclGinSignal_t signal; uint64_t value; };
struct ncclGin_VASignalInc { ncclWindow_t signalWindow; size_t signalOffset; };
struct ncclGin_StrongVASignalInc { ncclWindow_t signalWindow; size_t signalOffset; };
struct ncclGin_WeakVASignalInc { ncclWindow_t signalWindow; size_t signalOffset; };
struct ncclGin_VASignalAdd { ncclWindow_t signalWindow; size_t signalOffset; uint64_t value; };
struct ncclGin_StrongVASignalAdd { ncclWindow_t signalWindow; size_t signalOffset; uint64_t value; };
struct ncclGin_WeakVASignalAdd { ncclWindow_t signalWindow; size_t signalOffset; uint64_t value; };
struct ncclGin_CounterInc { ncclGinCounter_t counter; };
struct ncclGin_WeakCounterInc { ncclGinCounter_t counter; };
namespace nccl_device {
struct GinAction {   /* normal form of the action types above */
  int signal;                 /* signal id, or -1 */
  ncclWindow_t window;        /* VA signal: window and byte offset of the 64-bit word, else NULL */
  size_t offset;
  unsigned long long add;
  int counter;                /* counter id, or -1 */
};
__device__ inline GinAction ginAction(ncclGin_None) { GinAction a = {-1, nullptr, 0, 0, -1}; return a; }
#define NCCL_GIN_ACTION_ID_INC(T) __device__ inline GinAction ginAction(T x) { GinAction a = {(int)x.signal, nullptr, 0, 1, -1}; return a; }
#define NCCL_GIN_ACTION_ID_ADD(T) __device__ inline GinAction ginAction(T x) { GinAction a = {(int)x.signal, nullptr, 0, x.value, -1}; return a; }
#define NCCL_GIN_ACTION_VA_INC(T) __device__ inline GinAction ginAction(T x) { GinAction a = {-1, x.signalWindow, x.signalOffset, 1, -1}; return a; }
#define NCCL_GIN_ACTION_VA_ADD(T) __device__ inline GinAction ginAction(T x) { GinAction a = {-1, x.signalWindow, x.signalOffset, x.value, -1}; return a; }
#define NCCL_GIN_ACTION_COUNTER(T) __device__ inline GinAction ginAction(T x) { GinAction a = {-1, nullptr, 0, 0, (int)x.counter}; return a; }
NCCL_GIN_ACTION_ID_INC(ncclGin_SignalInc) NCCL_GIN_ACTION_ID_INC(ncclGin_StrongSignalInc) NCCL_GIN_ACTION_ID_INC(ncclGin_WeakSignalInc)
NCCL_GIN_ACTION_ID_ADD(ncclGin_SignalAdd) NCCL_GIN_ACTION_ID_ADD(ncclGin_StrongSignalAdd) NCCL_GIN_ACTION_ID_ADD(ncclGin_WeakSignalAdd)
NCCL_GIN_ACTION_VA_INC(ncclGin_VASignalInc) NCCL_GIN_ACTION_VA_INC(ncclGin_StrongVASignalInc) NCCL_GIN_ACTION_VA_INC(ncclGin_WeakVASignalInc)
NCCL_GIN_ACTION_VA_ADD(ncclGin_VASignalAdd) NCCL_GIN_ACTION_VA_ADD(ncclGin_StrongVASignalAdd) NCCL_GIN_ACTION_VA_ADD(ncclGin_WeakVASignalAdd)
NCCL_GIN_ACTION_COUNTER(ncclGin_CounterInc) NCCL_GIN_ACTION_COUNTER(ncclGin_WeakCounterInc)
#undef NCCL_GIN_ACTION_ID_INC
#undef NCCL_GIN_ACTION_ID_ADD
#undef NCCL_GIN_ACTION_VA_INC
#undef NCCL_GIN_ACTION_VA_ADD
#undef NCCL_GIN_ACTION_COUNTER
}  // namespace nccl_device
struct ncclGin {
  const ncclDevComm_t& comm;
  __device__ explicit ncclGin(const ncclDevComm_t& c, int /*context*/ = 0) : comm(c) {}

  __device__ unsigned long long* signalWord(int owner, int id) const {
    return (unsigned long long*)((char*)comm.resource.peerPtr[owner] + comm.ginSignalOffset) + id;
  }
  __device__ unsigned long long* counterWord(int id) const {
    return (unsigned long long*)((char*)comm.resource.peerPtr[comm.lsaRank] + comm.ginCounterOffset) + id;
  }

  /* ---- proxy mode */
  __device__ bool proxied() const { return comm.ginProxyRing != nullptr; }
  /* Queues one operation (called by one thread). ncclTimeout when the ring stayed full for the whole budget. */
  __device__ ncclResult_t proxyPost(void* dst, const void* src, unsigned long long bytes, unsigned long long* sig, unsigned long long add,
                                    unsigned long long* counter) const {
    const unsigned long long idx = atomicAdd(comm.ginProxyHead, 1ull);
    const long long start = clock64();
    unsigned spins = 0;
    while (idx - *comm.ginProxyTail > (unsigned long long)comm.ginProxyMask) {
      if ((++spins & 0xff) == 0 && ((unsigned long long)(clock64() - start) >= comm.timeoutCycles || ncclTestAbort(comm))) return ncclTimeout;
    }
    ncclGinProxyDesc* d = comm.ginProxyRing + (idx & comm.ginProxyMask);
    d->dst = dst; d->src = src; d->bytes = bytes; d->signal = sig; d->signalAdd = add; d->counter = counter;
    __threadfence_system();
    d->seq = idx + 1;
    return ncclSuccess;
  }
  /* Waits until every operation queued so far (by any thread of this GPU) has completed. */
  __device__ ncclResult_t proxyDrain() const {
    const unsigned long long want = *(volatile unsigned long long*)comm.ginProxyHead;
    const long long start = clock64();
    unsigned spins = 0;
    while (*comm.ginProxyDone < want) {
      if ((++spins & 0xff) == 0 && ((unsigned long long)(clock64() - start) >= comm.timeoutCycles || ncclTestAbort(comm))) return ncclTimeout;
    }
    nccl_device::fenceAcqRelSys();
    return ncclSuccess;
  }

  /* Everything this thread (and, after a group sync, its group) wrote earlier is visible to the peer
   * once it observes the signal. */
  __device__ ncclResult_t signal(ncclTeam_t team, int peer, int id, unsigned long long add = 1) {
    const int world = ncclTeamRankToWorld(comm, team, peer);
    if (world < 0 || world >= comm.lsaSize || id < 0 || id >= comm.ginSignalCount) return ncclInvalidUsage;
    if (proxied()) { __threadfence_system(); return proxyPost(nullptr, nullptr, 0, signalWord(world, id), add, nullptr); }
    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(signalWord(world, id)), "l"(add) : "memory");
    return ncclSuccess;
  }

  template <typename Coop>
  __device__ ncclResult_t put(Coop coop, ncclTeam_t team, int peer, ncclWindow_t dstWin, size_t dstOffset, ncclWindow_t srcWin, size_t srcOffset,
                              size_t bytes, int signalId = -1, int counterId = -1) {
    const int world = ncclTeamRankToWorld(comm, team, peer);
    if (world < 0 || world >= comm.lsaSize) return ncclInvalidUsage;
    const char* s = (const char*)ncclGetLocalPointer(srcWin, srcOffset);
    char* d = (char*)ncclGetLsaPointer(dstWin, dstOffset, world);
    if (proxied()) {
      // the source must be complete before the host thread starts the copy: the group's writes are fenced, then one thread posts
      __threadfence_system();
      coop.sync();
      ncclResult_t r = ncclSuccess;
      if (coop.thread_rank() == 0)
        r = proxyPost(d, s, bytes, signalId >= 0 && signalId < comm.ginSignalCount ? signalWord(world, signalId) : nullptr, 1,
                      counterId >= 0 && counterId < comm.ginCounterCount ? counterWord(counterId) : nullptr);
      return r;
    }
    if ((((uintptr_t)s | (uintptr_t)d) & 15) == 0) {
      for (size_t i = (size_t)coop.thread_rank() * 16; i + 16 <= bytes; i += (size_t)coop.size() * 16) *(uint4*)(d + i) = *(const uint4*)(s + i);
      for (size_t b = bytes / 16 * 16 + coop.thread_rank(); b < bytes; b += coop.size()) d[b] = s[b];
    } else {
      for (size_t b = coop.thread_rank(); b < bytes; b += coop.size()) d[b] = s[b];
    }
    coop.sync();
    if (coop.thread_rank() == 0) {
      if (signalId >= 0) signal(team, peer, signalId);
      if (counterId >= 0 && counterId < comm.ginCounterCount) atomicAdd(counterWord(counterId), 1ull);
    }
    return ncclSuccess;
  }

  __device__ unsigned long long readSignal(int id) const {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(signalWord(comm.lsaRank, id)) : "memory");
    return v;
  }
  __device__ unsigned long long readCounter(int id) const { return *(volatile unsigned long long*)counterWord(id); }

  /* Returns ncclTimeout when the signal did not reach `value` within the budget (or the communicator was aborted). */
  __device__ ncclResult_t waitSignal(int id, unsigned long long value, unsigned long long timeoutCycles = 0) const {
    if (id < 0 || id >= comm.ginSignalCount) return ncclInvalidUsage;
    const unsigned long long budget = timeoutCycles ? timeoutCycles : comm.timeoutCycles;
    const long long start = clock64();
    unsigned spins = 0;
    while (readSignal(id) < value) {
      if ((++spins & 0xff) == 0 && ((unsigned long long)(clock64() - start) >= budget || ncclTestAbort(comm))) return ncclTimeout;
    }
    nccl_device::fenceAcqRelSys();
    return ncclSuccess;
  }
  __device__ void resetSignal(int id) { *(volatile unsigned long long*)signalWord(comm.lsaRank, id) = 0; }
  __device__ void resetCounter(int id) { *(volatile unsigned long long*)counterWord(id) = 0; }
  __device__ void flush() {
    if (proxied()) { (void)proxyDrain(); return; }
    nccl_device::fenceAcqRelSys();
  }

  /* ---- the reference's call shapes (team first, actions as typed values, cooperative group last) */
  __device__ void applyRemote(int world, const nccl_device::GinAction& a) const {
    if (proxied()) {
      unsigned long long* w = a.signal >= 0 && a.signal < comm.ginSignalCount ? signalWord(world, a.signal)
                              : a.window ? (unsigned long long*)ncclGetLsaPointer(a.window, a.offset, world) : nullptr;
      if (w) (void)proxyPost(nullptr, nullptr, 0, w, a.add, nullptr);   // queued behind the put of the same thread: runs after it
      return;
    }
    if (a.signal >= 0 && a.signal < comm.ginSignalCount)
      asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(signalWord(world, a.signal)), "l"(a.add) : "memory");
    else if (a.window)
      asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(ncclGetLsaPointer(a.window, a.offset, world)), "l"(a.add) : "memory");
  }
  template <typename RemoteAction = ncclGin_None, typename LocalAction = ncclGin_None, typename Coop = ncclCoopThread>
  __device__ void put(ncclTeam_t team, int peer, ncclWindow_t dstWin, size_t dstOffset, ncclWindow_t srcWin, size_t srcOffset, size_t bytes,
                      RemoteAction remoteAction = ncclGin_None{}, LocalAction localAction = ncclGin_None{}, Coop coop = ncclCoopThread{}) {
    const nccl_device::GinAction ra = nccl_device::ginAction(remoteAction), la = nccl_device::ginAction(localAction);
    if (put(coop, team, peer, dstWin, dstOffset, srcWin, srcOffset, bytes, -1, la.counter) != ncclSuccess) return;
    if (coop.thread_rank() == 0) applyRemote(ncclTeamRankToWorld(comm, team, peer), ra);
  }
  template <typename T, typename RemoteAction = ncclGin_None, typename Coop = ncclCoopThread>
  __device__ void putValue(ncclTeam_t team, int peer, ncclWindow_t dstWin, size_t dstOffset, T value, RemoteAction remoteAction = ncclGin_None{},
                           Coop coop = ncclCoopThread{}) {
    static_assert(sizeof(T) <= 8, "putValue moves at most eight bytes");
    const int world = ncclTeamRankToWorld(comm, team, peer);
    if (world < 0 || world >= comm.lsaSize) return;
    if (coop.thread_rank() == 0) {
      if (proxied()) (void)proxyDrain();   // a direct store must not overtake puts that are still queued
      *(volatile T*)ncclGetLsaPointer(dstWin, dstOffset, world) = value;
      if (proxied()) __threadfence_system();
      applyRemote(world, nccl_device::ginAction(remoteAction));
    }
  }
  template <typename RemoteAction, typename Coop = ncclCoopThread>
  __device__ void signal(ncclTeam_t team, int peer, RemoteAction remoteAction, Coop coop = ncclCoopThread{}) {
    const int world = ncclTeamRankToWorld(comm, team, peer);
    if (world < 0 || world >= comm.lsaSize) return;
    coop.sync();
    if (coop.thread_rank() == 0) applyRemote(world, nccl_device::ginAction(remoteAction));
  }
  template <typename Coop>
  __device__ void waitSignal(Coop coop, ncclGinSignal_t id, uint64_t least, int /*bits*/ = 64, cuda::memory_order = cuda::memory_order_acquire) const {
    if (coop.thread_rank() == 0) (void)waitSignal((int)id, (unsigned long long)least, 0ull);
    coop.sync();
  }
  template <typename Coop>
  __device__ void waitCounter(Coop coop, ncclGinCounter_t id, uint64_t least, int /*bits*/ = 64, cuda::memory_order = cuda::memory_order_acquire) const {
    if (coop.thread_rank() == 0 && (int)id < comm.ginCounterCount) {
      const long long start = clock64();
      unsigned spins = 0;
      while (readCounter((int)id) < least)
        if ((++spins & 0xff) == 0 && ((unsigned long long)(clock64() - start) >= comm.timeoutCycles || ncclTestAbort(comm))) break;
    }
    coop.sync();
  }
  __device__ uint64_t readSignal(ncclGinSignal_t id, int /*bits*/, cuda::memory_order = cuda::memory_order_acquire) const { return readSignal((int)id); }
  __device__ uint64_t readCounter(ncclGinCounter_t id, int /*bits*/, cuda::memory_order = cuda::memory_order_acquire) const { return readCounter((int)id); }
  template <typename Coop>
  __device__ void flush(Coop coop, cuda::memory_order = cuda::memory_order_acquire) const {
    if (proxied()) { if (coop.thread_rank() == 0) (void)proxyDrain(); }
    else nccl_device::fenceAcqRelSys();
    coop.sync();
  }
};
#endif
#endif
