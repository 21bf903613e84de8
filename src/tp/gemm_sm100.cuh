// sm_100a building blocks for the tensor-parallel GEMM kernels: mbarriers with bounded waits,
// TMA tile loads (no cluster multicast anywhere), tcgen05 tensor-memory allocation, UMMA shared
// memory / instruction descriptors, tcgen05.mma issue and commit, tcgen05.ld for the epilogue.
// Written against the public PTX ISA (tcgen05.*, cp.async.bulk.tensor, mbarrier).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {
namespace sm100 {

__device__ __forceinline__ uint32_t smemAddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbarInit(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarInitFence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbarExpectTx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbarTry(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded: gives up after `limit` polls (each poll itself blocks for a hardware-defined while).
__device__ __forceinline__ bool mbarWait(uint32_t bar, uint32_t parity, uint32_t limit = 1u << 24) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbarTry(bar, parity)) return true;
  return false;
}

// ---------------------------------------------------------------- TMA (tile mode, one CTA, no multicast)
__device__ __forceinline__ void tmaLoad2d(uint32_t dstSmem, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dstSmem), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
// ---------------------------------------------------------------- bulk copies (no tensor map, no multicast)
// global -> shared, completion counted on an mbarrier; the source may be a peer GPU's memory
__device__ __forceinline__ void bulkLoad(uint32_t dstSmem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dstSmem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// shared -> global, tracked by bulk groups
__device__ __forceinline__ void bulkStore(void* dst, uint32_t srcSmem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(srcSmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulkCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulkWaitRead() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulkWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Moves `bytes` (a multiple of 16) from `from` (possibly peer memory) to `to` (local memory) through a
// ring of shared-memory stages with bulk copies issued by ONE thread: several loads stay in flight
// over NVLink while earlier chunks are written out, without occupying the other threads of the CTA.
// `bars` are kStages initialised mbarriers (count 1); `phase` carries their parity across calls.
// Returns false when a load did not arrive within the wait limit (nothing is left in flight then).
template <int kStages, uint32_t kChunk>
__device__ __forceinline__ bool bulkPipe(char* to, const char* from, size_t bytes, uint32_t smemBase, uint64_t* bars, uint32_t& phaseBits) {
  const int total = (int)((bytes + kChunk - 1) / kChunk);
  constexpr int kAhead = kStages - 2;    // loads in flight ahead of the store being issued
  bool ok = true;
  int stored = 0;
  for (int i = 0; i < total + kAhead && ok; ++i) {
    if (i < total) {
      const int s = i % kStages;
      // the store that last used this stage was committed two stores ago: at most one newer group may still be reading
      if (i >= kStages) bulkWaitRead<1>();
      const uint32_t n = (uint32_t)(bytes - (size_t)i * kChunk < kChunk ? bytes - (size_t)i * kChunk : kChunk);
      const uint32_t b = smemAddr(&bars[s]);
      mbarExpectTx(b, n);
      bulkLoad(smemBase + s * kChunk, from + (size_t)i * kChunk, n, b);
    }
    if (i >= kAhead) {
      const int j = i - kAhead, s = j % kStages;
      const uint32_t n = (uint32_t)(bytes - (size_t)j * kChunk < kChunk ? bytes - (size_t)j * kChunk : kChunk);
      if (!mbarWait(smemAddr(&bars[s]), (phaseBits >> s) & 1u)) { ok = false; break; }
      phaseBits ^= 1u << s;
      bulkStore(to + (size_t)j * kChunk, smemBase + s * kChunk, n);
      bulkCommit();
      ++stored;
    }
  }
  if (!ok) {
    // loads already issued still write into shared memory: give them a bounded chance to land
    for (int j = stored; j < total && j < stored + kStages; ++j) mbarWait(smemAddr(&bars[j % kStages]), (phaseBits >> (j % kStages)) & 1u, 1u << 20);
  }
  bulkWaitAll();
  return ok;
}

// ---------------------------------------------------------------- CTA pairs (cluster of two, cta_group::2)
__device__ __forceinline__ uint32_t clusterCtaRank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// All threads of every CTA of the cluster meet; shared-memory writes before it are visible after it.
__device__ __forceinline__ void clusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of this CTA's shared-memory location `addr` as seen in CTA `ctaRank` of the cluster.
__device__ __forceinline__ uint32_t mapaShared(uint32_t addr, uint32_t ctaRank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(ctaRank));
  return r;
}
__device__ __forceinline__ void mbarArriveCluster(uint32_t clusterAddr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
__device__ __forceinline__ void stSharedCluster(uint32_t clusterAddr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(clusterAddr), "r"(v) : "memory");
}
// Tile load into this CTA's shared memory whose completion bytes are counted on an mbarrier of
// either CTA of the pair (cluster address). No multicast.
__device__ __forceinline__ void tmaLoad2dPair(uint32_t dstSmem, const CUtensorMap* map, int c0, int c1, uint32_t barCluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dstSmem), "l"(map), "r"(c0), "r"(c1), "r"(barCluster) : "memory");
}

__device__ __forceinline__ void prefetchTensorMap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void fenceProxyAsync() { asm volatile("fence.proxy.async;" ::: "memory"); }

// ---------------------------------------------------------------- tensor memory
// One warp allocates `cols` columns (power of two, 32..512); the base address lands in shared memory.
__device__ __forceinline__ void tmemAlloc(uint32_t dstSmem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dstSmem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmemRelinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmemDealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// Pair allocation: one warp in EACH CTA of the pair issues these collectively.
__device__ __forceinline__ void tmemAllocPair(uint32_t dstSmem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dstSmem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmemRelinquishPair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmemDeallocPair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---------------------------------------------------------------- UMMA descriptors
// Shared-memory matrix descriptor for a K-major operand tile stored by TMA with 128-byte swizzle:
// rows of 128 bytes (64 bf16 / 128 fp8 along K), groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t umDescK128(uint32_t smemByteAddr) {
  uint64_t d = 0;
  d |= (uint64_t)((smemByteAddr & 0x3FFFF) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                           // leading byte offset (unused with swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset: next 8-row group
  d |= (uint64_t)1 << 46;                           // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                           // swizzle mode: 128 bytes
  return d;
}
// Instruction descriptor, kind::f16 with bf16 inputs and fp32 accumulation, both operands K-major.
__host__ __device__ constexpr uint32_t umInstrBf16(int M, int N) {
  return (1u << 4) /* D = f32 */ | (1u << 7) /* A = bf16 */ | (1u << 10) /* B = bf16 */ | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// kind::f8f6f4 with e4m3 inputs (format code 0) and fp32 accumulation.
__host__ __device__ constexpr uint32_t umInstrE4m3(int M, int N) {
  return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T ; accumulate = 0 overwrites D.
__device__ __forceinline__ void ummaBf16(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void ummaF8(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
      ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void ummaCommit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// CTA pair: one thread of the leader CTA issues a 256 x N x 16 MMA over both CTAs' shared memory (each
// holds 128 rows of A and N/2 rows of B at the same offsets) into both CTAs' tensor memory.
__device__ __forceinline__ void ummaBf16Pair(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the mbarrier at the same shared-memory offset in every CTA of `ctaMask` once the MMAs
// issued so far have completed (this multicast is an mbarrier signal, not a load).
__device__ __forceinline__ void ummaCommitPair(uint32_t bar, uint16_t ctaMask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(ctaMask) : "memory");
}

// ---------------------------------------------------------------- epilogue loads
// 32 lanes x 32 columns of fp32: thread i of the warp receives columns [col, col+32) of lane i.
__device__ __forceinline__ void tmemLd32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmemLdWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ bool electOne() {
  uint32_t pred;
  asm volatile(
      "{\n.reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(pred));
  return pred != 0;
}

// 16 bytes of fp32 added into (possibly remote) global memory in one instruction.
__device__ __forceinline__ void redAddF32x4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

}  // namespace sm100
}  // namespace b200
