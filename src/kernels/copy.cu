// Data-movement kernels without arithmetic.
//   copyCollKernel   all-gather, broadcast, all-to-all, gather and scatter as direct peer stores
//                    (push), peer loads (pull) or one multimem.st stream (mc). Every transfer is a
//                    list of equal segments; CTAs interleave over segments so that all peers are
//                    in flight at once, and segment order is rotated by rank so that no two ranks
//                    target the same peer first.
//   p2pKernel        grouped send/recv through per-pair mailboxes in the receiver's resource
//                    window: chunked, kP2pSlots chunks in flight, ready/ack flags per slot.
//   scaleKernel      dst = src * scalar (pre-multiplied sums, single-rank communicators).
//   signal kernels   one-sided signal / wait-signal counters.
// Reference parity: src/device/symmetric/all_gather.cuh:13-303 (ST / STMC), src/device/sendrecv.h,
// contrib/custom_algos/alltoall/lsa_simple_alltoall_kernel.cuh, src/device/onerank.cu, src/rma/rma_ce.cc.
#include "common.cuh"
#include "../tp/gemm_sm100.cuh"
#include "launch.h"
#include "../comm/comm.h"

namespace b200 {

struct Seg {
  const char* src;
  char* dst;
  int mc;
};

__device__ __forceinline__ int buildSegs(const CollArgs& a, int rank, Seg* segs) {
  const int n = a.nRanks;
  const size_t SS = a.sendStride, RS = a.recvStride;  // block pitch of inputs / outputs (>= a.count)
  int k = 0;
  const char* ls = (const char*)a.lsend[rank];
  char* lr = (char*)a.lrecv[rank];
  switch (a.func) {
    case FUNC_ALLGATHER:
      if (a.mode == MODE_MC) {
        segs[k++] = Seg{ls, (char*)a.recvMc + rank * RS, 1};
      } else if (a.mode == MODE_PUSH) {
        for (int j = 0; j < n; ++j) {
          int p = (rank + j) % n;
          char* d = (char*)a.recv[p] + rank * RS;
          if (d != ls) segs[k++] = Seg{ls, d, 0};
        }
      } else {
        for (int j = 0; j < n; ++j) {
          int p = (rank + j) % n;
          const char* s = p == rank ? ls : (const char*)a.send[p];
          if (s != lr + p * RS) segs[k++] = Seg{s, lr + p * RS, 0};
        }
      }
      break;
    case FUNC_BROADCAST:
      if (a.mode == MODE_MC) {
        if (rank == a.root) segs[k++] = Seg{ls, (char*)a.recvMc, 1};
      } else if (a.mode == MODE_PUSH) {
        if (rank == a.root)
          for (int j = 0; j < n; ++j) {
            int p = (rank + j) % n;
            char* d = (char*)a.recv[p];
            if (d != ls) segs[k++] = Seg{ls, d, 0};
          }
      } else {
        const char* s = rank == a.root ? ls : (const char*)a.send[a.root];
        if (s != lr) segs[k++] = Seg{s, lr, 0};
      }
      break;
    case FUNC_ALLTOALL:
      for (int j = 0; j < n; ++j) {
        int p = (rank + j) % n;
        if (a.mode == MODE_PUSH) segs[k++] = Seg{ls + p * SS, (char*)a.recv[p] + rank * RS, 0};
        else segs[k++] = Seg{(p == rank ? ls : (const char*)a.send[p]) + rank * SS, lr + p * RS, 0};
      }
      break;
    case FUNC_GATHER:
      if (a.mode == MODE_PUSH) {
        segs[k++] = Seg{ls, (char*)a.recv[a.root] + rank * RS, 0};
      } else if (rank == a.root) {
        for (int j = 0; j < n; ++j) {
          int p = (rank + j) % n;
          segs[k++] = Seg{p == rank ? ls : (const char*)a.send[p], lr + p * RS, 0};
        }
      }
      break;
    case FUNC_SCATTER:
      if (a.mode == MODE_PUSH) {
        if (rank == a.root)
          for (int j = 0; j < n; ++j) {
            int p = (rank + j) % n;
            segs[k++] = Seg{ls + p * SS, (char*)a.recv[p], 0};
          }
      } else {
        segs[k++] = Seg{(rank == a.root ? ls : (const char*)a.send[a.root]) + rank * SS, lr, 0};
      }
      break;
    default: break;
  }
  return k;
}

constexpr int kTilePacks = kCtaThreads * 4;  // 32 KiB per CTA tile

__global__ void __launch_bounds__(kCtaThreads, 1) copyCollKernel(const __grid_constant__ CollArgs a) {
  const int rank = ctaRank(a.emu, a.rank);
  pdlEnter();
  KernelStamp stamp(a.sync.stamps);
  CtaBarrier bar;
  bar.init(a.sync, rank, a.nRanks, blockIdx.x);
  if (a.func == FUNC_BROADCAST && a.mode == MODE_SPLIT) {
    // Large broadcast with the work shared out: every rank but the root pulls one share of the root's buffer (one pass
    // over the root's links) and stores it into its own output and into the other non-root ranks' outputs; the root
    // copies its output locally. The stores of all GPUs work, not only the root's. The root's buffer is found through the
    // descriptor that every CTA of the root publishes before the opening barrier (its window slot and offset), since only
    // the root knows its own send pointer; without a window the root pushes everything itself.
    const int n = a.nRanks, root = a.root;
    __shared__ uint4 sDesc;
    if (rank == root && a.winTable != nullptr && threadIdx.x < n && threadIdx.x != rank) {
      // Every CTA of the root writes the same line before it arrives at its barrier slot, and the matching CTA of a peer reads
      // it after that barrier: the line a peer sees is this launch's (the root cannot start the next launch before every
      // CTA of every peer has arrived at the closing barrier, which comes after the read).
      uint4 d = make_uint4(1u, (uint32_t)a.bcastSlot, (uint32_t)a.bcastOff, (uint32_t)(a.bcastOff >> 32));
      stVolatile16((char*)a.sync.inbox[threadIdx.x] + kOffBcastDesc, d);
    }
    bool ok = bar.sync(rank == root, rank != root);
    const char* src = (const char*)a.send[root];   // emulation: given directly
    if (a.winTable != nullptr && rank != root) {
      if (threadIdx.x == 0) sDesc = ldVolatile16((const char*)a.sync.inbox[rank] + kOffBcastDesc);
      __syncthreads();
      const uint4 d = sDesc;
      src = d.y ? (const char*)a.winTable[(size_t)(d.y - 1) * kMaxRanks + root] + (((size_t)d.w << 32) | d.z) : nullptr;
      if (d.x != 1u) ok = false;   // never written: leave the data alone
    }
    const bool shared = rank == root ? (a.winTable != nullptr ? a.bcastSlot != 0 : true) : src != nullptr;
    const size_t B = a.count;
    const size_t packs = B / 16;
    const char* ls = (const char*)a.lsend[rank];
    char* lr = (char*)a.lrecv[rank];
    if (ok && B > 0 && rank == root && !a.vec16) {
      // the root's buffer is not 16-byte aligned: nothing is shared out (bcastSlot is 0), the root stores every byte itself
      for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < B; i += (size_t)gridDim.x * blockDim.x) {
        const char v = ls[i];
        for (int j = 0; j < n; ++j) {
          char* d = j == 0 ? lr : (char*)a.recv[(rank + j) % n];
          if (d != ls) d[i] = v;
        }
      }
    } else if (ok && B > 0 && a.vec16) {
      if (rank == root) {
        // local copy into the root's own output; without a window also the push to everybody
        const int nDst = shared ? 1 : n;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < packs; i += (size_t)gridDim.x * blockDim.x) {
          const uint4 v = ldStream16(ls + i * 16);
          for (int j = 0; j < nDst; ++j) {
            char* d = j == 0 ? lr : (char*)a.recv[(rank + j) % n];
            if (d != ls) st16(d + i * 16, v);
          }
        }
      } else if (shared) {
        const int w = (rank - root - 1 + n) % n;                       // worker index among the n - 1 non-root ranks
        const size_t share = ((packs + (n - 1) - 1) / (n - 1));        // packs per worker
        const size_t first = (size_t)w * share, last = first + share < packs ? first + share : packs;
        const size_t stride = (size_t)gridDim.x * blockDim.x;
        size_t i = first + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
        for (; i + 3 * stride < last; i += 4 * stride) {
          uint4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) v[u] = ldStream16(src + (i + u * stride) * 16);
#pragma unroll
          for (int j = 0; j < kMaxRanks; ++j) {
            const int p = (rank + j) % n;
            if (j < n && p != root) {
              char* d = p == rank ? lr : (char*)a.recv[p];
#pragma unroll
              for (int u = 0; u < 4; ++u) st16(d + (i + u * stride) * 16, v[u]);
            }
          }
        }
        for (; i < last; i += stride) {
          const uint4 v = ldStream16(src + i * 16);
          for (int j = 0; j < n; ++j) {
            const int p = (rank + j) % n;
            if (p != root) st16((p == rank ? lr : (char*)a.recv[p]) + i * 16, v);
          }
        }
      }
    }
    bar.sync(true, false);
    bar.finish();
    return;
  }
  bool ok = bar.sync(false, false);   // every rank's kernel has started: inputs final, outputs free
  __shared__ Seg segs[kMaxRanks];
  __shared__ int nSeg;
  if (threadIdx.x == 0) nSeg = buildSegs(a, rank, segs);
  __syncthreads();
  const size_t B = a.count;
  if (ok && nSeg > 0 && B > 0) {
    if (a.vec16) {
      const size_t packs = B / 16;
      const size_t tilesPerSeg = (packs + kTilePacks - 1) / kTilePacks;
      const size_t tiles = tilesPerSeg * nSeg;
      for (size_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const Seg s = segs[t % nSeg];
        const size_t base = (t / nSeg) * kTilePacks;
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          size_t i = base + u * kCtaThreads + threadIdx.x;
          if (i < packs) v[u] = ldStream16(s.src + i * 16);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          size_t i = base + u * kCtaThreads + threadIdx.x;
          if (i < packs) { if (s.mc) mcSt16(s.dst + i * 16, v[u]); else st16(s.dst + i * 16, v[u]); }
        }
      }
      // bytes past the last whole pack (multicast stores need 16-byte units: the host only picks
      // MODE_MC when B is a multiple of 16)
      const size_t rem = B - packs * 16;
      if (rem && blockIdx.x == 0)
        for (size_t j = threadIdx.x; j < rem * nSeg; j += blockDim.x) {
          const Seg s = segs[j / rem];
          s.dst[packs * 16 + j % rem] = s.src[packs * 16 + j % rem];
        }
    } else {
      const size_t stride = (size_t)gridDim.x * blockDim.x;
      for (int si = 0; si < nSeg; ++si) {
        const Seg s = segs[si];
        for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < B; j += stride) s.dst[j] = s.src[j];
      }
    }
  }
  bar.sync(true, false);
  bar.finish();
}

// The same collectives moved by the bulk-copy engine of each SM instead of by its threads: one
// thread per CTA streams its contiguous share of every segment through a ring of shared-memory
// stages (cp.async.bulk global -> shared -> global; sources and destinations may be peer memory or
// the multicast alias; no cluster multicast anywhere). A CTA keeps four 32 KiB loads in flight while
// earlier chunks drain, so a dozen CTAs fill the links and the other SMs stay with the compute
// kernels the collective overlaps. Needs 16-byte aligned pointers and a block size that is a
// multiple of 16 bytes (the host picks the thread kernel otherwise).
// Reference parity: the TMA variants of src/device/symmetric/all_gather.cuh:277-308.
constexpr int kCollBulkStages = 6;
constexpr uint32_t kCollBulkChunk = 32768;
__global__ void __launch_bounds__(32, 1) copyCollBulkKernel(const __grid_constant__ CollArgs a) {
  extern __shared__ uint8_t collBulkRaw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)collBulkRaw + 127) & ~(uintptr_t)127);
  uint64_t* bars = (uint64_t*)(sm + (size_t)kCollBulkStages * kCollBulkChunk);
  const int rank = ctaRank(a.emu, a.rank);
  pdlEnter();
  KernelStamp stamp(a.sync.stamps);
  CtaBarrier bar;
  bar.init(a.sync, rank, a.nRanks, blockIdx.x);
  bool ok = bar.sync(false, false);
  __shared__ Seg segs[kMaxRanks];
  __shared__ int nSeg;
  if (threadIdx.x == 0) nSeg = buildSegs(a, rank, segs);
  __syncthreads();
  const size_t B = a.count;
  if (threadIdx.x == 0 && ok && nSeg > 0 && B > 0) {
    for (int s = 0; s < kCollBulkStages; ++s) sm100::mbarInit(sm100::smemAddr(&bars[s]), 1);
    sm100::mbarInitFence();
    const size_t chunks = (B + kCollBulkChunk - 1) / kCollBulkChunk;
    const size_t per = (chunks + gridDim.x - 1) / gridDim.x;
    const size_t lo = (size_t)blockIdx.x * per * kCollBulkChunk;
    if (lo < B) {
      const size_t n = B - lo < per * kCollBulkChunk ? B - lo : per * kCollBulkChunk;
      uint32_t phaseBits = 0;
      bool moved = true;
      // CTAs start on different segments so that no peer is hit by all of them at once
      for (int si = 0; si < nSeg && moved; ++si) {
        const Seg sg = segs[(si + blockIdx.x) % nSeg];
        moved = sm100::bulkPipe<kCollBulkStages, kCollBulkChunk>(sg.dst + lo, sg.src + lo, n, sm100::smemAddr(sm), bars, phaseBits);
      }
      if (!moved) {
        // a load did not arrive within the wait limit: report it like any other wait that ran out
        uint32_t* st = a.sync.status[rank];
        if (ldRelaxedSys(st) == DEV_OK) { st[1] = WAIT_TILE; st[2] = (uint32_t)rank; st[3] = 0; __threadfence_system(); stRelaxedSys(st, DEV_TIMEOUT); }
      }
    }
  }
  bar.sync(true, false);
  bar.finish();
}
const void* copyBulkKernelFn() { return (const void*)copyCollBulkKernel; }
size_t copyBulkSmemBytes() { return 128 + (size_t)kCollBulkStages * kCollBulkChunk + kCollBulkStages * 8; }

// ------------------------------------------------------------------------- send / recv
__device__ __forceinline__ void copyChunk(char* dst, const char* src, size_t bytes) {
  if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
    const size_t packs = bytes / 16;
    size_t i = threadIdx.x;
    // eight independent 16-byte loads in flight per thread: one CTA moves a chunk at a time, so its own queue depth is what counts
    for (; i + 7 * blockDim.x < packs; i += 8 * blockDim.x) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = ldStream16(src + (i + u * blockDim.x) * 16);
#pragma unroll
      for (int u = 0; u < 8; ++u) st16(dst + (i + u * blockDim.x) * 16, v[u]);
    }
    for (; i < packs; i += blockDim.x) st16(dst + i * 16, ldStream16(src + i * 16));
    for (size_t j = packs * 16 + threadIdx.x; j < bytes; j += blockDim.x) dst[j] = src[j];
  } else {
    for (size_t j = threadIdx.x; j < bytes; j += blockDim.x) dst[j] = src[j];
  }
}

// Grid-strided copy of [begin, begin + bytes) by the CTAs `local` of `count` of one operation (16-byte packs when aligned).
__device__ __forceinline__ void copyShare(char* dst, const char* src, size_t bytes, int local, int count) {
  if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
    const size_t packs = bytes / 16;
    const size_t stride = (size_t)count * blockDim.x;
    size_t i = (size_t)local * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < packs; i += 4 * stride) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = ldStream16(src + (i + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < 4; ++u) st16(dst + (i + u * stride) * 16, v[u]);
    }
    for (; i < packs; i += stride) st16(dst + i * 16, ldStream16(src + i * 16));
    if (local == 0) for (size_t j = packs * 16 + threadIdx.x; j < bytes; j += blockDim.x) dst[j] = src[j];
  } else {
    const size_t stride = (size_t)count * blockDim.x;
    for (size_t j = (size_t)local * blockDim.x + threadIdx.x; j < bytes; j += stride) dst[j] = src[j];
  }
}

// Send / receive. Two protocols, chosen from the byte count (both sides know it) and the receiver's buffer:
//   mailbox     the sender copies chunks into the receiver's mailbox (slots per ordered pair, ready / ack flags),
//               the receiver copies them out: works for any buffer, two passes over the data;
//   rendezvous  (large messages) the receiver first posts a 16-byte descriptor into the sender's flag page: its
//               buffer lies in a peer-mapped window (slot, offset) or not. If it does, all CTAs of the send write
//               straight into the receiver's buffer and the last one publishes one flag; the receiver only waits.
//               If not, the message goes through the mailbox as above.
// Sequence numbers count chunks per ordered pair in both protocols, so the two sides stay in step whichever ran.
__global__ void __launch_bounds__(kCtaThreads, 1) p2pKernel(const __grid_constant__ P2pArgs a) {
  const int rank = ctaRank(a.emu, a.rank);
  pdlEnter();
  KernelStamp stamp(a.sync.stamps);
  const int nOps = a.nOps[rank];
  const P2pOp* ops = a.ops + a.opBase[rank];
  WaitCtx w{&a.sync, a.sync.status[rank]};
  uint32_t* seq = a.seq[rank];  // [0,kMaxRanks) send counters, [kMaxRanks,2*kMaxRanks) recv counters, [2*kMaxRanks] finished CTAs
  __shared__ uint4 sDesc;
  int mine = -1;
  for (int i = 0; i < nOps; ++i)
    if ((int)blockIdx.x >= ops[i].ctaBegin && (int)blockIdx.x < ops[i].ctaBegin + ops[i].ctaCount) mine = i;
  if (mine >= 0) {
    const P2pOp op = ops[mine];
    const int local = blockIdx.x - op.ctaBegin;
    const size_t chunkBytes = p2pChunkOf(op.bytes);
    const size_t nChunks = (op.bytes + chunkBytes - 1) / chunkBytes;
    const uint32_t base = (op.isSend ? seq[op.peer] : seq[kMaxRanks + op.peer]) + op.seqOffset;
    const uint32_t qLast = base + (uint32_t)nChunks - 1;
    bool ok = true;
    bool direct = false;
    const bool rdvMode = a.winTable != nullptr && op.rdvLine >= 0 && op.bytes >= kP2pDirectMin;
    if (rdvMode) {
      const uint32_t tag = base + 1;
      if (op.isSend) {
        // where does the receiver want the data?
        if (threadIdx.x == 0) {
          const uint4* line = (const uint4*)a.rdv[rank] + op.peer * kP2pRdvLines + op.rdvLine;
          uint4 d = make_uint4(0, 0, 0, 0);
          ok = boundedWait(w, WAIT_P2P_READY, (uint32_t)op.peer, tag, [&] { d = ldVolatile16(line); return d.x == tag; });
          sDesc = d;
        }
        ok = __syncthreads_and(ok);
        const uint4 d = sDesc;
        if (ok && d.y != 0) {
          direct = true;
          char* dst = (char*)a.winTable[(size_t)(d.y - 1) * kMaxRanks + op.peer] + (((size_t)d.w << 32) | d.z);
          copyShare(dst, (const char*)op.buf, op.bytes, local, op.ctaCount);
          __syncthreads();
          if (threadIdx.x == 0) {
            fenceSys();   // this CTA's stores are ordered before the counter, and through it before the flag of the last CTA
            uint32_t* doneCnt = a.opDone[rank] + mine;
            if (atomicAdd(doneCnt, 1u) == (uint32_t)op.ctaCount - 1) {
              *doneCnt = 0;
              fenceSys();
              stRelaxedSys(a.ready[op.peer] + rank * kP2pSlots + (qLast % kP2pSlots), qLast + 1);
            }
          }
        }
      } else {
        direct = op.winSlot >= 0;
        if (local == 0 && threadIdx.x == 0) {
          uint4 d = make_uint4(tag, direct ? (uint32_t)op.winSlot + 1 : 0u, (uint32_t)op.winOff, (uint32_t)(op.winOff >> 32));
          stVolatile16((uint4*)a.rdv[op.peer] + rank * kP2pRdvLines + op.rdvLine, d);
        }
        if (direct) {
          if (threadIdx.x == 0) {
            const uint32_t* rdy = a.ready[rank] + op.peer * kP2pSlots + (qLast % kP2pSlots);
            const uint32_t want = qLast + 1;
            ok = boundedWait(w, WAIT_P2P_READY, (uint32_t)op.peer, want, [&] { return (int32_t)(ldRelaxedSys(rdy) - want) >= 0; });
            fenceSys();   // acquire: the data behind the flag
            // the mailbox slots were not used: tell the sender that all of them are free up to this message
            if (ok && local == 0)
              for (int sl = 0; sl < kP2pSlots; ++sl) stRelaxedSys(a.ack[op.peer] + rank * kP2pSlots + sl, qLast + 1);
          }
          ok = __syncthreads_and(ok);
        }
      }
    }
    if (!rdvMode && op.bytes <= kP2pLLMax && nChunks == 1 && local == 0) {
      // ---- small message: flagged lines, one chunk, one CTA
      const uint32_t q = base, tag = base + 1;
      const int slot = q % kP2pSlots;
      const size_t nLines = (op.bytes + 7) / 8;
      if (op.isSend) {
        if (threadIdx.x == 0 && q >= (uint32_t)kP2pSlots) {
          const uint32_t* ackp = a.ack[rank] + op.peer * kP2pSlots + slot;
          const uint32_t want = q - kP2pSlots + 1;
          ok = boundedWait(w, WAIT_P2P_ACK, (uint32_t)op.peer, want, [&] { return (int32_t)(ldRelaxedSys(ackp) - want) >= 0; });
        }
        ok = __syncthreads_and(ok);
        char* dst = a.llbox[op.peer] + ((size_t)rank * kP2pSlots + slot) * kP2pLLSlotBytes;
        const char* src = (const char*)op.buf;
        for (size_t l = threadIdx.x; ok && l < nLines; l += blockDim.x) {
          uint64_t d = 0;
          const size_t valid = op.bytes - l * 8;
          if (valid >= 8 && (((uintptr_t)src + l * 8) & 7) == 0) d = *(const uint64_t*)(src + l * 8);
          else for (size_t b = 0; b < 8 && b < valid; ++b) d |= (uint64_t)(uint8_t)src[l * 8 + b] << (8 * b);
          stVolatile16(dst + l * 16, make_uint4((uint32_t)d, tag, (uint32_t)(d >> 32), tag));
        }
      } else {
        const char* src = a.llbox[rank] + ((size_t)op.peer * kP2pSlots + slot) * kP2pLLSlotBytes;
        char* dst = (char*)op.buf;
        for (size_t l = threadIdx.x; ok && l < nLines; l += blockDim.x) {
          uint4 v = ldVolatile16(src + l * 16);
          if (v.y != tag || v.w != tag) ok = boundedWait(w, WAIT_P2P_READY, (uint32_t)op.peer, tag, [&] { v = ldVolatile16(src + l * 16); return v.y == tag && v.w == tag; });
          if (!ok) break;
          const uint64_t d = (uint64_t)v.x | ((uint64_t)v.z << 32);
          const size_t valid = op.bytes - l * 8;
          if (valid >= 8 && (((uintptr_t)dst + l * 8) & 7) == 0) *(uint64_t*)(dst + l * 8) = d;
          else for (size_t b = 0; b < 8 && b < valid; ++b) dst[l * 8 + b] = (char)(d >> (8 * b));
        }
        ok = __syncthreads_and(ok);
        if (ok && threadIdx.x == 0) stRelaxedSys(a.ack[op.peer] + rank * kP2pSlots + slot, q + 1);   // every line was read before the barrier
      }
      direct = true;   // nothing left for the chunk loop
    }
    for (size_t c = local; !direct && c < nChunks && ok; c += op.ctaCount) {
      const uint32_t q = base + (uint32_t)c;
      const int slot = q % kP2pSlots;
      const size_t off = c * chunkBytes;
      const size_t len = op.bytes - off < chunkBytes ? op.bytes - off : chunkBytes;
      if (op.isSend) {
        // the slot is free once the receiver has consumed the chunk that used it last (q - slots)
        // (sequence numbers run across calls, so this also covers slots used by the previous call)
        if (threadIdx.x == 0 && q >= (uint32_t)kP2pSlots) {
          const uint32_t* ackp = a.ack[rank] + op.peer * kP2pSlots + slot;
          const uint32_t want = q - kP2pSlots + 1;
          ok = boundedWait(w, WAIT_P2P_ACK, (uint32_t)op.peer, want, [&] { return (int32_t)(ldRelaxedSys(ackp) - want) >= 0; });   // permission only: no data to acquire
        }
        ok = __syncthreads_and(ok);
        if (!ok) break;
        char* dst = a.mailbox[op.peer] + ((size_t)rank * kP2pSlots + slot) * kP2pChunkBytes;
        copyChunk(dst, (const char*)op.buf + off, len);
        __syncthreads();
        if (threadIdx.x == 0) {
          fenceSys();
          stRelaxedSys(a.ready[op.peer] + rank * kP2pSlots + slot, q + 1);
        }
      } else {
        if (threadIdx.x == 0) {
          const uint32_t* rdy = a.ready[rank] + op.peer * kP2pSlots + slot;
          const uint32_t want = q + 1;
          ok = boundedWait(w, WAIT_P2P_READY, (uint32_t)op.peer, want, [&] { return (int32_t)(ldRelaxedSys(rdy) - want) >= 0; });
          fenceSys();   // acquire: the chunk behind the flag
        }
        ok = __syncthreads_and(ok);
        if (!ok) break;
        const char* src = a.mailbox[rank] + ((size_t)op.peer * kP2pSlots + slot) * kP2pChunkBytes;
        copyChunk((char*)op.buf + off, src, len);
        __syncthreads();
        if (threadIdx.x == 0) {
          stRelaxedSys(a.ack[op.peer] + rank * kP2pSlots + slot, q + 1);   // the reads above completed before the barrier
        }
      }
    }
  }
  // The last CTA of the grid advances the per-peer sequence numbers for the next launch.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t done = atomicAdd(&seq[2 * kMaxRanks], 1u);
    if (done == gridDim.x - 1) {
      seq[2 * kMaxRanks] = 0;
      for (int i = 0; i < nOps; ++i) {
        const size_t cb = p2pChunkOf(ops[i].bytes);
        uint32_t chunks = (uint32_t)((ops[i].bytes + cb - 1) / cb);
        if (ops[i].isSend) seq[ops[i].peer] += chunks; else seq[kMaxRanks + ops[i].peer] += chunks;
      }
    }
  }
}

// ------------------------------------------------------------------------- mesh-to-mesh reshard
// One launch per rank: after a barrier (every rank's kernel has started, so every source tile is final) the CTAs share the
// 64 KiB tiles of all runs round-robin and copy them with peer loads; a closing barrier tells the sources that nobody
// reads their tiles any more. No mailbox, no matching of sends and receives.
// Reference parity: the pull kernels of contrib/nccl_m2n (src/m2n_kernels.cu).
__global__ void __launch_bounds__(kCtaThreads, 1) reshardKernel(const __grid_constant__ ReshardArgs a) {
  const int rank = ctaRank(a.emu, a.rank);
  pdlEnter();
  KernelStamp stamp(a.sync.stamps);
  CtaBarrier bar;
  bar.init(a.sync, rank, a.nRanks, blockIdx.x);
  const bool ok = bar.sync(false, false);
  constexpr unsigned long long kTile = 64 << 10;
  if (ok) {
    unsigned long long firstTile = 0;   // index of the run's first tile in the round-robin over all runs
    for (int r = 0; r < a.nRuns; ++r) {
      const ReshardRun run = a.runs[r];
      const unsigned long long tiles = (run.bytes + kTile - 1) / kTile;
      const char* src = a.winPeer[run.srcRank] + a.tileOff[run.srcRank] + run.srcOff;
      char* dst = a.dst + run.dstOff;
      // first tile of this run that belongs to this CTA
      unsigned long long t = ((unsigned long long)blockIdx.x + gridDim.x - firstTile % gridDim.x) % gridDim.x;
      for (; t < tiles; t += gridDim.x) {
        const unsigned long long off = t * kTile;
        const unsigned long long len = run.bytes - off < kTile ? run.bytes - off : kTile;
        copyChunk(dst + off, src + off, (size_t)len);
      }
      firstTile += tiles;
    }
  }
  bar.sync(false, false);
  bar.finish();
}
const void* reshardKernelFn() { return (const void*)reshardKernel; }

// ------------------------------------------------------------------------- local scale
template <typename T>
__global__ void scaleKernel(ScaleArgs a) {
  using A = typename Elem<T>::Acc;
  T s;
  if (a.scalarPtr) s = *(const T*)a.scalarPtr;
  else memcpy(&s, &a.scalarBits, sizeof(T));
  const A sa = Elem<T>::ld(s);
  const T* src = (const T*)a.src;
  T* dst = (T*)a.dst;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.count; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = Elem<T>::st(Elem<T>::ld(src[i]) * sa);
}

const void* scaleKernelFn(ncclDataType_t type) {
  switch (type) {
    case ncclInt8: return (const void*)scaleKernel<int8_t>;
    case ncclUint8: return (const void*)scaleKernel<uint8_t>;
    case ncclInt32: return (const void*)scaleKernel<int32_t>;
    case ncclUint32: return (const void*)scaleKernel<uint32_t>;
    case ncclInt64: return (const void*)scaleKernel<int64_t>;
    case ncclUint64: return (const void*)scaleKernel<uint64_t>;
    case ncclFloat16: return (const void*)scaleKernel<__half>;
    case ncclFloat32: return (const void*)scaleKernel<float>;
    case ncclFloat64: return (const void*)scaleKernel<double>;
    case ncclBfloat16: return (const void*)scaleKernel<__nv_bfloat16>;
    case ncclFloat8e4m3: return (const void*)scaleKernel<F8E4>;
    case ncclFloat8e5m2: return (const void*)scaleKernel<F8E5>;
    default: return nullptr;
  }
}

// Local copy of `count` bytes: the data movement of a single-rank communicator (out-of-place
// collectives reduce to dst = src) and of staged transfers. A CTA moves contiguous tiles of
// U x blockDim x 16 bytes (all loads of a tile issued before its stores), and CTAs stride over
// tiles, so that each DRAM page is opened once and enough bytes are in flight for HBM speed.
template <int U>
__global__ void __launch_bounds__(512) localCopyKernel(ScaleArgs a) {
  const char* src = (const char*)a.src;
  char* dst = (char*)a.dst;
  const size_t bytes = a.count;
  if ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
    const size_t packs = bytes / 16;
    const size_t tilePacks = (size_t)U * blockDim.x;
    const size_t fullTiles = packs / tilePacks;
    for (size_t t = blockIdx.x; t < fullTiles; t += gridDim.x) {
      const size_t base = t * tilePacks + threadIdx.x;
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = ldStream16(src + (base + (size_t)u * blockDim.x) * 16);
#pragma unroll
      for (int u = 0; u < U; ++u) st16(dst + (base + (size_t)u * blockDim.x) * 16, v[u]);
    }
    // remainder: packs past the last full tile, then loose bytes
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (size_t i = fullTiles * tilePacks + tid; i < packs; i += stride) st16(dst + i * 16, ldStream16(src + i * 16));
    for (size_t j = packs * 16 + tid; j < bytes; j += stride) dst[j] = src[j];
  } else {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < bytes; i += stride) dst[i] = src[i];
  }
}
// The same copy driven by the bulk-copy engines of each SM: one thread per CTA moves its contiguous
// share through a ring of shared-memory stages (cp.async.bulk global -> shared -> global), several
// 32 KiB chunks in flight per SM. Needs 16-byte aligned pointers; bytes past the last multiple of 16
// are copied by thread 0 of CTA 0.
constexpr int kBulkStages = 6;
constexpr uint32_t kBulkChunk = 32768;
__global__ void __launch_bounds__(32) localBulkCopyKernel(ScaleArgs a) {
  extern __shared__ uint8_t bulkSmemRaw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)bulkSmemRaw + 127) & ~(uintptr_t)127);
  uint64_t* bars = (uint64_t*)(sm + (size_t)kBulkStages * kBulkChunk);
  const size_t bytes16 = a.count & ~(size_t)15;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kBulkStages; ++s) sm100::mbarInit(sm100::smemAddr(&bars[s]), 1);
    sm100::mbarInitFence();
    // contiguous share per CTA, in whole chunks
    const size_t chunks = (bytes16 + kBulkChunk - 1) / kBulkChunk;
    const size_t per = (chunks + gridDim.x - 1) / gridDim.x;
    const size_t lo = (size_t)blockIdx.x * per * kBulkChunk;
    if (lo < bytes16) {
      const size_t n = bytes16 - lo < per * kBulkChunk ? bytes16 - lo : per * kBulkChunk;
      uint32_t phaseBits = 0;
      sm100::bulkPipe<kBulkStages, kBulkChunk>((char*)a.dst + lo, (const char*)a.src + lo, n, sm100::smemAddr(sm), bars, phaseBits);
    }
    if (blockIdx.x == 0)
      for (size_t j = bytes16; j < a.count; ++j) ((char*)a.dst)[j] = ((const char*)a.src)[j];
  }
}
const void* localBulkCopyKernelFn() { return (const void*)localBulkCopyKernel; }
size_t localBulkCopySmemBytes() { return 128 + (size_t)kBulkStages * kBulkChunk + kBulkStages * 8; }

const void* localCopyKernelFn(int unroll) { return unroll >= 8 ? (const void*)localCopyKernel<8> : (const void*)localCopyKernel<4>; }

// ------------------------------------------------------------------------- signals
__global__ void signalKernel(OneSignalArgs a) {
  if (threadIdx.x == 0) {
    redReleaseSysAdd64(a.target, 1);
  }
}

__global__ void waitSignalKernel(const __grid_constant__ WaitSignalArgs a) {
  int t = threadIdx.x;
  if (t < a.nDesc) {
    WaitCtx w{&a.sync, a.sync.status[a.rank]};
    const uint64_t want = *a.seen[t] + a.opCnt[t];
    const uint64_t* c = a.counter[t];
    bool ok = boundedWait(w, WAIT_SIGNAL, (uint32_t)t, (uint32_t)want, [&] { return ldRelaxedSys64(c) >= want; });
    fenceSys();
    if (ok) *a.seen[t] = want;
  }
}

const void* copyKernelFn() { return (const void*)copyCollKernel; }
const void* p2pKernelFn() { return (const void*)p2pKernel; }
const void* signalKernelFn() { return (const void*)signalKernel; }
const void* waitSignalKernelFn() { return (const void*)waitSignalKernel; }

B200_PARAM(MemSyncDomain, "MEM_SYNC_DOMAIN", 1, "Memory synchronisation domain of the communication kernels: 1 = remote (their fences do not wait for the traffic of compute kernels), 0 = default")

ncclResult_t launchKernel(const void* fn, dim3 grid, dim3 block, size_t smem, void* argStruct, cudaStream_t stream,
                          bool cooperative, bool pdl) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[3];
  int na = 0;
  if (cooperative) {
    attrs[na].id = cudaLaunchAttributeCooperative;
    attrs[na].val.cooperative = 1;
    ++na;
  }
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  // stores to peers are ordered in the "remote" memory-synchronisation domain so that fences of
  // this kernel do not wait for unrelated local traffic of concurrent compute kernels (NCCL_MEM_SYNC_DOMAIN=0: default domain)
  attrs[na].id = cudaLaunchAttributeMemSyncDomain;
  attrs[na].val.memSyncDomain = paramMemSyncDomain() ? cudaLaunchMemSyncDomainRemote : cudaLaunchMemSyncDomainDefault;
  ++na;
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  void* args[1] = {argStruct};
  cudaError_t e = cudaLaunchKernelExC(&cfg, fn, args);
  if (e != cudaSuccess) {
    WARN("kernel launch failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return ncclUnhandledCudaError;
  }
  return ncclSuccess;
}

}  // namespace b200
