// Argument block of the expert-parallel dispatch / combine kernels (shared by host and device).
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "../kernels/args.h"

namespace b200 {

struct EpArgs {
  int rank, nRanks, emu;
  int numExperts, expertsPerRank, topk, hidden;
  int maxTokens;                               // capacity: tokens a rank may dispatch per call
  int fp8;                                     // dispatch payload: 1 = e4m3 + one fp32 scale per 128 channels, 0 = bf16
  int layout;                                  // EP_EXPERT_MAJOR / EP_RANK_MAJOR / EP_FLAT (see below)
  int bulkStages;                              // dispatch: > 0 = packed tokens leave through the bulk-copy engine from a ring of this many
                                               // shared-memory stages (the warps only quantise); 0 = the warps store them
  int outSlots;                                // flat layout: rows of the output tensors (tokens beyond are dropped, the total is still reported)
  int numTokens[kMaxRanks];                    // tokens of rank r in this call
  // rank-private inputs
  const __nv_bfloat16* x[kMaxRanks];           // dispatch: [numTokens, hidden]; combine: expert outputs [E_local, cap, hidden]
  const int64_t* topkIdx[kMaxRanks];           // [numTokens, topk], -1 = unused entry
  const float* topkW[kMaxRanks];               // [numTokens, topk]
  // peer-visible windows
  char* recvBuf[kMaxRanks];                    // dispatch landing zone [E_local][nRanks][maxTokens] slots
  unsigned long long* recvCount[kMaxRanks];    // [E_local][nRanks]: epoch << 32 | count
  char* combBuf[kMaxRanks];                    // combine landing zone [maxTokens][topk][hidden] bf16
  unsigned long long* combFlag[kMaxRanks];     // [nRanks]: epoch of the last completed combine per source
  // rank-private state and outputs
  uint32_t* state[kMaxRanks];                  // [0] epoch, [1] CTAs past the send phase, [2] CTAs finished, [8 ..] per-expert send counters
  void* outTokens[kMaxRanks];                  // dispatch: [E_local, cap, hidden] fp8 or bf16 ; combine: [numTokens, hidden] bf16
  float* outScales[kMaxRanks];                 // dispatch fp8: [E_local, cap, hidden/128]
  int* expertCount[kMaxRanks];                 // [E_local] tokens received per local expert
  int2* srcInfo[kMaxRanks];                    // [E_local, cap] {source rank, token * topk + k}; written by dispatch, read by combine
                                               // (rank-major / flat: [cap] {source rank or -1, token})
  long long* outTopkIdx[kMaxRanks];            // rank-major / flat: [slots, topk] expert ids of the token that are local to this rank, else -1
  float* outTopkW[kMaxRanks];                  // rank-major / flat: [slots, topk] the token's weights (may be null)
  int* recvTotal[kMaxRanks];                   // flat: number of tokens received (may be null)
  // split-phase calls and rank masks
  int phases;                                  // bit 0: sending half of the kernel, bit 1: receiving half (send_only + ncclEpComplete run them apart)
  int enableMask;                              // a wait on a rank that runs out leaves that rank out from then on instead of failing the call
  uint32_t* mask[kMaxRanks];                   // mask[r]: rank r's private [nRanks] words; non-zero = that rank is left out (no sends to it, no waits on it)
  unsigned absent;                             // emulation only: bit r set = rank r never shows up (its CTAs return at once), which makes its peers' waits run out
  SyncArgs sync;
};

// Layouts of the dispatched tokens.
//   expert-major  [local experts][capacity][hidden]: one copy of a token per selected expert, packed per expert; combine
//                 applies the weights and sums the selected experts' rows.
//   rank-major    [source ranks][max tokens][hidden]: one copy per destination RANK however many of its experts the token
//                 selected, at the row of the token's index on its source rank; unused rows have topk_idx = -1. The caller
//                 runs its local experts on a row and pre-reduces them with the weights; combine sums one row per rank.
//   flat          [received tokens][hidden]: as rank-major but packed (grouped by source rank, in arrival order).
// Reference parity: contrib/nccl_ep/include/ep_enums.h:20-122.
enum EpLayout : int { EP_EXPERT_MAJOR = 0, EP_RANK_MAJOR = 1, EP_FLAT = 2 };

// Bytes a token's routing row (top-k expert ids as int32 and weights as fp32) adds to a landing slot of the per-rank layouts.
__host__ __device__ inline size_t epMetaBytes(int topk) { return ((size_t)topk * 8 + 15) / 16 * 16; }

__host__ __device__ inline size_t epSlotBytes(int hidden, int fp8) {
  size_t b = fp8 ? (size_t)hidden + (size_t)(hidden / 128) * 4 : (size_t)hidden * 2;
  return (b + 16 + 15) / 16 * 16;              // payload + 16-byte header, 16-byte aligned
}

constexpr int kEpBulkStages = 4;
constexpr int kEpMaxLocalExperts = 256;   // experts per rank
constexpr int kEpMaxCells = 2048;         // experts per rank x ranks
// Bytes of one shared-memory stage of the dispatch kernel (one packed token, 128-byte aligned).
__host__ __device__ inline size_t epStageBytes(int hidden, int fp8) { return (epSlotBytes(hidden, fp8) - 16 + 127) / 128 * 128; }

const void* epDispatchKernelFn();
const void* epCombineKernelFn();

}  // namespace b200
