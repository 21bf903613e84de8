// Internal interface between the tensor-parallel host code and its sm_100a kernels.
#pragma once
#include "../kernels/args.h"

namespace b200 {

enum TpMode : int {
  TP_MODE_STORE = 0,    // C = A * W^T, stored locally
  TP_MODE_REDUCE = 1,   // GEMM -> reduce-scatter: bf16 partial tiles are stored into the owner's staging buffer, summed there afterwards
  TP_MODE_GATHER = 2,   // all-gather -> GEMM: comm CTAs pull remote row blocks while the GEMM runs
};

struct TpGemmArgs {
  void* C;                        // bf16 output [M, ldc] (STORE / GATHER)
  int ldc;
  void* partial[kMaxRanks];       // REDUCE: partial[p] = rank p's staging buffer, bf16 [nRanks sources][M / nRanks][N], mapped here
  const void* peerA[kMaxRanks];   // GATHER: peerA[p] = rank p's A buffer [M, K] bf16, mapped here
  uint32_t* blockFlags;           // GATHER: one word per 128-row block of A, set to flagEpoch when landed
  uint32_t flagEpoch;
  int M, N, K;
  int mode;
  int rank, nRanks;
  int gemmCtas;                   // GATHER: CTAs [0, gemmCtas) compute, the rest gather
  SyncArgs sync;
  // block-scaled fp8 (e4m3) operands: A scaled per row and 128 columns, W per 128 x 128 block
  const float* scaleA;            // [K/128][M]   (for GATHER: inside the gathered window, see scaleOffset)
  const float* scaleW;            // [K/128][N/128]
  size_t scaleOffset;             // GATHER, fp8: byte offset of the scales inside every rank's activation window
};

#if defined(__CUDACC__)
constexpr int kTpBM = 128, kTpBN = 256;
struct TileCoord { int mBlk, nBlk, owner; };
// Tile j of a block of `rows` x `tilesN` tiles, visited in panels of kTpPanel tile columns, row by row
// inside a panel: the tiles in flight at any time (one per CTA or CTA pair) then cover a roughly square
// region, so every operand tile fetched into L2 is reused by several CTAs before it is evicted, instead
// of streaming the whole of W once per tile row.
constexpr int kTpPanel = 8;
constexpr int kTpChunkRows = 2048;   // rows of one owner walked together in the fused modes
__device__ __forceinline__ void panelOrder(int j, int rows, int tilesN, int* r, int* c) {
  const int perPanel = kTpPanel * rows;
  const int p = j / perPanel;
  const int width = tilesN - p * kTpPanel < kTpPanel ? tilesN - p * kTpPanel : kTpPanel;
  const int k = j - p * perPanel;
  *r = k / width;
  *c = p * kTpPanel + k % width;
}
// Tile t of this CTA's walk: the whole output for plain GEMMs; owner by owner for the fused modes
// (REDUCE starts with the next rank so that every step each GPU receives from one peer; GATHER
// starts with the rows that are already local), panel order inside each block of rows.
// `bm` is the tile height in rows (128 for one CTA, 256 for a CTA pair); mBlk counts tiles of that height.
__device__ __forceinline__ TileCoord tileOf(const TpGemmArgs& a, int t, int bm = kTpBM) {
  const int tilesN = a.N / kTpBN;
  TileCoord c;
  if (a.mode == TP_MODE_STORE || a.nRanks == 1) {
    panelOrder(t, a.M / bm, tilesN, &c.mBlk, &c.nBlk);
    c.owner = a.rank;
    if (a.mode == TP_MODE_REDUCE) c.owner = 0;
    return c;
  }
  const int tilesMPerRank = a.M / a.nRanks / bm;
  const int per = tilesMPerRank * tilesN;
  const int step = t / per, j = t % per;
  const int who = a.mode == TP_MODE_REDUCE ? (a.rank + 1 + step) % a.nRanks : (a.rank + step) % a.nRanks;
  // an owner's rows are walked in chunks of kTpChunkRows rows, panel order inside a chunk: all-gather -> GEMM then
  // needs a peer's rows chunk by chunk instead of all of them for the first panel
  const int chunkTiles = kTpChunkRows / bm;
  const int chunk = j / (chunkTiles * tilesN);
  const int rowsHere = tilesMPerRank - chunk * chunkTiles < chunkTiles ? tilesMPerRank - chunk * chunkTiles : chunkTiles;
  int r;
  panelOrder(j - chunk * chunkTiles * tilesN, rowsHere, tilesN, &r, &c.nBlk);
  r += chunk * chunkTiles;
  c.owner = who;
  c.mBlk = who * tilesMPerRank + r;
  return c;
}
#endif

const void* tpGemmKernelFn();
const void* tpGemmPairKernelFn();      // CTA-pair variant (cluster of two, 256 x 256 tiles): same arguments, W map with 128-row boxes
const void* tpGemmFp8KernelFn();
const void* tpQuantRowsKernelFn();     // (const bf16* x, uint8_t* q, float* scales, int rows, int K): 1 x 128 blocks, scales [K/128][rows]
const void* tpQuantBlocksKernelFn();   // same arguments: 128 x 128 blocks, scales [K/128][rows/128]
size_t tpGemmFp8SmemBytes();
int tpGemmFp8Threads();
const void* tpReduceKernelFn();        // (const bf16* staged, bf16* out, size_t count, int nSources): out = sum over sources, fp32 accumulation
size_t tpGemmSmemBytes();
size_t tpGemmPairSmemBytes();
int tpGemmPairThreads();
int tpGemmThreads();

}  // namespace b200
