// Mesh-to-mesh resharding: see include/nccl_m2n.h. With a window that holds the source tiles every destination rank pulls
// its runs with one kernel (reshardKernel in kernels/copy.cu); without one the runs move as grouped send / receive.
// Reference parity: contrib/nccl_m2n (ncclReshardWithWindow, src/nccl_m2n.h:175; mesh / placement
// model of its README "Concepts"); the reference moves data with one-sided kernels over windows and
// adds hierarchical routing for multi-node NVLink domains, which a single node does not need.
#include "nccl_m2n.h"

#include <algorithm>
#include <map>
#include <mutex>
#include <vector>

#include "../comm/comm.h"
#include "../comm/device_plane.h"
#include "../kernels/args.h"
#include "../mem/symmetric.h"

using namespace b200;

namespace {

struct Side {
  const ncclMesh_t* mesh;
  int nRanks;
  int shardAxis;      // mesh axis that shards
  int shardDim;       // tensor dimension it shards
  int shards;         // number of shards
  int replicas;       // ranks holding each shard
  size_t local[NCCL_RESHARD_MAX_TENSOR_DIMS];
};

ncclResult_t describe(const ncclDistTensor_t* t, const char* which, Side* s) {
  const ncclMesh_t* m = t->mesh;
  if (!m || m->dims[0] <= 0 || m->dims[1] <= 0 || m->startRank < 0) { WARN("ncclReshardWithWindow: %s mesh is malformed", which); return ncclInvalidArgument; }
  s->mesh = m;
  s->nRanks = m->dims[0] * m->dims[1];
  int sharding = 0;
  s->shardAxis = -1;
  for (int a = 0; a < 2; ++a) {
    if (m->placement[a] == NCCL_RESHARD_REPLICATE) continue;
    if (m->placement[a] < 0 || m->placement[a] >= t->ndims) { WARN("ncclReshardWithWindow: %s placement[%d] names tensor dimension %d of %d", which, a, m->placement[a], t->ndims); return ncclInvalidArgument; }
    ++sharding;
    s->shardAxis = a;
  }
  if (sharding > 1) { WARN("ncclReshardWithWindow: %s mesh shards on both axes; exactly one axis may shard", which); return ncclInvalidArgument; }
  if (sharding == 0) {   // fully replicated: one shard covering everything
    s->shardAxis = 0;
    s->shardDim = 0;
    s->shards = 1;
    s->replicas = s->nRanks;
  } else {
    s->shardDim = m->placement[s->shardAxis];
    s->shards = m->dims[s->shardAxis];
    s->replicas = s->nRanks / s->shards;
  }
  for (int d = 0; d < NCCL_RESHARD_MAX_TENSOR_DIMS; ++d) s->local[d] = d < t->ndims ? t->localShape[d] : 1;
  return ncclSuccess;
}

// shard index and replica index of world rank r on this side (-1 when r is not on it)
bool locate(const Side& s, int r, int* shard, int* replica) {
  const int idx = r - s.mesh->startRank;
  if (idx < 0 || idx >= s.nRanks) return false;
  const int c[2] = {idx / s.mesh->dims[1], idx % s.mesh->dims[1]};
  if (s.shards == 1) { *shard = 0; *replica = idx; return true; }
  *shard = c[s.shardAxis];
  *replica = c[1 - s.shardAxis];
  return true;
}
int rankOf(const Side& s, int shard, int replica) {
  if (s.shards == 1) return s.mesh->startRank + replica;
  int c[2];
  c[s.shardAxis] = shard;
  c[1 - s.shardAxis] = replica;
  return s.mesh->startRank + c[0] * s.mesh->dims[1] + c[1];
}

struct Run { size_t srcOff, dstOff, count; };   // element offsets into the local tiles

// Contiguous runs of the intersection of source shard `ss` and destination shard `ds`, in canonical order.
void runsOf(const Side& S, const Side& D, int ndims, const size_t* global, int ss, int ds, std::vector<Run>* out) {
  size_t lo[3] = {0, 0, 0}, hi[3] = {1, 1, 1};
  size_t sOrg[3] = {0, 0, 0}, dOrg[3] = {0, 0, 0};
  for (int d = 0; d < ndims; ++d) hi[d] = global[d];
  if (S.shards > 1) { sOrg[S.shardDim] = (size_t)ss * S.local[S.shardDim]; lo[S.shardDim] = std::max(lo[S.shardDim], sOrg[S.shardDim]); hi[S.shardDim] = std::min(hi[S.shardDim], sOrg[S.shardDim] + S.local[S.shardDim]); }
  if (D.shards > 1) { dOrg[D.shardDim] = (size_t)ds * D.local[D.shardDim]; lo[D.shardDim] = std::max(lo[D.shardDim], dOrg[D.shardDim]); hi[D.shardDim] = std::min(hi[D.shardDim], dOrg[D.shardDim] + D.local[D.shardDim]); }
  for (int d = 0; d < ndims; ++d) if (lo[d] >= hi[d]) return;
  // view everything as 3-D with leading extents of 1
  size_t sl[3] = {1, 1, 1}, dl[3] = {1, 1, 1}, b0[3] = {0, 0, 0}, b1[3] = {1, 1, 1}, so[3] = {0, 0, 0}, dof[3] = {0, 0, 0};
  const int pad = 3 - ndims;
  for (int d = 0; d < ndims; ++d) { sl[pad + d] = S.local[d]; dl[pad + d] = D.local[d]; b0[pad + d] = lo[d]; b1[pad + d] = hi[d]; so[pad + d] = sOrg[d]; dof[pad + d] = dOrg[d]; }
  const size_t len = b1[2] - b0[2];
  for (size_t i = b0[0]; i < b1[0]; ++i)
    for (size_t j = b0[1]; j < b1[1]; ++j) {
      Run r;
      r.srcOff = ((i - so[0]) * sl[1] + (j - so[1])) * sl[2] + (b0[2] - so[2]);
      r.dstOff = ((i - dof[0]) * dl[1] + (j - dof[1])) * dl[2] + (b0[2] - dof[2]);
      r.count = len;
      // merge with the previous run when both sides continue without a gap
      if (!out->empty() && out->back().srcOff + out->back().count == r.srcOff && out->back().dstOff + out->back().count == r.dstOff) out->back().count += len;
      else out->push_back(r);
    }
}

size_t elemSize(ncclDataType_t t) {
  switch (t) {
    case ncclInt8: case ncclUint8: case ncclFloat8e4m3: case ncclFloat8e5m2: return 1;
    case ncclFloat16: case ncclBfloat16: return 2;
    case ncclInt32: case ncclUint32: case ncclFloat32: return 4;
    default: return 8;
  }
}

// Device words of a communicator for the offset exchange: [0] this rank's offset, [8 ..) the gathered table.
std::mutex gWordsLock;
std::map<ncclComm*, unsigned long long*> gWords;
ncclResult_t m2nWords(ncclComm* comm, unsigned long long** out) {
  std::lock_guard<std::mutex> g(gWordsLock);
  unsigned long long*& w = gWords[comm];
  if (!w) {
    CUDACHECK(cudaMalloc((void**)&w, (8 + kMaxRanks) * sizeof(unsigned long long)));
    CUDACHECK(cudaMemset(w, 0, (8 + kMaxRanks) * sizeof(unsigned long long)));
  }
  *out = w;
  return ncclSuccess;
}

}  // namespace

namespace b200 {
void m2nCommRelease(ncclComm* comm) {
  std::lock_guard<std::mutex> g(gWordsLock);
  auto it = gWords.find(comm);
  if (it == gWords.end()) return;
  cudaFree(it->second);
  (void)cudaGetLastError();
  gWords.erase(it);
}
}  // namespace b200

extern "C" {

ncclResult_t ncclM2nInit(ncclM2nConfig_t* config) {
  if (config && (config->magic != NCCL_M2N_API_MAGIC || config->size != sizeof(ncclM2nConfig_t))) return ncclInvalidArgument;
  return ncclSuccess;
}
ncclResult_t ncclM2nFinalize(void) { return ncclSuccess; }

ncclResult_t ncclReshardWithWindow(ncclComm_t comm, ncclWindow_t window, const ncclDistTensor_t* src, const ncclDistTensor_t* dst, cudaStream_t stream) {
  if (!commValid(comm) || !src || !dst) return ncclInvalidArgument;
  if (src->ndims != dst->ndims || src->dtype != dst->dtype || src->ndims < 1 || src->ndims > NCCL_RESHARD_MAX_TENSOR_DIMS) {
    WARN("ncclReshardWithWindow: source and destination must agree on 1 to 3 dimensions and on the data type");
    return ncclInvalidArgument;
  }
  Side S, D;
  NCCLCHECK(describe(src, "source", &S));
  NCCLCHECK(describe(dst, "destination", &D));
  if (S.mesh->startRank + S.nRanks > comm->nRanks || D.mesh->startRank + D.nRanks > comm->nRanks) { WARN("ncclReshardWithWindow: a mesh reaches beyond the communicator"); return ncclInvalidArgument; }
  const int nd = src->ndims;
  // Every rank must be able to compute the plan, so the tile shapes of both sides have to be known
  // everywhere: ranks that are not on a side still pass that side's localShape.
  size_t gS[3], gD[3];
  for (int d = 0; d < nd; ++d) {
    gS[d] = S.local[d] * (S.shards > 1 && d == S.shardDim ? S.shards : 1);
    gD[d] = D.local[d] * (D.shards > 1 && d == D.shardDim ? D.shards : 1);
    if (gS[d] != gD[d]) { WARN("ncclReshardWithWindow: global extent of dimension %d differs (source %zu, destination %zu)", d, gS[d], gD[d]); return ncclInvalidArgument; }
  }
  const size_t es = elemSize(src->dtype);
  int mySS = -1, mySR = -1, myDS = -1, myDR = -1;
  const bool onS = locate(S, comm->rank, &mySS, &mySR) && src->dataPtr;
  const bool onD = locate(D, comm->rank, &myDS, &myDR) && dst->dataPtr;
  // ---- with a window that holds the source tiles, on GPUs that map each other: one pull kernel per rank
  // (every rank passes the window or none does: the choice below must be the same everywhere)
  if (window && !comm->hostOnly && comm->devPlane && (comm->nRanks == 1 || comm->lsaAll) && groupDepth() == 0) {
    if (window->magic != kWindowMagic || !window->hostState) { WARN("ncclReshardWithWindow: not a window handle"); return ncclInvalidArgument; }
    SymWindow* w = (SymWindow*)window->hostState;
    unsigned long long myOff = 0;
    if (onS) {
      const char* base = (const char*)w->host.userPtr;
      size_t tileBytes = es;
      for (int d = 0; d < nd; ++d) tileBytes *= S.local[d];
      if ((const char*)src->dataPtr < base || (const char*)src->dataPtr + tileBytes > base + w->host.size) {
        WARN("ncclReshardWithWindow: the source tile does not lie inside the window");
        return ncclInvalidArgument;
      }
      myOff = (unsigned long long)((const char*)src->dataPtr - base);
    }
    std::vector<ReshardRun> pulls;
    size_t dstTileBytes = es;
    for (int d = 0; d < nd; ++d) dstTileBytes *= D.local[d];
    if (onD) {
      for (int ss = 0; ss < S.shards; ++ss) {
        const int dr = comm->rank - D.mesh->startRank;
        const int sRank = rankOf(S, ss, dr % S.replicas);
        std::vector<Run> runs;
        runsOf(S, D, nd, gS, ss, myDS, &runs);
        for (const Run& r : runs) pulls.push_back(ReshardRun{r.srcOff * es, r.dstOff * es, r.count * es, sRank, 0});
      }
    }
    // where every rank's source tile sits inside the window: eight bytes per rank, gathered on the stream
    unsigned long long* words = nullptr;
    NCCLCHECK(m2nWords(comm, &words));
    CUDACHECK(cudaMemcpyAsync(words, &myOff, sizeof(myOff), cudaMemcpyHostToDevice, stream));
    NCCLCHECK(ncclAllGather(words, words + 8, sizeof(myOff), ncclUint8, comm, stream));
    return devPlaneRunReshard(comm, w, pulls.data(), (int)pulls.size(), words + 8, onD ? dst->dataPtr : nullptr, dstTileBytes, stream);
  }

  struct Op { bool send; int peer; void* p; size_t count; };
  std::vector<Op> ops;
  // canonical order: destination ranks ascending, then source shards ascending, then runs
  for (int dr = 0; dr < D.nRanks; ++dr) {
    const int dRank = D.mesh->startRank + dr;
    int ds, drep;
    locate(D, dRank, &ds, &drep);
    for (int ss = 0; ss < S.shards; ++ss) {
      const int sRank = rankOf(S, ss, dr % S.replicas);   // replicas of a slice serve destinations round-robin
      const bool iSend = onS && comm->rank == sRank, iRecv = onD && comm->rank == dRank;
      if (!iSend && !iRecv) continue;
      std::vector<Run> runs;
      runsOf(S, D, nd, gS, ss, ds, &runs);
      for (const Run& r : runs) {
        if (sRank == dRank) {   // both tiles are local: plain copy
          if (iSend) ops.push_back(Op{true, dRank, (char*)src->dataPtr + r.srcOff * es, r.count});
          if (iRecv) ops.push_back(Op{false, sRank, (char*)dst->dataPtr + r.dstOff * es, r.count});
          continue;
        }
        if (iSend) ops.push_back(Op{true, dRank, (char*)src->dataPtr + r.srcOff * es, r.count});
        if (iRecv) ops.push_back(Op{false, sRank, (char*)dst->dataPtr + r.dstOff * es, r.count});
      }
    }
  }
  // Groups keep sends and receives of one peer pair in posting order; a bounded number of operations per group.
  const size_t kPerGroup = 24;
  // All ranks must run the same number of groups only if groups synchronise ranks; they do not
  // (a group only batches this rank's own operations), so each rank batches its own list.
  for (size_t i = 0; i < ops.size(); i += kPerGroup) {
    NCCLCHECK(ncclGroupStart());
    ncclResult_t r = ncclSuccess;
    for (size_t k = i; k < std::min(ops.size(), i + kPerGroup) && r == ncclSuccess; ++k) {
      const Op& o = ops[k];
      r = o.send ? ncclSend(o.p, o.count, src->dtype, o.peer, comm, stream) : ncclRecv(o.p, o.count, src->dtype, o.peer, comm, stream);
    }
    ncclResult_t e = ncclGroupEnd();
    if (r != ncclSuccess) return r;
    NCCLCHECK(e);
  }
  return ncclSuccess;
}

}  // extern "C"
