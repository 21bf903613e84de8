// Public collective, point-to-point and one-sided entry points: each fills a Task and hands it
// to the scheduler. Argument validation follows NCCL_CHECK_MODE.
// Reference parity: src/collectives.cc:129-398 (API shims), src/misc/argcheck.cc (checks).
#include "../plugin/profiler.h"
#include "comm.h"

using namespace b200;

namespace b200 {

extern int64_t paramCheckMode();
// Pointer validation asks the driver about both buffers on every call (about a microsecond each):
// off by default like the reference's NCCL_CHECK_POINTERS (src/init.cc, src/misc/argcheck.cc).
B200_PARAM(CheckPointers, "CHECK_POINTERS", 0, "Validate send / receive pointers with the CUDA driver on every call")

ncclResult_t argCheck(const Task& t, const char* opName) {
  ncclComm* comm = t.comm;
  if (paramCheckMode() == 0) return ncclSuccess;
  if ((int)t.type < 0 || t.type >= ncclNumTypes) { WARN("%s : invalid type %d", opName, (int)t.type); return ncclInvalidArgument; }
  const bool rooted = t.func == FUNC_BROADCAST || t.func == FUNC_REDUCE || t.func == FUNC_GATHER || t.func == FUNC_SCATTER ||
                      t.func == FUNC_SEND || t.func == FUNC_RECV || t.func == FUNC_PUTSIGNAL || t.func == FUNC_SIGNAL;
  if (rooted && (t.root < 0 || t.root >= comm->nRanks)) { WARN("%s : invalid root/peer %d (root should be in the 0..%d range)", opName, t.root, comm->nRanks); return ncclInvalidArgument; }
  const bool reduces = t.func == FUNC_ALLREDUCE || t.func == FUNC_REDUCE || t.func == FUNC_REDUCESCATTER;
  if (reduces) {
    if (t.op < 0 || t.op >= ncclMaxRedOp) { WARN("%s : invalid reduction operation %d", opName, t.op); return ncclInvalidArgument; }
    if (t.op >= ncclNumOps) {
      int idx = t.op - ncclNumOps;
      if (idx >= (int)comm->userOps.size() || !comm->userOps[idx].used) { WARN("%s : reduction operation %d was not created for this communicator", opName, t.op); return ncclInvalidArgument; }
    }
  }
  if (t.count == 0) return ncclSuccess;
  if (t.func == FUNC_SIGNAL || t.func == FUNC_WAITSIGNAL) return ncclSuccess;
  const bool needSend = !(t.func == FUNC_RECV) && !((t.func == FUNC_BROADCAST || t.func == FUNC_SCATTER) && comm->rank != t.root);
  const bool needRecv = !(t.func == FUNC_SEND || t.func == FUNC_PUTSIGNAL) && !((t.func == FUNC_REDUCE || t.func == FUNC_GATHER) && comm->rank != t.root);
  if (needSend && !t.send) { WARN("%s : sendbuff is NULL", opName); return ncclInvalidArgument; }
  if (needRecv && !t.recv) { WARN("%s : recvbuff is NULL", opName); return ncclInvalidArgument; }
  if (!comm->hostOnly && paramCheckPointers()) {
    // pointers must be device-accessible memory of this communicator's device
    auto check = [&](const void* p, const char* what) -> ncclResult_t {
      cudaPointerAttributes attr;
      cudaError_t e = cudaPointerGetAttributes(&attr, p);
      if (e != cudaSuccess) { (void)cudaGetLastError(); WARN("%s : %s %p is not a valid pointer", opName, what, p); return ncclInvalidArgument; }
      if (attr.type == cudaMemoryTypeUnregistered) { WARN("%s : %s %p is pageable host memory", opName, what, p); return ncclInvalidArgument; }
      if (attr.type == cudaMemoryTypeDevice && attr.device != comm->cudaDev) {
        WARN("%s : %s allocated on device %d mismatches with NCCL device %d", opName, what, attr.device, comm->cudaDev);
        return ncclInvalidArgument;
      }
      return ncclSuccess;
    };
    if (needSend) NCCLCHECK(check(t.send, "sendbuff"));
    if (needRecv) NCCLCHECK(check(t.recv, "recvbuff"));
  }
  return ncclSuccess;
}

static ncclResult_t submit(int func, const void* send, void* recv, size_t count, ncclDataType_t type, int op, int root,
                           ncclComm_t comm, cudaStream_t stream) {
  if (!commValid(comm)) { WARN("%s : invalid communicator", funcName(func)); return ncclInvalidArgument; }
  Task t{};
  t.func = func;
  t.send = send;
  t.recv = recv;
  t.count = count;
  t.type = type;
  t.op = op;
  t.root = root;
  t.comm = comm;
  t.stream = stream;
  ProfilerApiScope scope(comm, t);
  return enqueueTask(t);
}

}  // namespace b200

extern "C" {

ncclResult_t ncclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
  return submit(FUNC_ALLREDUCE, sendbuff, recvbuff, count, datatype, op, 0, comm, stream);
}
ncclResult_t ncclReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, int root, ncclComm_t comm, cudaStream_t stream) {
  return submit(FUNC_REDUCE, sendbuff, recvbuff, count, datatype, op, root, comm, stream);
}
ncclResult_t ncclBroadcast(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
  return submit(FUNC_BROADCAST, sendbuff, recvbuff, count, datatype, ncclSum, root, comm, stream);
}
ncclResult_t ncclBcast(void* buff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
  return ncclBroadcast(buff, buff, count, datatype, root, comm, stream);
}
ncclResult_t ncclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
  return submit(FUNC_REDUCESCATTER, sendbuff, recvbuff, recvcount, datatype, op, 0, comm, stream);
}
ncclResult_t ncclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream) {
  return submit(FUNC_ALLGATHER, sendbuff, recvbuff, sendcount, datatype, ncclSum, 0, comm, stream);
}
ncclResult_t ncclAlltoAll(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream) {
  return submit(FUNC_ALLTOALL, sendbuff, recvbuff, count, datatype, ncclSum, 0, comm, stream);
}
ncclResult_t ncclGather(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
  return submit(FUNC_GATHER, sendbuff, recvbuff, count, datatype, ncclSum, root, comm, stream);
}
ncclResult_t ncclScatter(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
  return submit(FUNC_SCATTER, sendbuff, recvbuff, count, datatype, ncclSum, root, comm, stream);
}
ncclResult_t ncclSend(const void* sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream) {
  return submit(FUNC_SEND, sendbuff, nullptr, count, datatype, ncclSum, peer, comm, stream);
}
ncclResult_t ncclRecv(void* recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream) {
  return submit(FUNC_RECV, nullptr, recvbuff, count, datatype, ncclSum, peer, comm, stream);
}

ncclResult_t ncclPutSignal(const void* localbuff, size_t count, ncclDataType_t datatype, int peer, ncclWindow_t peerWin, size_t peerWinOffset,
                           int sigIdx, int ctx, unsigned int flags, ncclComm_t comm, cudaStream_t stream) {
  if (!commValid(comm)) return ncclInvalidArgument;
  if (flags != 0) { WARN("ncclPutSignal : flags must be 0"); return ncclInvalidArgument; }
  Task t{};
  t.func = FUNC_PUTSIGNAL;
  t.send = localbuff;
  t.count = count;
  t.type = datatype;
  t.root = peer;
  t.comm = comm;
  t.stream = stream;
  t.win = peerWin;
  t.winOffset = peerWinOffset;
  t.sigIdx = sigIdx;
  t.ctx = ctx;
  return enqueueTask(t);
}
ncclResult_t ncclSignal(int peer, int sigIdx, int ctx, unsigned int flags, ncclComm_t comm, cudaStream_t stream) {
  if (!commValid(comm)) return ncclInvalidArgument;
  if (flags != 0) { WARN("ncclSignal : flags must be 0"); return ncclInvalidArgument; }
  Task t{};
  t.func = FUNC_SIGNAL;
  t.root = peer;
  t.comm = comm;
  t.stream = stream;
  t.sigIdx = sigIdx;
  t.ctx = ctx;
  t.type = ncclInt8;
  return enqueueTask(t);
}
ncclResult_t ncclWaitSignal(int nDesc, ncclWaitSignalDesc_t* signalDescs, ncclComm_t comm, cudaStream_t stream) {
  if (!commValid(comm)) return ncclInvalidArgument;
  if (nDesc <= 0 || !signalDescs) { WARN("ncclWaitSignal : no descriptors"); return ncclInvalidArgument; }
  // one task per descriptor; they are waited for together by the same kernel when grouped
  ncclResult_t r = ncclSuccess;
  groupStart();
  for (int i = 0; i < nDesc && r == ncclSuccess; ++i) {
    Task t{};
    t.func = FUNC_WAITSIGNAL;
    t.root = signalDescs[i].peer;
    t.comm = comm;
    t.stream = stream;
    t.sigIdx = signalDescs[i].sigIdx;
    t.ctx = signalDescs[i].ctx;
    t.opCnt = signalDescs[i].opCnt;
    t.type = ncclInt8;
    if (t.root < 0 || t.root >= comm->nRanks) { WARN("ncclWaitSignal : invalid peer %d", t.root); r = ncclInvalidArgument; break; }
    r = enqueueTask(t);
  }
  ncclResult_t e = groupEnd(nullptr);
  return r != ncclSuccess ? r : e;
}

ncclResult_t pncclAllReduce(const void* s, void* r, size_t c, ncclDataType_t t, ncclRedOp_t o, ncclComm_t comm, cudaStream_t st) { return ncclAllReduce(s, r, c, t, o, comm, st); }
ncclResult_t pncclReduce(const void* s, void* r, size_t c, ncclDataType_t t, ncclRedOp_t o, int root, ncclComm_t comm, cudaStream_t st) { return ncclReduce(s, r, c, t, o, root, comm, st); }
ncclResult_t pncclBroadcast(const void* s, void* r, size_t c, ncclDataType_t t, int root, ncclComm_t comm, cudaStream_t st) { return ncclBroadcast(s, r, c, t, root, comm, st); }
ncclResult_t pncclBcast(void* b, size_t c, ncclDataType_t t, int root, ncclComm_t comm, cudaStream_t st) { return ncclBcast(b, c, t, root, comm, st); }
ncclResult_t pncclReduceScatter(const void* s, void* r, size_t c, ncclDataType_t t, ncclRedOp_t o, ncclComm_t comm, cudaStream_t st) { return ncclReduceScatter(s, r, c, t, o, comm, st); }
ncclResult_t pncclAllGather(const void* s, void* r, size_t c, ncclDataType_t t, ncclComm_t comm, cudaStream_t st) { return ncclAllGather(s, r, c, t, comm, st); }
ncclResult_t pncclAlltoAll(const void* s, void* r, size_t c, ncclDataType_t t, ncclComm_t comm, cudaStream_t st) { return ncclAlltoAll(s, r, c, t, comm, st); }
ncclResult_t pncclGather(const void* s, void* r, size_t c, ncclDataType_t t, int root, ncclComm_t comm, cudaStream_t st) { return ncclGather(s, r, c, t, root, comm, st); }
ncclResult_t pncclScatter(const void* s, void* r, size_t c, ncclDataType_t t, int root, ncclComm_t comm, cudaStream_t st) { return ncclScatter(s, r, c, t, root, comm, st); }
ncclResult_t pncclSend(const void* s, size_t c, ncclDataType_t t, int p, ncclComm_t comm, cudaStream_t st) { return ncclSend(s, c, t, p, comm, st); }
ncclResult_t pncclRecv(void* r, size_t c, ncclDataType_t t, int p, ncclComm_t comm, cudaStream_t st) { return ncclRecv(r, c, t, p, comm, st); }
ncclResult_t pncclPutSignal(const void* l, size_t c, ncclDataType_t t, int p, ncclWindow_t w, size_t o, int s, int x, unsigned int f, ncclComm_t comm, cudaStream_t st) { return ncclPutSignal(l, c, t, p, w, o, s, x, f, comm, st); }
ncclResult_t pncclSignal(int p, int s, int x, unsigned int f, ncclComm_t comm, cudaStream_t st) { return ncclSignal(p, s, x, f, comm, st); }
ncclResult_t pncclWaitSignal(int n, ncclWaitSignalDesc_t* d, ncclComm_t comm, cudaStream_t st) { return ncclWaitSignal(n, d, comm, st); }

}  // extern "C"
