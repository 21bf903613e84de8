/*
 * All-reduce of data that lives in pinned host memory: the input is copied to the device, reduced across the ranks
 * and the result copied back to the host, in chunks, so that the host-to-device copy of chunk i + 1, the all-reduce
 * of chunk i and the device-to-host copy of chunk i - 1 run at the same time (the two copy directions of PCIe are
 * independent, and the collective hides behind them). For callers whose tensors are produced and consumed on the host
 * (parameter servers, CPU optimisers, offloaded gradients). Without a counterpart in the reference, whose callers
 * write the three steps one after the other.
 */
#ifndef NCCL_HOST_STAGED_H_
#define NCCL_HOST_STAGED_H_
#include "nccl.h"

#ifdef __cplusplus
extern "C" {
#endif
/* hostSend / hostRecv: page-locked host buffers of `count` elements (may be the same buffer).
 * devSend / devRecv: device buffers of `count` elements used as staging (may be the same buffer; registered windows make
 * the collective zero-copy). chunkBytes: 0 = default (32 MiB). All work is ordered after what `stream` holds at the time
 * of the call, and `stream` is made to wait for the last device-to-host copy, so an event recorded on `stream` afterwards
 * covers the whole operation. */
ncclResult_t ncclAllReduceFromHost(const void* hostSend, void* hostRecv, void* devSend, void* devRecv, size_t count, ncclDataType_t datatype,
                                   ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream, size_t chunkBytes);
#ifdef __cplusplus
}
#endif
#endif
