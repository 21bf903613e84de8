// All-reduce over N buffers of one GPU that never allocates memory.
//
// This entry point has no counterpart in the reference library. It exists for callers that are not
// allowed to allocate device memory at the moment they need a reduction: code running under a
// memory budget that was handed out in full at start-up (inference servers that give every byte of
// the device to their own pool), code inside an allocator or out-of-memory callback, and code on a
// path where cudaMalloc's implicit device synchronisation is unacceptable. The regular entry points
// of this library take their flagged-line buffers, epochs and status words from memory obtained
// with cudaMalloc / ncclMemAlloc when a communicator (or an emulation context) is created; this one
// keeps the same working memory in a fixed array inside the library image instead.
//
//   * What it computes: recv[r][i] = sum over p of send[p][i], for every r in [0, nRanks), with the
//     one-shot flagged-line kernel of the library (fp32 accumulation for 16-bit types, ranks added
//     in index order, identical bits in every recv[r]). One cooperative grid plays all ranks.
//   * Limits: nRanks in [1, 8]; count * sizeof(type) <= B200_NOALLOC_MAX_BYTES (4096); types fp32,
//     fp16, bf16. Anything larger is refused with ncclInvalidArgument and a message in the log;
//     nothing is launched in that case.
//   * Memory: the scratch array (B200_NOALLOC_SCRATCH_BYTES, a little over 1 MiB) is part of the
//     library image, so every GPU on which a process has loaded this library holds it until the
//     process exits, whether or not this function is ever called.
//   * First call on a device: looks up the device address of the array (cudaGetSymbolAddress, with
//     that device current) and caches it per device; that first call should come before any
//     stream capture. Every call, the first included, also synchronises `stream` and reads the
//     status words back with a blocking copy before it returns (see below).
//   * Every call uses the same array, which still holds whatever the previous call left there.
//     The words that must start at zero (the status record) are cleared on `stream` before the
//     launch; the flagged lines are never cleared because each call tags its lines with a new
//     epoch kept in the array (one epoch word for the whole call, shared by all ranks, so calls
//     with different nRanks can follow each other in any order). Two calls that overlap on the
//     GPU (different streams, or two host threads) race on the array: callers must serialise
//     calls per device.
//   * The call returns after the kernel has finished (it synchronises `stream`) so that a wait
//     that ran out of time is reported by this call: ncclTimeout, with the context still usable.
//   * It calls no cudaMalloc, cudaFree, or any library routine that allocates.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include "nccl.h"

#define B200_NOALLOC_MAX_RANKS 8
#define B200_NOALLOC_MAX_BYTES 4096
// [rank][parity 2][source 8][line 512] 16-byte lines + one 256-byte control block per rank
#define B200_NOALLOC_SCRATCH_BYTES (8 * (2 * 8 * 512 * 16 + 256))

#ifdef __cplusplus
extern "C" {
#endif

ncclResult_t b200NoAllocAllReduce(int nRanks, ncclDataType_t type, size_t count, const void* const* send, void* const* recv,
                                  cudaStream_t stream);

#ifdef __cplusplus
}
#endif
