/*
 * Checkpoint support: take communicators down before a process-level checkpoint (CRIU,
 * cuda-checkpoint) and bring them back afterwards, possibly in a restored process.
 *
 *   ncclCheckpointPrepare  collective; waits for the communicator's work, records how it was made
 *                          (size, rank, configuration, the user windows registered with it) and
 *                          destroys it: no sockets, threads, shared-memory names or peer mappings
 *                          of it remain in the process. Objects built on the communicator (tensor-
 *                          parallel, expert-parallel and device communicators) must be destroyed first.
 *   ncclCheckpointSave / Load   the record as a flat byte string, to keep inside or beside the image.
 *   ncclCheckpointRestore  collective; with a fresh unique id (broadcast by the application as at
 *                          start-up) it creates an equivalent communicator and registers the
 *                          recorded windows again (their memory is the application's and must exist).
 *
 * The reference ships this as an LD_PRELOAD shim around an unmodified library plus a key-value
 * store (contrib/nccl_checkpoint: shim.cc, shim_checkpoint.cc, nccl_checkpoint.h:
 * ncclCheckpointPrepare / ncclCheckpointRestore); here it is part of the library and the unique id
 * travels through the application's own launcher.
 */
#ifndef NCCL_CHECKPOINT_H_
#define NCCL_CHECKPOINT_H_
#include "nccl.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ncclCheckpointState* ncclCheckpoint_t;

ncclResult_t ncclCheckpointPrepare(ncclComm_t comm, ncclCheckpoint_t* state);
/* *bytes: in = capacity of buf, out = bytes needed / written. buf may be NULL to query the size. */
ncclResult_t ncclCheckpointSave(ncclCheckpoint_t state, void* buf, size_t* bytes);
ncclResult_t ncclCheckpointLoad(const void* buf, size_t bytes, ncclCheckpoint_t* state);
/* windows: receives up to maxWindows re-registered window handles in registration order (may be NULL). */
ncclResult_t ncclCheckpointRestore(ncclCheckpoint_t state, ncclUniqueId uniqueId, ncclComm_t* comm, ncclWindow_t* windows, int maxWindows);
ncclResult_t ncclCheckpointFree(ncclCheckpoint_t state);

#ifdef __cplusplus
}
#endif
#endif
