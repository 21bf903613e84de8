/*
 * Checkpoint support: release what the library holds on the GPU (and, for a restore in another process, the
 * communicator itself) before a process-level checkpoint (cuda-checkpoint, CRIU) and bring it back afterwards.
 *
 * Process-wide calls, with the signatures of the reference's contrib/nccl_checkpoint (nccl_checkpoint.h:22-24;
 * there they live in an LD_PRELOAD shim around the library, here they are part of it):
 *   ncclCheckpointPrepare()   collective over every communicator of the process, in creation order: drains each GPU
 *                             communicator and releases the library's device memory and peer mappings. All
 *                             ncclComm_t handles stay valid.
 *   ncclCheckpointRestore()   maps everything again; collectives may be issued afterwards.
 *   ncclCheckpointGetVersion()
 * ncclCheckpointApi and its helpers resolve these at run time, for applications that must not link them.
 *
 * Per-communicator calls, for a restore that needs a new rendezvous (another process or host):
 *   ncclCommCheckpointPrepare  collective; waits for the communicator's work, records how it was made (size, rank,
 *                              configuration, the user windows registered with it) and destroys it: no sockets,
 *                              threads, shared-memory names or peer mappings of it remain. Objects built on the
 *                              communicator (tensor-parallel, expert-parallel, device communicators) go first.
 *   ncclCommCheckpointSave / Load   the record as a flat byte string, to keep inside or beside the image.
 *   ncclCommCheckpointRestore  collective; with a fresh unique id (broadcast by the application as at start-up) it
 *                              creates an equivalent communicator and registers the recorded windows again (their
 *                              memory is the application's and must exist).
 */
#ifndef NCCL_CHECKPOINT_H_
#define NCCL_CHECKPOINT_H_
#include <dlfcn.h>
#include <stddef.h>

#include "nccl.h"

#define NCCL_CHECKPOINT_VERSION 1

#ifdef __cplusplus
extern "C" {
#endif

/* ---- process-wide */
ncclResult_t ncclCheckpointPrepare(void);
ncclResult_t ncclCheckpointRestore(void);
ncclResult_t ncclCheckpointGetVersion(int* checkpointVersion, int* ncclVersion);

typedef ncclResult_t (*ncclCheckpointPrepareFn)(void);
typedef ncclResult_t (*ncclCheckpointRestoreFn)(void);
typedef ncclResult_t (*ncclCheckpointGetVersionFn)(int* checkpointVersion, int* ncclVersion);
typedef struct ncclCheckpointApi {
  ncclCheckpointPrepareFn prepare;
  ncclCheckpointRestoreFn restore;
  ncclCheckpointGetVersionFn getVersion;
} ncclCheckpointApi;

static inline void ncclCheckpointApiClear(ncclCheckpointApi* api) {
  if (api) { api->prepare = NULL; api->restore = NULL; api->getVersion = NULL; }
}
static inline int ncclCheckpointApiIsLoaded(const ncclCheckpointApi* api) {
  return api && api->prepare && api->restore && api->getVersion;
}
/* 0 when all three entry points were found among the loaded libraries */
static inline int ncclCheckpointApiLoad(ncclCheckpointApi* api) {
  if (!api) return 1;
  api->prepare = (ncclCheckpointPrepareFn)dlsym(RTLD_DEFAULT, "ncclCheckpointPrepare");
  api->restore = (ncclCheckpointRestoreFn)dlsym(RTLD_DEFAULT, "ncclCheckpointRestore");
  api->getVersion = (ncclCheckpointGetVersionFn)dlsym(RTLD_DEFAULT, "ncclCheckpointGetVersion");
  return ncclCheckpointApiIsLoaded(api) ? 0 : 1;
}

/* ---- per communicator */
typedef struct ncclCheckpointState* ncclCheckpoint_t;

ncclResult_t ncclCommCheckpointPrepare(ncclComm_t comm, ncclCheckpoint_t* state);
/* *bytes: in = capacity of buf, out = bytes needed / written. buf may be NULL to query the size. */
ncclResult_t ncclCommCheckpointSave(ncclCheckpoint_t state, void* buf, size_t* bytes);
ncclResult_t ncclCommCheckpointLoad(const void* buf, size_t bytes, ncclCheckpoint_t* state);
/* windows: receives up to maxWindows re-registered window handles in registration order (may be NULL). */
ncclResult_t ncclCommCheckpointRestore(ncclCheckpoint_t state, ncclUniqueId uniqueId, ncclComm_t* comm, ncclWindow_t* windows, int maxWindows);
ncclResult_t ncclCommCheckpointFree(ncclCheckpoint_t state);

#ifdef __cplusplus
}
#endif
#endif
