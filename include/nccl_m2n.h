/*
 * Resharding between two device meshes (M ranks -> N ranks), e.g. from a training layout to an
 * inference layout: every destination rank receives exactly the slice of the global tensor that its
 * placement asks for, from source ranks that hold it. Descriptors follow the reference's public
 * header (contrib/nccl_m2n/src/nccl_m2n.h): a 2-D mesh over a contiguous rank interval, one mesh
 * axis sharding one tensor dimension and the other replicating; tensors of 1 to 3 dimensions,
 * row-major local tiles.
 *
 * The plan is computed identically on every rank from the two descriptors (replicas of a source slice
 * are dealt round-robin to the destination ranks that need it). With `window` = a registered window
 * that contains the source tile of every source rank (all ranks pass it, or none), every destination
 * rank pulls its contiguous runs out of the sources' tiles with peer loads in one kernel. With
 * `window` = NULL, or on ranks that cannot map each other, the runs move as grouped ncclSend / ncclRecv.
 */
#ifndef NCCL_M2N_H_
#define NCCL_M2N_H_
#include <limits.h>
#include <stddef.h>

#include "nccl.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  int dims[2];        /* mesh extents; dims[0] * dims[1] ranks, row-major: rank = startRank + i * dims[1] + j */
  int startRank;
  int placement[2];   /* per mesh axis: NCCL_RESHARD_REPLICATE or NCCL_RESHARD_SHARD(tensor dimension) */
} ncclMesh_t;

#define NCCL_RESHARD_REPLICATE (-1)
#define NCCL_RESHARD_SHARD(td) (td)
#define NCCL_RESHARD_MAX_TENSOR_DIMS 3

typedef struct {
  void* dataPtr;                                      /* local tile, or NULL when this rank is not on this side */
  size_t localShape[NCCL_RESHARD_MAX_TENSOR_DIMS];    /* elements per dimension of the local tile */
  int ndims;
  ncclDataType_t dtype;
  const ncclMesh_t* mesh;                             /* required on every rank */
} ncclDistTensor_t;

#define NCCL_M2N_CONFIG_UNDEF_INT INT_MIN
#define NCCL_M2N_API_MAGIC 0x4d324e00u

typedef struct ncclM2nConfig_v1 {
  size_t size;
  unsigned int magic;
  int maxCta;
} ncclM2nConfig_t;

#define NCCL_M2N_CONFIG_INITIALIZER { sizeof(ncclM2nConfig_t), NCCL_M2N_API_MAGIC, NCCL_M2N_CONFIG_UNDEF_INT }

ncclResult_t ncclM2nInit(ncclM2nConfig_t* config);
ncclResult_t ncclM2nFinalize(void);
/* Collective over comm. localShape of a side must be the same on all of its ranks; ranks that are on
 * neither side still call (they take part in nothing but must not be left out of the collective). */
ncclResult_t ncclReshardWithWindow(ncclComm_t comm, ncclWindow_t window, const ncclDistTensor_t* src, const ncclDistTensor_t* dst, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
