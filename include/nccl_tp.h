/*
 * Fused tensor-parallel linear layers on sm_100a: a bf16 GEMM (tcgen05 tensor cores, fp32
 * accumulation in tensor memory) fused with the collective next to it, so that NVLink traffic
 * overlaps the math tile by tile.
 *
 *   ncclTpGemm               C[M,N] = A[M,K] * W[N,K]^T                       (no communication)
 *   ncclTpGemmReduceScatter  out[M/n,N] = reduce_scatter_rows( A[M,Ks] * W[N,Ks]^T )   row-parallel layer
 *   ncclTpAllGatherGemm      C[M,N] = all_gather_rows(A)[M,K] * W[N,K]^T                column-parallel layer
 *
 * A and W are row-major bf16 with K contiguous (the layout of torch.nn.Linear weights). M must be
 * a multiple of 128 * nRanks, N of 256, K of 64. These entry points extend the reference API (it
 * has no compute kernels); its equivalent is ncclReduceScatter / ncclAllGather plus a separate GEMM.
 */
#ifndef NCCL_TP_H_
#define NCCL_TP_H_

#include "nccl.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ncclTpContext* ncclTp_t;

/* Collective over comm. maxRows x maxCols bounds the outputs of ncclTpGemmReduceScatter
 * (fp32 accumulation window of maxRows/nRanks x maxCols per rank). */
ncclResult_t ncclTpCreate(ncclComm_t comm, size_t maxRows, size_t maxCols, ncclTp_t* tp);
ncclResult_t ncclTpDestroy(ncclTp_t tp);

/* A window for the activations of ncclTpAllGatherGemm: rows x cols bf16, symmetric over comm.
 * Every rank writes its own rows [rank*rows/n, (rank+1)*rows/n) before the call. Collective. */
ncclResult_t ncclTpAllocGathered(ncclTp_t tp, size_t rows, size_t cols, void** ptr);
ncclResult_t ncclTpFreeGathered(ncclTp_t tp, void* ptr);

ncclResult_t ncclTpGemm(ncclTp_t tp, const void* A, const void* W, void* C, int M, int N, int K, cudaStream_t stream);
ncclResult_t ncclTpGemmReduceScatter(ncclTp_t tp, const void* A, const void* W, void* out, int M, int N, int K, cudaStream_t stream);
ncclResult_t ncclTpAllGatherGemm(ncclTp_t tp, void* gatheredA, const void* W, void* C, int M, int N, int K, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
