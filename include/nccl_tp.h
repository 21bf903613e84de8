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

/* Collective over comm. maxRows x maxCols bounds the products of ncclTpGemmReduceScatter
 * (a symmetric bf16 staging window of maxRows x maxCols per rank). */
ncclResult_t ncclTpCreate(ncclComm_t comm, size_t maxRows, size_t maxCols, ncclTp_t* tp);
ncclResult_t ncclTpDestroy(ncclTp_t tp);

/* A window for the activations of ncclTpAllGatherGemm: rows x cols bf16, symmetric over comm.
 * Every rank writes its own rows [rank*rows/n, (rank+1)*rows/n) before the call. Collective. */
ncclResult_t ncclTpAllocGathered(ncclTp_t tp, size_t rows, size_t cols, void** ptr);
ncclResult_t ncclTpFreeGathered(ncclTp_t tp, void* ptr);

ncclResult_t ncclTpGemm(ncclTp_t tp, const void* A, const void* W, void* C, int M, int N, int K, cudaStream_t stream);
ncclResult_t ncclTpGemmReduceScatter(ncclTp_t tp, const void* A, const void* W, void* out, int M, int N, int K, cudaStream_t stream);
ncclResult_t ncclTpAllGatherGemm(ncclTp_t tp, void* gatheredA, const void* W, void* C, int M, int N, int K, cudaStream_t stream);

/* ---- block-scaled fp8 (e4m3) variants, fp32 accumulation, bf16 output --------------------------
 * Activations carry one fp32 scale per row and 128 columns, stored K-block-major: scaleA[K/128][M].
 * Weights carry one scale per 128 x 128 block: scaleW[K/128][N/128]. x ~= q * scale.
 * M multiple of 128 * nRanks, N of 256, K of 128. */
/* Quantises a row-major bf16 matrix [rows, K]: blockRows 1 (activations) or 128 (weights). */
ncclResult_t ncclTpQuantizeFp8(ncclTp_t tp, const void* x, void* q, float* scales, int rows, int K, int blockRows, cudaStream_t stream);
ncclResult_t ncclTpGemmFp8(ncclTp_t tp, const void* A, const float* scaleA, const void* W, const float* scaleW, void* C, int M, int N, int K,
                           cudaStream_t stream);
ncclResult_t ncclTpGemmReduceScatterFp8(ncclTp_t tp, const void* A, const float* scaleA, const void* W, const float* scaleW, void* out, int M, int N,
                                        int K, cudaStream_t stream);
/* Symmetric activation window for ncclTpAllGatherGemmFp8: rows x cols e4m3 followed by its scales
 * [cols/128][rows]; every rank fills its own rows and their scales before the call. Collective.
 * Free with ncclTpFreeGathered(tp, *q). */
ncclResult_t ncclTpAllocGatheredFp8(ncclTp_t tp, size_t rows, size_t cols, void** q, float** scales);
ncclResult_t ncclTpAllGatherGemmFp8(ncclTp_t tp, void* gatheredA, const void* W, const float* scaleW, void* C, int M, int N, int K, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
