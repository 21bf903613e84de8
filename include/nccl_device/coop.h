/*
 * Cooperative groups of the device API: the set of threads that executes a collective call
 * together (one thread, a tile of a warp, a warp, several warps, the whole CTA).
 * Reference parity: src/include/nccl_device/coop.h.
 */
#ifndef NCCL_DEVICE_COOP_H_
#define NCCL_DEVICE_COOP_H_
#if defined(__CUDACC__)
struct ncclCoopThread {
  __device__ int thread_rank() const { return 0; }
  __device__ int size() const { return 1; }
  __device__ void sync() const {}
};
template <int N>
struct ncclCoopTile {   /* N consecutive lanes of a warp, N a power of two */
  __device__ int thread_rank() const { return (threadIdx.x % 32) % N; }
  __device__ int size() const { return N; }
  __device__ void sync() const {
    unsigned lane = threadIdx.x % 32, base = lane / N * N;
    unsigned mask = N == 32 ? 0xffffffffu : (((1u << N) - 1) << base);
    __syncwarp(mask);
  }
};
typedef ncclCoopTile<32> ncclCoopWarp;
struct ncclCoopWarpSpan {   /* warps [warp0, warp0 + nWarps) of the CTA, synchronised with a named barrier */
  int warp0, nWarps, barrierId;
  __device__ ncclCoopWarpSpan(int w0, int n, int id) : warp0(w0), nWarps(n), barrierId(id) {}
  __device__ int thread_rank() const { return threadIdx.x - 32 * warp0; }
  __device__ int size() const { return 32 * nWarps; }
  __device__ void sync() const { asm volatile("barrier.sync %0, %1;" ::"r"(barrierId + 1), "r"(32 * nWarps) : "memory"); }
};
struct ncclCoopCta {
  __device__ int thread_rank() const { return threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z); }
  __device__ int size() const { return blockDim.x * blockDim.y * blockDim.z; }
  __device__ void sync() const { __syncthreads(); }
};
#endif
#endif
