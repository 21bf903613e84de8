// Every rank sends a block to its successor and receives one from its predecessor inside one
// group; a second group sends two blocks per peer to show that several operations per peer keep
// their posting order. (Pattern of the reference's examples/02_point_to_point/01_ring_pattern.)
#include <atomic>

#include "common.h"

int main() {
  const int n = exampleGpus();
  std::atomic<int> bad{0};
  runThreadPerGpu(n, [&](int rank, int nRanks, ncclComm_t comm) {
    const size_t count = 3 << 18;   // 3 MiB of floats / 4: several mailbox chunks
    const int next = (rank + 1) % nRanks, prev = (rank + nRanks - 1) % nRanks;
    cudaStream_t s;
    CUDA_OK(cudaStreamCreate(&s));
    float *send, *recv;
    CUDA_OK(cudaMalloc(&send, 2 * count * sizeof(float)));
    CUDA_OK(cudaMalloc(&recv, 2 * count * sizeof(float)));
    std::vector<float> h(2 * count);
    for (size_t i = 0; i < 2 * count; ++i) h[i] = (float)rank * 1000.0f + (float)(i % 997);
    CUDA_OK(cudaMemcpy(send, h.data(), 2 * count * sizeof(float), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemset(recv, 0, 2 * count * sizeof(float)));
    // one block each way
    NCCL_OK(ncclGroupStart());
    NCCL_OK(ncclSend(send, count, ncclFloat, next, comm, s));
    NCCL_OK(ncclRecv(recv, count, ncclFloat, prev, comm, s));
    NCCL_OK(ncclGroupEnd());
    // two blocks per peer in one group
    NCCL_OK(ncclGroupStart());
    NCCL_OK(ncclSend(send, count, ncclFloat, next, comm, s));
    NCCL_OK(ncclSend(send + count, count, ncclFloat, next, comm, s));
    NCCL_OK(ncclRecv(recv, count, ncclFloat, prev, comm, s));
    NCCL_OK(ncclRecv(recv + count, count, ncclFloat, prev, comm, s));
    NCCL_OK(ncclGroupEnd());
    CUDA_OK(cudaStreamSynchronize(s));
    CUDA_OK(cudaMemcpy(h.data(), recv, 2 * count * sizeof(float), cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < 2 * count; ++i)
      if (h[i] != (float)prev * 1000.0f + (float)(i % 997)) { bad++; break; }
    CUDA_OK(cudaFree(send));
    CUDA_OK(cudaFree(recv));
    CUDA_OK(cudaStreamDestroy(s));
  });
  printf("sendrecv_ring: %d GPU(s): %s\n", n, bad ? "FAILED" : "ok");
  return bad ? 1 : 0;
}
