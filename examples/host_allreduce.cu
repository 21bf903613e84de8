// All-reduce of data that lives in pinned host memory (gradients of a CPU optimiser, offloaded state):
// ncclAllReduceFromHost copies in, reduces and copies out chunk by chunk, so that the two PCIe directions
// and the collective overlap. Compared here with the three steps issued one after the other.
#include <atomic>
#include <chrono>

#include "common.h"
#include "nccl_host_staged.h"

int main() {
  const int n = exampleGpus();
  std::atomic<int> bad{0};
  std::vector<double> overlappedMs(n), serialMs(n);
  runThreadPerGpu(n, [&](int rank, int nRanks, ncclComm_t comm) {
    const size_t count = (size_t)64 << 20;   // 256 MiB of floats
    cudaStream_t s;
    CUDA_OK(cudaStreamCreate(&s));
    float *hin, *hout, *din, *dout;
    CUDA_OK(cudaMallocHost((void**)&hin, count * sizeof(float)));
    CUDA_OK(cudaMallocHost((void**)&hout, count * sizeof(float)));
    NCCL_OK(ncclMemAlloc((void**)&din, count * sizeof(float)));
    NCCL_OK(ncclMemAlloc((void**)&dout, count * sizeof(float)));
    ncclWindow_t wi, wo;
    NCCL_OK(ncclCommWindowRegister(comm, din, count * sizeof(float), &wi, NCCL_WIN_COLL_SYMMETRIC));
    NCCL_OK(ncclCommWindowRegister(comm, dout, count * sizeof(float), &wo, NCCL_WIN_COLL_SYMMETRIC));
    for (size_t i = 0; i < count; ++i) hin[i] = (float)(rank + 1) + (float)(i & 3);
    auto timeIt = [&](const std::function<void()>& step) {
      step();   // warm-up
      CUDA_OK(cudaStreamSynchronize(s));
      auto t0 = std::chrono::steady_clock::now();
      for (int it = 0; it < 3; ++it) step();
      CUDA_OK(cudaStreamSynchronize(s));
      return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / 3;
    };
    overlappedMs[rank] = timeIt([&] { NCCL_OK(ncclAllReduceFromHost(hin, hout, din, dout, count, ncclFloat, ncclSum, comm, s, 0)); });
    const float want = (float)(nRanks * (nRanks + 1) / 2);
    for (size_t i : {(size_t)0, count / 2 + 1, count - 1})
      if (hout[i] != want + (float)nRanks * (float)(i & 3)) bad++;
    serialMs[rank] = timeIt([&] {
      CUDA_OK(cudaMemcpyAsync(din, hin, count * sizeof(float), cudaMemcpyHostToDevice, s));
      NCCL_OK(ncclAllReduce(din, dout, count, ncclFloat, ncclSum, comm, s));
      CUDA_OK(cudaMemcpyAsync(hout, dout, count * sizeof(float), cudaMemcpyDeviceToHost, s));
    });
    NCCL_OK(ncclCommWindowDeregister(comm, wi));
    NCCL_OK(ncclCommWindowDeregister(comm, wo));
    NCCL_OK(ncclMemFree(din));
    NCCL_OK(ncclMemFree(dout));
    CUDA_OK(cudaFreeHost(hin));
    CUDA_OK(cudaFreeHost(hout));
    CUDA_OK(cudaStreamDestroy(s));
  });
  printf("host_allreduce: %d GPU(s), 256 MiB per rank: %.1f ms overlapped, %.1f ms one step after the other: %s\n", n, overlappedMs[0], serialMs[0],
         bad ? "FAILED" : "ok");
  return bad ? 1 : 0;
}
