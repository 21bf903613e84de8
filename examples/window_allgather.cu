// Symmetric memory: buffers from ncclMemAlloc registered as windows, then an all-gather and a
// reduce-scatter that run without staging copies. (Pattern of the reference's
// examples/04_user_buffer_registration and examples/05_symmetric_memory.)
#include <atomic>

#include "common.h"

int main() {
  const int n = exampleGpus();
  std::atomic<int> bad{0};
  runThreadPerGpu(n, [&](int rank, int nRanks, ncclComm_t comm) {
    const size_t per = 1 << 20;   // floats per rank
    cudaStream_t s;
    CUDA_OK(cudaStreamCreate(&s));
    float *part, *all;
    NCCL_OK(ncclMemAlloc((void**)&part, per * sizeof(float)));
    NCCL_OK(ncclMemAlloc((void**)&all, per * nRanks * sizeof(float)));
    ncclWindow_t wPart, wAll;
    NCCL_OK(ncclCommWindowRegister(comm, part, per * sizeof(float), &wPart, NCCL_WIN_COLL_SYMMETRIC));
    NCCL_OK(ncclCommWindowRegister(comm, all, per * nRanks * sizeof(float), &wAll, NCCL_WIN_COLL_SYMMETRIC));
    std::vector<float> h(per * nRanks);
    for (size_t i = 0; i < per; ++i) h[i] = (float)(rank + 1);
    CUDA_OK(cudaMemcpy(part, h.data(), per * sizeof(float), cudaMemcpyHostToDevice));
    NCCL_OK(ncclAllGather(part, all, per, ncclFloat, comm, s));
    NCCL_OK(ncclReduceScatter(all, part, per, ncclFloat, ncclSum, comm, s));   // block `rank` of every rank's gathered copy
    CUDA_OK(cudaStreamSynchronize(s));
    CUDA_OK(cudaMemcpy(h.data(), all, per * nRanks * sizeof(float), cudaMemcpyDeviceToHost));
    for (int r = 0; r < nRanks; ++r)
      if (h[(size_t)r * per] != (float)(r + 1) || h[(size_t)r * per + per - 1] != (float)(r + 1)) bad++;
    CUDA_OK(cudaMemcpy(h.data(), part, per * sizeof(float), cudaMemcpyDeviceToHost));
    if (h[0] != (float)(nRanks * (rank + 1)) || h[per - 1] != (float)(nRanks * (rank + 1))) bad++;
    NCCL_OK(ncclCommWindowDeregister(comm, wPart));
    NCCL_OK(ncclCommWindowDeregister(comm, wAll));
    NCCL_OK(ncclMemFree(part));
    NCCL_OK(ncclMemFree(all));
    CUDA_OK(cudaStreamDestroy(s));
  });
  printf("window_allgather: %d GPU(s): %s\n", n, bad ? "FAILED" : "ok");
  return bad ? 1 : 0;
}
