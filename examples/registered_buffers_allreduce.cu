// User-buffer registration: plain cudaMalloc buffers are registered with ncclCommRegister once, then used by several
// all-reduces (in place, out of place, with a pre-multiplied sum) that find the registration and run without staging
// copies; the handle is given back before the buffers are freed. Registration is a collective call here: every rank
// registers its buffers in the same order. (Pattern of the reference's examples/04_user_buffer_registration.)
#include <atomic>

#include "common.h"

int main() {
  const int n = exampleGpus();
  std::atomic<int> bad{0};
  runThreadPerGpu(n, [&](int rank, int nRanks, ncclComm_t comm) {
    const size_t count = 1 << 20;
    cudaStream_t s;
    CUDA_OK(cudaStreamCreate(&s));
    float *a, *b;
    CUDA_OK(cudaMalloc(&a, count * sizeof(float)));
    CUDA_OK(cudaMalloc(&b, count * sizeof(float)));
    void *ha = nullptr, *hb = nullptr;
    NCCL_OK(ncclCommRegister(comm, a, count * sizeof(float), &ha));
    NCCL_OK(ncclCommRegister(comm, b, count * sizeof(float), &hb));
    std::vector<float> h(count);
    for (size_t i = 0; i < count; ++i) h[i] = (float)(rank + 1);
    CUDA_OK(cudaMemcpy(a, h.data(), count * sizeof(float), cudaMemcpyHostToDevice));
    const float total = (float)(nRanks * (nRanks + 1) / 2);
    // out of place, then in place on the result: b = sum, b = nRanks * sum
    NCCL_OK(ncclAllReduce(a, b, count, ncclFloat, ncclSum, comm, s));
    NCCL_OK(ncclAllReduce(b, b, count, ncclFloat, ncclSum, comm, s));
    // average through a pre-multiplied sum: every contribution is scaled by 1 / nRanks before it is added
    ncclRedOp_t avg;
    const float scale = 1.0f / (float)nRanks;
    NCCL_OK(ncclRedOpCreatePreMulSum(&avg, (void*)&scale, ncclFloat, ncclScalarHostImmediate, comm));
    NCCL_OK(ncclAllReduce(a, a, count, ncclFloat, avg, comm, s));
    CUDA_OK(cudaStreamSynchronize(s));
    NCCL_OK(ncclRedOpDestroy(avg, comm));
    CUDA_OK(cudaMemcpy(h.data(), b, count * sizeof(float), cudaMemcpyDeviceToHost));
    if (h[0] != total * (float)nRanks || h[count - 1] != total * (float)nRanks) bad++;
    CUDA_OK(cudaMemcpy(h.data(), a, count * sizeof(float), cudaMemcpyDeviceToHost));
    const float mean = total / (float)nRanks;
    if (h[0] < mean - 1e-3f || h[0] > mean + 1e-3f || h[count / 2] < mean - 1e-3f || h[count / 2] > mean + 1e-3f) bad++;
    ncclResult_t async;
    NCCL_OK(ncclCommGetAsyncError(comm, &async));
    if (async != ncclSuccess) bad++;
    NCCL_OK(ncclCommDeregister(comm, ha));
    NCCL_OK(ncclCommDeregister(comm, hb));
    CUDA_OK(cudaFree(a));
    CUDA_OK(cudaFree(b));
    CUDA_OK(cudaStreamDestroy(s));
  });
  printf("registered_buffers_allreduce: %d GPU(s): %s\n", n, bad ? "FAILED" : "ok");
  return bad ? 1 : 0;
}
