// One thread drives every GPU: ncclCommInitAll, then a grouped ncclAllReduce over all
// communicators, checked on the host. (Pattern of the reference's examples/01_communicators and
// examples/03_collectives/01_allreduce.)
#include "common.h"

int main() {
  const int n = exampleGpus();
  const size_t count = 1 << 20;
  std::vector<ncclComm_t> comms(n);
  NCCL_OK(ncclCommInitAll(comms.data(), n, nullptr));
  std::vector<float*> buf(n);
  std::vector<cudaStream_t> streams(n);
  std::vector<float> host(count);
  for (int d = 0; d < n; ++d) {
    CUDA_OK(cudaSetDevice(d));
    CUDA_OK(cudaMalloc(&buf[d], count * sizeof(float)));
    CUDA_OK(cudaStreamCreate(&streams[d]));
    for (size_t i = 0; i < count; ++i) host[i] = (float)(d + 1) + (float)(i % 7);
    CUDA_OK(cudaMemcpy(buf[d], host.data(), count * sizeof(float), cudaMemcpyHostToDevice));
  }
  NCCL_OK(ncclGroupStart());
  for (int d = 0; d < n; ++d) NCCL_OK(ncclAllReduce(buf[d], buf[d], count, ncclFloat, ncclSum, comms[d], streams[d]));
  NCCL_OK(ncclGroupEnd());
  int bad = 0;
  for (int d = 0; d < n; ++d) {
    CUDA_OK(cudaSetDevice(d));
    CUDA_OK(cudaStreamSynchronize(streams[d]));
    CUDA_OK(cudaMemcpy(host.data(), buf[d], count * sizeof(float), cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < count; ++i) {
      const float want = (float)(n * (n + 1) / 2) + (float)n * (float)(i % 7);
      if (host[i] != want) { if (!bad) fprintf(stderr, "GPU %d element %zu: %f, expected %f\n", d, i, host[i], want); ++bad; }
    }
    ncclResult_t async;
    NCCL_OK(ncclCommGetAsyncError(comms[d], &async));
    if (async != ncclSuccess) ++bad;
  }
  for (int d = 0; d < n; ++d) {
    CUDA_OK(cudaSetDevice(d));
    CUDA_OK(cudaFree(buf[d]));
    CUDA_OK(cudaStreamDestroy(streams[d]));
    NCCL_OK(ncclCommDestroy(comms[d]));
  }
  printf("allreduce_all_devices: %d GPU(s), %zu floats: %s\n", n, count, bad ? "FAILED" : "ok");
  return bad ? 1 : 0;
}
