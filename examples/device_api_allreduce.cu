// A user kernel on the device API: every CTA synchronises the ranks with a load/store barrier,
// sums its share of a registered window over all peers with plain peer loads, stores the result
// to every peer and synchronises again. (Pattern of the reference's examples/06_device_api.)
#include <atomic>

#include "common.h"
#include "nccl_device.h"

constexpr int kCtas = 16, kThreads = 256;

__global__ void __launch_bounds__(kThreads) sumKernel(ncclDevComm_t dc, ncclWindow_t win, size_t count, int* status) {
  ncclCoopCta cta;
  ncclLsaBarrierSession<ncclCoopCta> bar(cta, dc, ncclTeamLsa(dc), blockIdx.x);
  if (bar.sync(0, false, false) != ncclSuccess) {   // every rank's input is in place
    if (threadIdx.x == 0) atomicExch(status, 1);
    bar.finish();
    return;
  }
  const int n = dc.lsaSize;
  const size_t per = (count + n - 1) / n;
  const size_t lo = min(count, per * dc.lsaRank), hi = min(count, lo + per);
  for (size_t i = lo + (size_t)blockIdx.x * kThreads + threadIdx.x; i < hi; i += (size_t)gridDim.x * kThreads) {
    float acc = 0.0f;
    for (int p = 0; p < n; ++p) acc += ((const float*)ncclGetLsaPointer(win, 0, p))[i];
    for (int p = 0; p < n; ++p) ((float*)ncclGetLsaPointer(win, count * sizeof(float), p))[i] = acc;
  }
  if (bar.sync(0, true, false) != ncclSuccess && threadIdx.x == 0) atomicExch(status, 2);   // results are visible everywhere
  bar.finish();
}

int main() {
  const int n = exampleGpus();
  std::atomic<int> bad{0};
  runThreadPerGpu(n, [&](int rank, int nRanks, ncclComm_t comm) {
    const size_t count = 1 << 18;
    cudaStream_t s;
    CUDA_OK(cudaStreamCreate(&s));
    float* buf;   // [0, count): input, [count, 2 count): output
    NCCL_OK(ncclMemAlloc((void**)&buf, 2 * count * sizeof(float)));
    ncclWindow_t win;
    NCCL_OK(ncclCommWindowRegister(comm, buf, 2 * count * sizeof(float), &win, NCCL_WIN_COLL_SYMMETRIC));
    ncclWindow_t devWin;   // the handle kernels take: a device copy of the window description
    NCCL_OK(ncclWinGetDeviceHandle(win, &devWin));
    ncclDevCommRequirements_t reqs = NCCL_DEV_COMM_REQUIREMENTS_INITIALIZER;
    reqs.lsaBarrierCount = kCtas;
    ncclDevComm_t dc;
    NCCL_OK(ncclDevCommCreate(comm, &reqs, &dc));
    std::vector<float> h(count);
    for (size_t i = 0; i < count; ++i) h[i] = (float)(rank + 1) * (float)(i % 5);
    CUDA_OK(cudaMemcpyAsync(buf, h.data(), count * sizeof(float), cudaMemcpyHostToDevice, s));
    int* status;
    CUDA_OK(cudaMalloc(&status, sizeof(int)));
    CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int), s));
    sumKernel<<<kCtas, kThreads, 0, s>>>(dc, devWin, count, status);
    CUDA_OK(cudaGetLastError());
    // The handle from ncclCommWindowRegister is itself readable from kernels (pinned, mapped host memory);
    // the device copy above is only the faster of the two. Run once more with it.
    sumKernel<<<kCtas, kThreads, 0, s>>>(dc, win, count, status);
    CUDA_OK(cudaGetLastError());
    int st = -1;
    CUDA_OK(cudaMemcpyAsync(&st, status, sizeof(int), cudaMemcpyDeviceToHost, s));
    CUDA_OK(cudaMemcpyAsync(h.data(), buf + count, count * sizeof(float), cudaMemcpyDeviceToHost, s));
    CUDA_OK(cudaStreamSynchronize(s));
    if (st != 0) { fprintf(stderr, "rank %d: barrier status %d\n", rank, st); bad++; }
    const float tri = (float)(nRanks * (nRanks + 1) / 2);
    for (size_t i = 0; i < count; ++i)
      if (h[i] != tri * (float)(i % 5)) { bad++; break; }
    NCCL_OK(ncclDevCommDestroy(comm, &dc));
    NCCL_OK(ncclCommWindowDeregister(comm, win));
    NCCL_OK(ncclMemFree(buf));
    CUDA_OK(cudaFree(status));
    CUDA_OK(cudaStreamDestroy(s));
  });
  printf("device_api_allreduce: %d GPU(s): %s\n", n, bad ? "FAILED" : "ok");
  return bad ? 1 : 0;
}
