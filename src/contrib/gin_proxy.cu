// Host thread behind the proxy mode of the GPU-initiated put / signal surface: kernels queue descriptors in a ring
// in pinned host memory; this thread takes them in order and runs each one on a stream of its own: the copy on the
// copy engines, then the add on the remote signal word and on the local completion counter (a one-thread kernel:
// stream memory operations cannot add), then a 64-bit stream write of the operation's index into the "done" word that
// flush() polls. It is the structure of a network proxy (the kernel describes, the host posts) with NVLink as the
// wire: the destination is the peer's mapping inside this process. A network backend would replace the three stream
// operations by an RDMA write with immediate and keep ring, flow control and completion word as they are.
// The add kernels need one free SM: a caller kernel that fills the GPU with CTAs that all spin on a signal can delay
// them until its waits run out, which is the same rule as for any kernel that waits on work of another stream.
// Reference parity: src/gin/gin_host_proxy.cc:172-328 (descriptor queue, progress thread, completion counters).
#include <cuda_runtime.h>

#include <atomic>
#include <thread>

#include "../comm/comm.h"
#include "../core/cudawrap.h"
#include "gin_proxy.h"

namespace b200 {

__global__ void ginProxyAddKernel(unsigned long long* word, unsigned long long add) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(word), "l"(add) : "memory");
}

struct GinProxy {
  int dev = 0;
  unsigned size = 0;
  ncclGinProxyDesc* ring = nullptr;       // pinned, mapped
  ncclGinProxyDesc* ringDev = nullptr;
  unsigned long long* tailHost = nullptr;   // pinned, mapped
  unsigned long long* tailDev = nullptr;
  unsigned long long* words = nullptr;      // device: [0] head, [1] done
  cudaStream_t stream = nullptr;
  std::thread thread;
  std::atomic<bool> stop{false};
  std::atomic<int> error{0};
  std::atomic<unsigned long long> served{0};
};

static void proxyLoop(GinProxy* p) {
  if (cudaSetDevice(p->dev) != cudaSuccess) { p->error = (int)ncclUnhandledCudaError; return; }
  const CuApi* cu = cuApi();
  unsigned long long tail = 0;
  unsigned idle = 0;
  while (!p->stop.load(std::memory_order_acquire)) {
    volatile ncclGinProxyDesc* d = p->ring + (tail & (p->size - 1));
    if (d->seq != tail + 1) {
      if (++idle > 2000) std::this_thread::sleep_for(std::chrono::microseconds(20));
      else std::this_thread::yield();
      continue;
    }
    idle = 0;
    std::atomic_thread_fence(std::memory_order_acquire);
    ncclGinProxyDesc op;
    op.dst = d->dst; op.src = d->src; op.bytes = d->bytes; op.signal = d->signal; op.signalAdd = d->signalAdd; op.counter = d->counter;
    bool ok = true;
    if (op.bytes && op.dst && op.src) ok = cudaMemcpyAsync(op.dst, op.src, op.bytes, cudaMemcpyDeviceToDevice, p->stream) == cudaSuccess;
    if (ok && op.signal) { ginProxyAddKernel<<<1, 1, 0, p->stream>>>(op.signal, op.signalAdd); ok = cudaGetLastError() == cudaSuccess; }
    if (ok && op.counter) { ginProxyAddKernel<<<1, 1, 0, p->stream>>>(op.counter, 1ull); ok = cudaGetLastError() == cudaSuccess; }
    ++tail;
    if (ok && cu && cu->cuStreamWriteValue64) ok = cu->cuStreamWriteValue64((CUstream)p->stream, (CUdeviceptr)(p->words + 1), tail, CU_STREAM_WRITE_VALUE_DEFAULT) == CUDA_SUCCESS;
    else if (ok) { ginProxyAddKernel<<<1, 1, 0, p->stream>>>(p->words + 1, 1ull); ok = cudaGetLastError() == cudaSuccess; }
    if (!ok) { (void)cudaGetLastError(); p->error = (int)ncclUnhandledCudaError; }
    *(volatile unsigned long long*)p->tailHost = tail;   // the slot may be reused
    p->served.store(tail, std::memory_order_release);
  }
  cudaStreamSynchronize(p->stream);
}

ncclResult_t ginProxyCreate(int dev, int depth, GinProxy** out, ncclDevComm_t* dc) {
  unsigned size = 64;
  while (size < (unsigned)depth && size < 65536) size <<= 1;
  GinProxy* p = new GinProxy;
  p->dev = dev;
  p->size = size;
  void* d = nullptr;
  bool ok = cudaHostAlloc((void**)&p->ring, sizeof(ncclGinProxyDesc) * size, cudaHostAllocMapped) == cudaSuccess;
  if (ok) { memset(p->ring, 0, sizeof(ncclGinProxyDesc) * size); ok = cudaHostGetDevicePointer(&d, p->ring, 0) == cudaSuccess; p->ringDev = (ncclGinProxyDesc*)d; }
  ok = ok && cudaHostAlloc((void**)&p->tailHost, 64, cudaHostAllocMapped) == cudaSuccess;
  if (ok) { memset(p->tailHost, 0, 64); ok = cudaHostGetDevicePointer(&d, p->tailHost, 0) == cudaSuccess; p->tailDev = (unsigned long long*)d; }
  ok = ok && cudaMalloc((void**)&p->words, 64) == cudaSuccess && cudaMemset(p->words, 0, 64) == cudaSuccess;
  int lo = 0, hi = 0;
  ok = ok && cudaDeviceGetStreamPriorityRange(&lo, &hi) == cudaSuccess && cudaStreamCreateWithPriority(&p->stream, cudaStreamNonBlocking, hi) == cudaSuccess;
  // Everything the thread will launch later is launched once now: with lazy module loading the first launch of a
  // kernel may have to wait for running kernels to finish, and the kernels running then are the ones that wait for us.
  if (ok) {
    ginProxyAddKernel<<<1, 1, 0, p->stream>>>(p->words + 2, 1ull);
    ok = cudaGetLastError() == cudaSuccess && cudaMemcpyAsync(p->words + 4, p->words + 2, 8, cudaMemcpyDeviceToDevice, p->stream) == cudaSuccess;
    const CuApi* cu = cuApi();
    if (ok && cu && cu->cuStreamWriteValue64) ok = cu->cuStreamWriteValue64((CUstream)p->stream, (CUdeviceptr)(p->words + 3), 1, CU_STREAM_WRITE_VALUE_DEFAULT) == CUDA_SUCCESS;
  }
  ok = ok && cudaDeviceSynchronize() == cudaSuccess;
  if (!ok) {
    (void)cudaGetLastError();
    ginProxyDestroy(p);
    return ncclUnhandledCudaError;
  }
  p->thread = std::thread(proxyLoop, p);
  dc->ginProxyRing = p->ringDev;
  dc->ginProxyHead = p->words;
  dc->ginProxyTail = p->tailDev;
  dc->ginProxyDone = p->words + 1;
  dc->ginProxyMask = size - 1;
  *out = p;
  return ncclSuccess;
}

void ginProxyDestroy(GinProxy* p) {
  if (!p) return;
  p->stop.store(true, std::memory_order_release);
  if (p->thread.joinable()) p->thread.join();
  if (p->stream) cudaStreamDestroy(p->stream);
  if (p->words) cudaFree(p->words);
  if (p->tailHost) cudaFreeHost(p->tailHost);
  if (p->ring) cudaFreeHost(p->ring);
  (void)cudaGetLastError();
  delete p;
}

unsigned long long ginProxyServed(const GinProxy* p) { return p ? p->served.load(std::memory_order_acquire) : 0; }
int ginProxyError(const GinProxy* p) { return p ? p->error.load() : 0; }

}  // namespace b200
