/*
 * Cooperative reduce / copy loops over windows for fp32 and bf16:
 *   ncclLsaReduceSum        dst[i] = sum over the team of src_window[peer][i]   (peer loads)
 *   ncclMultimemReduceSum   the same through multimem.ld_reduce
 *   ncclLsaCopy             store a local buffer into every peer's window       (peer stores)
 *   ncclMultimemCopy        the same through multimem.st
 * Counts are in elements; pointers and counts must keep 16-byte alignment for the vector loops,
 * a scalar tail handles the rest (peer-load variants only).
 * Reference parity: src/include/nccl_device/reduce_copy.h, impl/reduce_copy__funcs.h.
 */
#ifndef NCCL_DEVICE_REDUCE_COPY_H_
#define NCCL_DEVICE_REDUCE_COPY_H_
#include "core.h"
#include "multimem.h"
#if defined(__CUDACC__)
namespace nccl_device {
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ void add(float (&a)[8], uint4 v) { a[0] += __uint_as_float(v.x); a[1] += __uint_as_float(v.y); a[2] += __uint_as_float(v.z); a[3] += __uint_as_float(v.w); }
  static __device__ uint4 pack(const float (&a)[8]) { return make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3])); }
  static __device__ uint4 mcLoad(const void* p) { return ncclMultimemLoadSumF32x4(p); }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ void add(float (&a)[8], uint4 v) {
    const __nv_bfloat162* p = (const __nv_bfloat162*)&v;
#pragma unroll
    for (int i = 0; i < 4; ++i) { a[2 * i] += __bfloat162float(p[i].x); a[2 * i + 1] += __bfloat162float(p[i].y); }
  }
  static __device__ uint4 pack(const float (&a)[8]) {
    uint4 v;
    __nv_bfloat162* p = (__nv_bfloat162*)&v;
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
    return v;
  }
  static __device__ uint4 mcLoad(const void* p) { return ncclMultimemLoadSumBf16x8(p); }
};
}  // namespace nccl_device

template <typename T, typename Coop>
__device__ void ncclLsaReduceSum(Coop coop, ncclWindow_t srcWin, size_t srcOffset, T* dst, size_t count, int lsaSize) {
  using V = nccl_device::Vec16<T>;
  const size_t packs = count / V::N;
  for (size_t i = coop.thread_rank(); i < packs; i += coop.size()) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < lsaSize; ++p) V::add(acc, *(const uint4*)((const char*)ncclGetLsaPointer(srcWin, srcOffset, p) + i * 16));
    *(uint4*)((char*)dst + i * 16) = V::pack(acc);
  }
  for (size_t e = packs * V::N + coop.thread_rank(); e < count; e += coop.size()) {
    float acc = 0;
    for (int p = 0; p < lsaSize; ++p) acc += (float)((const T*)ncclGetLsaPointer(srcWin, srcOffset, p))[e];
    dst[e] = (T)acc;
  }
}

template <typename T, typename Coop>
__device__ void ncclMultimemReduceSum(Coop coop, ncclWindow_t srcWin, size_t srcOffset, T* dst, size_t count) {
  using V = nccl_device::Vec16<T>;
  const char* mc = (const char*)ncclGetMultimemPointer(srcWin, srcOffset);
  for (size_t i = coop.thread_rank(); i < count / V::N; i += coop.size()) *(uint4*)((char*)dst + i * 16) = V::mcLoad(mc + i * 16);
}

template <typename T, typename Coop>
__device__ void ncclLsaCopy(Coop coop, const T* src, ncclWindow_t dstWin, size_t dstOffset, size_t count, int lsaSize) {
  const size_t bytes = count * sizeof(T), packs = bytes / 16;
  for (size_t i = coop.thread_rank(); i < packs; i += coop.size()) {
    uint4 v = *(const uint4*)((const char*)src + i * 16);
    for (int p = 0; p < lsaSize; ++p) *(uint4*)((char*)ncclGetLsaPointer(dstWin, dstOffset, p) + i * 16) = v;
  }
  for (size_t b = packs * 16 + coop.thread_rank(); b < bytes; b += coop.size())
    for (int p = 0; p < lsaSize; ++p) ((char*)ncclGetLsaPointer(dstWin, dstOffset, p))[b] = ((const char*)src)[b];
}

template <typename T, typename Coop>
__device__ void ncclMultimemCopy(Coop coop, const T* src, ncclWindow_t dstWin, size_t dstOffset, size_t count) {
  char* mc = (char*)ncclGetMultimemPointer(dstWin, dstOffset);
  for (size_t i = coop.thread_rank(); i < count * sizeof(T) / 16; i += coop.size()) ncclMultimemStore16(mc + i * 16, *(const uint4*)((const char*)src + i * 16));
}

/* Reduce through the switch and broadcast the result through the switch: a one-kernel all-reduce
 * of the slice [offset, offset + count) when every rank calls it on its own slice. */
template <typename T, typename Coop>
__device__ void ncclLsaReduceSumMultimemCopy(Coop coop, ncclWindow_t srcWin, size_t srcOffset, ncclWindow_t dstWin, size_t dstOffset, size_t count) {
  using V = nccl_device::Vec16<T>;
  const char* in = (const char*)ncclGetMultimemPointer(srcWin, srcOffset);
  char* out = (char*)ncclGetMultimemPointer(dstWin, dstOffset);
  for (size_t i = coop.thread_rank(); i < count / V::N; i += coop.size()) ncclMultimemStore16(out + i * 16, V::mcLoad(in + i * 16));
}
#endif
#endif
