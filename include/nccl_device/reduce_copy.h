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
#include "ptr.h"
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

/* ---- the reference's lambda and team forms (src/include/nccl_device/reduce_copy.h). A source lambda maps
 * i in [0, nSrc) to the i-th source pointer, a destination lambda j in [0, nDst) to the j-th destination; team forms
 * visit the window of every member of the team. Sums accumulate in fp32 in source order. float and bf16 use 16-byte
 * accesses when every pointer allows it; other types (and unaligned buffers) take the element loop. */
namespace nccl_device {
template <typename T> struct HasVec16 { static constexpr bool value = false; };
template <> struct HasVec16<float> { static constexpr bool value = true; };
template <> struct HasVec16<__nv_bfloat16> { static constexpr bool value = true; };

template <typename T, typename Coop, typename SrcLambda, typename DstLambda>
__device__ void reduceSumCopy(Coop coop, SrcLambda src, int nSrc, DstLambda dst, int nDst, size_t count) {
  size_t done = 0;
  if constexpr (HasVec16<T>::value) {
    using V = Vec16<T>;
    uintptr_t bits = 0;
    for (int i = 0; i < nSrc; ++i) bits |= (uintptr_t)src(i);
    for (int j = 0; j < nDst; ++j) bits |= (uintptr_t)dst(j);
    if ((bits & 15) == 0) {
      const size_t packs = count / V::N;
      for (size_t k = coop.thread_rank(); k < packs; k += coop.size()) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int i = 0; i < nSrc; ++i) V::add(acc, *(const uint4*)((const char*)src(i) + k * 16));
        const uint4 r = V::pack(acc);
        for (int j = 0; j < nDst; ++j) *(uint4*)((char*)dst(j) + k * 16) = r;
      }
      done = packs * V::N;
    }
  }
  for (size_t e = done + coop.thread_rank(); e < count; e += coop.size()) {
    float acc = 0;
    for (int i = 0; i < nSrc; ++i) acc += (float)((const T*)src(i))[e];
    for (int j = 0; j < nDst; ++j) ((T*)dst(j))[e] = (T)acc;
  }
}
}  // namespace nccl_device

template <typename T, typename Coop, typename SrcLambda, typename DstLambda, typename IntCount>
__device__ void ncclLsaReduceSumLsaCopy(Coop coop, SrcLambda src, int nSrc, DstLambda dst, int nDst, IntCount count) {
  nccl_device::reduceSumCopy<T>(coop, src, nSrc, dst, nDst, (size_t)count);
}
template <typename T, typename Coop, typename SrcLambda, typename IntCount>
__device__ void ncclLsaReduceSum(Coop coop, SrcLambda src, int nSrc, T* dst, IntCount count) {
  nccl_device::reduceSumCopy<T>(coop, src, nSrc, [=](int) { return dst; }, 1, (size_t)count);
}
template <typename T, typename Coop, typename SrcLambda, typename IntCount>
__device__ void ncclLocalReduceSum(Coop coop, SrcLambda src, int nSrc, T* dst, IntCount count) {
  nccl_device::reduceSumCopy<T>(coop, src, nSrc, [=](int) { return dst; }, 1, (size_t)count);
}
template <typename T, typename Coop, typename DstLambda, typename IntCount>
__device__ void ncclLsaCopy(Coop coop, T* src, DstLambda dst, int nDst, IntCount count) {
  nccl_device::reduceSumCopy<T>(coop, [=](int) { return src; }, 1, dst, nDst, (size_t)count);
}
template <typename T, typename Coop, typename DstLambda, typename IntCount>
__device__ void ncclLocalCopy(Coop coop, T* src, DstLambda dst, int nDst, IntCount count) {
  nccl_device::reduceSumCopy<T>(coop, [=](int) { return src; }, 1, dst, nDst, (size_t)count);
}
/* team forms: every member's window */
template <typename T, typename Coop, typename IntCount>
__device__ void ncclLsaReduceSum(Coop coop, ncclWindow_t win, size_t offset, T* dst, IntCount count, ncclTeam_t team) {
  nccl_device::reduceSumCopy<T>(coop, [=](int i) { return (T*)ncclGetPeerPointer(win, offset, team, i); }, team.nRanks, [=](int) { return dst; }, 1, (size_t)count);
}
template <typename T, typename Coop, typename IntCount>
__device__ void ncclLsaReduceSum(Coop coop, ncclWindow_t win, size_t offset, T* dst, IntCount count, const ncclDevComm_t& comm) {
  ncclLsaReduceSum<T>(coop, win, offset, dst, count, ncclTeamLsa(comm));
}
template <typename T, typename Coop, typename IntCount>
__device__ void ncclLsaReduceSum(Coop coop, ncclSymPtr<T> src, T* dst, IntCount count, ncclTeam_t team) { ncclLsaReduceSum<T>(coop, src.window, src.offset, dst, count, team); }
template <typename T, typename Coop, typename IntCount>
__device__ void ncclLsaCopy(Coop coop, T* src, ncclWindow_t win, size_t offset, IntCount count, ncclTeam_t team) {
  nccl_device::reduceSumCopy<T>(coop, [=](int) { return src; }, 1, [=](int j) { return (T*)ncclGetPeerPointer(win, offset, team, j); }, team.nRanks, (size_t)count);
}
template <typename T, typename Coop, typename IntCount>
__device__ void ncclLsaCopy(Coop coop, T* src, ncclWindow_t win, size_t offset, IntCount count, const ncclDevComm_t& comm) {
  ncclLsaCopy<T>(coop, src, win, offset, count, ncclTeamLsa(comm));
}
template <typename T, typename Coop, typename IntCount>
__device__ void ncclLsaCopy(Coop coop, T* src, ncclSymPtr<T> dst, IntCount count, ncclTeam_t team) { ncclLsaCopy<T>(coop, src, dst.window, dst.offset, count, team); }
template <typename T, typename Coop, typename IntCount>
__device__ void ncclLsaReduceSumCopy(Coop coop, ncclWindow_t srcWin, size_t srcOffset, ncclWindow_t dstWin, size_t dstOffset, IntCount count, ncclTeam_t team) {
  nccl_device::reduceSumCopy<T>(coop, [=](int i) { return (T*)ncclGetPeerPointer(srcWin, srcOffset, team, i); }, team.nRanks,
                                [=](int j) { return (T*)ncclGetPeerPointer(dstWin, dstOffset, team, j); }, team.nRanks, (size_t)count);
}
template <typename T, typename Coop, typename IntCount>
__device__ void ncclLsaReduceSumCopy(Coop coop, ncclWindow_t srcWin, size_t srcOffset, ncclWindow_t dstWin, size_t dstOffset, IntCount count, const ncclDevComm_t& comm) {
  ncclLsaReduceSumCopy<T>(coop, srcWin, srcOffset, dstWin, dstOffset, count, ncclTeamLsa(comm));
}
template <typename T, typename Coop, typename IntCount>
__device__ void ncclLsaReduceSumCopy(Coop coop, ncclSymPtr<T> src, ncclSymPtr<T> dst, IntCount count, ncclTeam_t team) {
  ncclLsaReduceSumCopy<T>(coop, src.window, src.offset, dst.window, dst.offset, count, team);
}
/* multicast forms on raw multicast pointers (count a multiple of the 16-byte vector) */
template <typename T, typename Coop, typename IntCount>
__device__ void ncclMultimemReduceSum(Coop coop, T* mcSrc, T* dst, IntCount count) {
  using V = nccl_device::Vec16<T>;
  for (size_t k = coop.thread_rank(); k < (size_t)count / V::N; k += coop.size()) *(uint4*)((char*)dst + k * 16) = V::mcLoad((const char*)mcSrc + k * 16);
}
template <typename T, typename Coop, typename IntCount>
__device__ void ncclMultimemCopy(Coop coop, T* src, T* mcDst, IntCount count) {
  for (size_t k = coop.thread_rank(); k < (size_t)count * sizeof(T) / 16; k += coop.size()) ncclMultimemStore16((char*)mcDst + k * 16, *(const uint4*)((const char*)src + k * 16));
}
template <typename T, typename Coop, typename IntCount>
__device__ void ncclMultimemReduceSumMultimemCopy(Coop coop, T* mcSrc, T* mcDst, IntCount count) {
  using V = nccl_device::Vec16<T>;
  for (size_t k = coop.thread_rank(); k < (size_t)count / V::N; k += coop.size()) ncclMultimemStore16((char*)mcDst + k * 16, V::mcLoad((const char*)mcSrc + k * 16));
}
#endif
#endif
