/*
 * Symmetric pointers: (window, offset) pairs that resolve to the local, a peer's, or the multicast
 * address of the same object. Reference parity: src/include/nccl_device/ptr.h.
 */
#ifndef NCCL_DEVICE_PTR_H_
#define NCCL_DEVICE_PTR_H_
#include "core.h"
#if defined(__CUDACC__)
template <typename T>
struct ncclSymPtr {
  ncclWindow_t window;
  size_t offset;   /* bytes */
  __host__ __device__ ncclSymPtr() : window(nullptr), offset(0) {}
  __host__ __device__ ncclSymPtr(ncclWindow_t w, size_t off) : window(w), offset(off) {}
  __device__ T* localPtr() const { return (T*)ncclGetLocalPointer(window, offset); }
  __device__ T* lsaPtr(int peer) const { return (T*)ncclGetLsaPointer(window, offset, peer); }
  __device__ T* peerPtr(ncclTeam_t team, int peer) const { return (T*)ncclGetPeerPointer(window, offset, team, peer); }
  __device__ T* multimemPtr() const { return (T*)ncclGetMultimemPointer(window, offset); }
  __host__ __device__ ncclSymPtr<T> operator+(ptrdiff_t n) const { return ncclSymPtr<T>(window, offset + n * sizeof(T)); }
  __host__ __device__ ncclSymPtr<T>& operator+=(ptrdiff_t n) { offset += n * sizeof(T); return *this; }
  template <typename U> __host__ __device__ explicit operator ncclSymPtr<U>() const { return ncclSymPtr<U>(window, offset); }
};
#endif
#endif
