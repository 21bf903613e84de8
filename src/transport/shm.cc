// See shm.h.
#include "shm.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace b200 {

static constexpr uint64_t kShmMagic = 0x53484d4c494e4b31ull;   // "SHMLINK1"

static ncclResult_t mapSegment(int fd, size_t bytes, ShmLink* l) {
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) { WARN("shm: mmap of %s failed: %s", l->name.c_str(), strerror(errno)); return ncclSystemError; }
  l->hdr = (ShmHeader*)p;
  l->data = (char*)p + 4096;
  l->mapBytes = bytes;
  return ncclSuccess;
}

ncclResult_t shmLinkCreate(const std::string& name, size_t capacity, ShmLink* l) {
  l->name = name;
  l->owner = true;
  shm_unlink(name.c_str());   // a stale segment of a crashed job
  int fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0) { WARN("shm: cannot create %s: %s", name.c_str(), strerror(errno)); return ncclSystemError; }
  const size_t bytes = 4096 + capacity;
  if (ftruncate(fd, (off_t)bytes) != 0) { WARN("shm: cannot size %s to %zu bytes: %s", name.c_str(), bytes, strerror(errno)); close(fd); shm_unlink(name.c_str()); return ncclSystemError; }
  NCCLCHECK(mapSegment(fd, bytes, l));
  new (&l->hdr->tail) std::atomic<uint64_t>(0);
  new (&l->hdr->head) std::atomic<uint64_t>(0);
  l->hdr->capacity = capacity;
  __atomic_store_n(&l->hdr->magic, kShmMagic, __ATOMIC_RELEASE);
  return ncclSuccess;
}

ncclResult_t shmLinkOpen(const std::string& name, ShmLink* l) {
  l->name = name;
  l->owner = false;
  int fd = shm_open(name.c_str(), O_RDWR, 0600);
  if (fd < 0) { WARN("shm: cannot open %s: %s", name.c_str(), strerror(errno)); return ncclSystemError; }
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size <= 4096) { WARN("shm: %s has no content", name.c_str()); close(fd); return ncclSystemError; }
  NCCLCHECK(mapSegment(fd, (size_t)st.st_size, l));
  if (__atomic_load_n(&l->hdr->magic, __ATOMIC_ACQUIRE) != kShmMagic) { WARN("shm: %s is not a link segment", name.c_str()); return ncclInternalError; }
  return ncclSuccess;
}

void shmLinkUnlink(ShmLink* l) {
  if (l->owner && !l->name.empty()) shm_unlink(l->name.c_str());
}

void shmLinkClose(ShmLink* l) {
  if (l->hdr) munmap((void*)l->hdr, l->mapBytes);
  l->hdr = nullptr;
  l->data = nullptr;
}

size_t shmLinkSend(ShmLink* l, const char* p, size_t n) {
  ShmHeader* h = l->hdr;
  const uint64_t tail = h->tail.load(std::memory_order_relaxed), head = h->head.load(std::memory_order_acquire);
  const size_t room = (size_t)(h->capacity - (tail - head));
  const size_t m = std::min(n, room);
  if (!m) return 0;
  const size_t at = (size_t)(tail % h->capacity), first = std::min(m, (size_t)h->capacity - at);
  memcpy(l->data + at, p, first);
  if (m > first) memcpy(l->data, p + first, m - first);
  h->tail.store(tail + m, std::memory_order_release);
  return m;
}

size_t shmLinkRecv(ShmLink* l, char* p, size_t n) {
  ShmHeader* h = l->hdr;
  const uint64_t head = h->head.load(std::memory_order_relaxed), tail = h->tail.load(std::memory_order_acquire);
  const size_t have = (size_t)(tail - head);
  const size_t m = std::min(n, have);
  if (!m) return 0;
  const size_t at = (size_t)(head % h->capacity), first = std::min(m, (size_t)h->capacity - at);
  memcpy(p, l->data + at, first);
  if (m > first) memcpy(p + first, l->data, m - first);
  h->head.store(head + m, std::memory_order_release);
  return m;
}

}  // namespace b200
