// Host shared-memory links between processes of one host: one single-producer single-consumer
// byte ring per ordered pair of ranks, in a POSIX shared-memory segment created by the receiver.
// Used by the host data plane when every rank of the communicator lives on the same host
// (NCCL_B200_HOST_SHM=1), instead of TCP over loopback.
// Reference parity: src/transport/shm.cc (host FIFO between ranks without peer access),
// src/misc/shmutils.cc (segment create / attach / unlink).
#pragma once
#include <atomic>
#include <string>

#include "../core/core.h"

namespace b200 {

struct ShmHeader {
  alignas(64) std::atomic<uint64_t> tail;   // bytes produced so far
  alignas(64) std::atomic<uint64_t> head;   // bytes consumed so far
  uint64_t capacity;
  uint64_t magic;
};

struct ShmLink {
  std::string name;
  ShmHeader* hdr = nullptr;
  char* data = nullptr;
  size_t mapBytes = 0;
  bool owner = false;
};

ncclResult_t shmLinkCreate(const std::string& name, size_t capacity, ShmLink* link);   // receiver
ncclResult_t shmLinkOpen(const std::string& name, ShmLink* link);                      // sender
void shmLinkUnlink(ShmLink* link);    // removes the name; mappings stay valid until closed
void shmLinkClose(ShmLink* link);
// Non-blocking: move what fits / what is there, return the number of bytes moved.
size_t shmLinkSend(ShmLink* link, const char* p, size_t n);
size_t shmLinkRecv(ShmLink* link, char* p, size_t n);

}  // namespace b200
