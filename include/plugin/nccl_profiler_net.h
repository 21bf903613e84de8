/*
 * Events that network backends hand to the profiler through the callback they get at init (ncclProfilerCallback_t):
 * the backend describes what it did in its own record, the core wraps it into an ncclProfileNetPlugin event under the
 * proxy operation it belongs to, and the profiler plugin tells the records apart by the plugin id
 * (backend type in the high bits, record version in the low 16).
 * Interface facts: src/include/plugin/nccl_profiler.h:99-106, src/include/plugin/profiler/net_ib_v1.h, net_socket_v1.h of the reference.
 */
#ifndef NCCL_PROFILER_NET_H_
#define NCCL_PROFILER_NET_H_
#include <stddef.h>
#include <stdint.h>

#define NCCL_PROFILER_NET_VER_BITS (16)
#define NCCL_PROFILER_NET_VER_MASK (~0U >> NCCL_PROFILER_NET_VER_BITS)
#define NCCL_PROFILER_NET_TYPE_MASK (~0U << NCCL_PROFILER_NET_VER_BITS)
enum {
  NCCL_PROFILER_NET_TYPE_IB = (1U << NCCL_PROFILER_NET_VER_BITS),
  NCCL_PROFILER_NET_TYPE_SOCK = (2U << NCCL_PROFILER_NET_VER_BITS)
};

#define NCCL_PROFILER_NET_IB_VER 1
enum { ncclProfileQp = (1 << 0) };
typedef struct {
  uint8_t type; /* ncclProfileQp */
  union {
    struct {
      int device;     /* network device */
      uint64_t wr_id; /* work request id */
      int opcode;     /* verbs opcode */
      int qpNum;      /* queue pair number */
      size_t length;  /* bytes of the work request */
    } qp;
  };
} ncclProfilerNetIbDescr_v1_t;

#define NCCL_PROFILER_NET_SOCKET_VER 1
enum { ncclProfileSocket = (1 << 0) };
typedef struct {
  uint8_t type; /* ncclProfileSocket */
  union {
    struct {
      int fd;
      int op; /* 0 send, 1 receive */
      size_t length;
    } sock;
  };
} ncclProfilerNetSockDescr_v1_t;

#endif
