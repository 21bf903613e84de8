/* A loop of collective calls for the timing harness (nccl_b200/utils/perf.py): the interpreter's cost per call (several
 * microseconds) would otherwise be timed as if it were the library's. The entry points of the library under test come in as
 * addresses, so the same loop serves this library and any other with the NCCL API; nothing here knows either.
 *   kind 0  fn(send, recv, count, type, op, comm, stream)          all-reduce, reduce-scatter
 *   kind 1  fn(send, recv, count, type, comm, stream)              all-gather, all-to-all
 *   kind 2  fn(send, recv, count, type, root, comm, stream)        broadcast
 *   kind 3  fn(send, recv, count, type, op, root, comm, stream)    reduce
 *   kind 4  groupStart(); send(send, count, type, next, comm, stream); recv(recv, count, type, prev, comm, stream); groupEnd()
 * Returns the first result that is not 0 (ncclSuccess), else 0. */
#include <stddef.h>

typedef int (*fn0_t)(const void*, void*, size_t, int, int, void*, void*);
typedef int (*fn1_t)(const void*, void*, size_t, int, void*, void*);
typedef int (*fn2_t)(const void*, void*, size_t, int, int, void*, void*);
typedef int (*fn3_t)(const void*, void*, size_t, int, int, int, void*, void*);
typedef int (*group_t)(void);
typedef int (*p2p_t)(const void*, size_t, int, int, void*, void*);

__attribute__((visibility("default"))) int perfLoop(int kind, void* const* fns, const void* send, void* recv, size_t count, int type, int op, int root,
                                                    int next, int prev, void* comm, void* stream, int iters) {
  int r = 0;
  for (int i = 0; i < iters && r == 0; ++i) {
    switch (kind) {
      case 0: r = ((fn0_t)fns[0])(send, recv, count, type, op, comm, stream); break;
      case 1: r = ((fn1_t)fns[0])(send, recv, count, type, comm, stream); break;
      case 2: r = ((fn2_t)fns[0])(send, recv, count, type, root, comm, stream); break;
      case 3: r = ((fn3_t)fns[0])(send, recv, count, type, op, root, comm, stream); break;
      case 4:
        r = ((group_t)fns[0])();
        if (r == 0) r = ((p2p_t)fns[1])(send, count, type, next, comm, stream);
        if (r == 0) r = ((p2p_t)fns[2])(recv, count, type, prev, comm, stream);
        if (r == 0) r = ((group_t)fns[3])();
        break;
      default: return -1;
    }
  }
  return r;
}
