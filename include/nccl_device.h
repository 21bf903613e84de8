/*
 * Device API umbrella header: include from CUDA code that talks to other ranks itself.
 *   core.h         ncclDevComm, windows, teams, pointer getters, host-side creation
 *   ptr.h          ncclSymPtr<T>
 *   coop.h         cooperative groups (thread, tile, warp, warp span, CTA)
 *   lsa_barrier.h  barrier among the load/store team, with time-outs
 *   ll_a2a.h       low-latency all-to-all sessions (flagged 16-byte lines)
 *   multimem.h     multimem.ld_reduce / st / red wrappers
 *   reduce_copy.h  cooperative reduce / copy loops over windows
 *   gin.h          GPU-initiated put / signal surface
 * Reference parity: src/include/nccl_device.h and src/include/nccl_device/.
 */
#ifndef NCCL_DEVICE_H_
#define NCCL_DEVICE_H_
#include "nccl_device/core.h"
#include "nccl_device/ptr.h"
#include "nccl_device/coop.h"
#include "nccl_device/utility.h"
#include "nccl_device/lsa_barrier.h"
#include "nccl_device/barrier.h"
#include "nccl_device/ll_a2a.h"
#include "nccl_device/multimem.h"
#include "nccl_device/reduce_copy.h"
#include "nccl_device/gin.h"
#endif
