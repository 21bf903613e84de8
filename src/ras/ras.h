// Reliability / availability / serviceability: a per-process background thread that tracks the
// communicators of the process, exchanges keep-alives with the other processes of the job and
// answers status queries from the ncclras client on localhost.
// Reference parity: src/ras/*.cc, src/include/ras.h, docs/userguide/source/troubleshooting/ras.rst.
#pragma once
#include "../comm/comm.h"
#include "../core/socket.h"

namespace b200 {
void rasCommAdd(ncclComm* comm);
void rasCommRemove(ncclComm* comm);
// Starts the RAS thread of the process if needed; returns the address other processes reach it at.
bool rasListenAddr(SockAddr* out);
void rasShutdown();
}  // namespace b200
