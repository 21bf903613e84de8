// Reliability / availability / serviceability: a per-process background thread that tracks the
// communicators of the process, exchanges keep-alives with the other processes of the job and
// answers status queries from the ncclras client on localhost.
// Reference parity: src/ras/*.cc, src/include/ras.h, docs/userguide/source/troubleshooting/ras.rst.
#pragma once
#include "../comm/comm.h"

namespace b200 {
void rasCommAdd(ncclComm* comm);
void rasCommRemove(ncclComm* comm);
}  // namespace b200
