// NVTX ranges around every public call, in the domain "NCCL". NVTX3 is header-only: without a
// profiling tool attached the calls are no-ops; with one (Nsight Systems) each API call shows up
// as a range named after the function, with message size and communicator in the text.
// Reference parity: src/include/nvtx.h (NVTX3_FUNC_WITH_PARAMS on each entry point),
// src/init_nvtx.cc (domain and payload registration).
#include <nvtx3/nvToolsExt.h>

#include "core.h"

namespace b200 {

B200_PARAM(NvtxDisable, "NVTX_DISABLE", 0, "1: emit no NVTX ranges");

static nvtxDomainHandle_t nvtxDomain() {
  static nvtxDomainHandle_t d = nvtxDomainCreateA("NCCL");
  return d;
}

void nvtxRangeBegin(const char* func, size_t bytes, uint64_t commHash, int rank) {
  if (paramNvtxDisable()) return;
  char msg[128];
  snprintf(msg, sizeof(msg), "%s %zu B comm %llx rank %d", func, bytes, (unsigned long long)commHash, rank);
  nvtxEventAttributes_t a = {};
  a.version = NVTX_VERSION;
  a.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
  a.messageType = NVTX_MESSAGE_TYPE_ASCII;
  a.message.ascii = msg;
  a.payloadType = NVTX_PAYLOAD_TYPE_UNSIGNED_INT64;
  a.payload.ullValue = bytes;
  nvtxDomainRangePushEx(nvtxDomain(), &a);
}

void nvtxRangeEnd() {
  if (paramNvtxDisable()) return;
  nvtxDomainRangePop(nvtxDomain());
}

}  // namespace b200
