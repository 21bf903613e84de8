// ncclparam: lists every parameter the library understands, with its current value and source.
//   ncclparam            -> documented parameters
//   ncclparam --all      -> every parameter
//   ncclparam KEY [...]  -> value of the given keys
// Reference parity: src/param/ncclparam.cc.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "nccl.h"

int main(int argc, char** argv) {
  if (argc >= 2 && (!strcmp(argv[1], "-h") || !strcmp(argv[1], "--help"))) {
    printf("usage: %s [--all | KEY...]\n", argv[0]);
    return 0;
  }
  if (argc >= 2 && !strcmp(argv[1], "--all")) {
    setenv("NCCL_PARAM_DUMP_ALL", "1", 1);
    ncclParamDumpAll();
    return 0;
  }
  if (argc == 1) {
    ncclParamDumpAll();
    return 0;
  }
  int rc = 0;
  for (int i = 1; i < argc; ++i) {
    const char* value = nullptr;
    int len = 0;
    if (ncclParamGetParameter(argv[i], &value, &len) != ncclSuccess) {
      fprintf(stderr, "%s: unknown parameter\n", argv[i]);
      rc = 1;
      continue;
    }
    printf("%s=%.*s\n", argv[i], len, value);
  }
  return rc;
}
