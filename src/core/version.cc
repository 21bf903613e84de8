// Build stamp: which source revision this library was built from (the build passes it in).
// Reference parity: src/misc/git_version.cc.
#include <cuda_runtime_api.h>

#ifndef B200_GIT_VERSION
#define B200_GIT_VERSION "unknown"
#endif
extern "C" __attribute__((visibility("default"))) const char* b200GitVersion() { return B200_GIT_VERSION; }
// CUDA toolkit the library was compiled with (CUDART_VERSION: 1000 * major + 10 * minor).
extern "C" __attribute__((visibility("default"))) int b200CudaBuildVersion() { return CUDART_VERSION; }
