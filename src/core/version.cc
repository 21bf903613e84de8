// Build stamp: which source revision this library was built from (the build passes it in).
// Reference parity: src/misc/git_version.cc.
#ifndef B200_GIT_VERSION
#define B200_GIT_VERSION "unknown"
#endif
extern "C" __attribute__((visibility("default"))) const char* b200GitVersion() { return B200_GIT_VERSION; }
