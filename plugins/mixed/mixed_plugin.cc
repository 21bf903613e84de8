// Example of one library that carries several plugins: the UNIX-socket network backend and the CSV tuner of the other
// examples, compiled together. With only NCCL_NET_PLUGIN pointing at it, the core finds the tuner in the same library
// (a tuner that is not named by NCCL_TUNER_PLUGIN is looked for in the network plugin's library).
// Reference parity: plugins/mixed/example/plugin.c (net + tuner symbols in one shared object).
#include "../net/unix_net.cc"
#include "../tuner/csv_tuner.cc"
