// One process per GPU without MPI: the parent creates the unique id and forks one child per GPU before anything touches
// CUDA; every child picks its device, joins the communicator with ncclCommInitRank and takes part in an all-reduce that it
// checks on the host. A job launcher (torchrun, srun, mpirun) plays the parent's role in a real job: it only has to hand the
// 128 bytes of the id to every process. (Pattern of the reference's examples/01_communicators/03_one_device_per_process_mpi.)
#include <sys/wait.h>
#include <unistd.h>

#include "common.h"

static int child(int rank, int n, const ncclUniqueId& id) {
  const size_t count = 1 << 18;
  CUDA_OK(cudaSetDevice(rank));
  ncclComm_t comm;
  NCCL_OK(ncclCommInitRank(&comm, n, id, rank));
  float* buf = nullptr;
  CUDA_OK(cudaMalloc(&buf, count * sizeof(float)));
  std::vector<float> host(count);
  for (size_t i = 0; i < count; ++i) host[i] = (float)(rank + 1) + (float)(i % 5);
  CUDA_OK(cudaMemcpy(buf, host.data(), count * sizeof(float), cudaMemcpyHostToDevice));
  cudaStream_t stream;
  CUDA_OK(cudaStreamCreate(&stream));
  NCCL_OK(ncclAllReduce(buf, buf, count, ncclFloat, ncclSum, comm, stream));
  CUDA_OK(cudaStreamSynchronize(stream));
  CUDA_OK(cudaMemcpy(host.data(), buf, count * sizeof(float), cudaMemcpyDeviceToHost));
  int bad = 0;
  for (size_t i = 0; i < count; ++i)
    if (host[i] != (float)(n * (n + 1) / 2) + (float)n * (float)(i % 5)) ++bad;
  int user = -1, nranks = -1;
  NCCL_OK(ncclCommUserRank(comm, &user));
  NCCL_OK(ncclCommCount(comm, &nranks));
  if (user != rank || nranks != n) ++bad;
  CUDA_OK(cudaStreamDestroy(stream));
  CUDA_OK(cudaFree(buf));
  NCCL_OK(ncclCommDestroy(comm));
  return bad ? 1 : 0;
}

int main() {
  // the device count comes from the environment or from a short-lived helper process: the parent itself must not
  // initialise CUDA before it forks
  int n = 0;
  {
    int fds[2];
    if (pipe(fds) != 0) return 2;
    pid_t p = fork();
    if (p == 0) {
      int c = exampleGpus();
      if (write(fds[1], &c, sizeof(c)) != (ssize_t)sizeof(c)) _exit(2);
      _exit(0);
    }
    close(fds[1]);
    if (read(fds[0], &n, sizeof(n)) != (ssize_t)sizeof(n)) n = 0;
    close(fds[0]);
    int st = 0;
    waitpid(p, &st, 0);
    if (n < 1) { fprintf(stderr, "no GPU visible\n"); return 2; }
  }
  ncclUniqueId id;
  NCCL_OK(ncclGetUniqueId(&id));   // host-side only: opens the listening socket of the bootstrap root
  std::vector<pid_t> kids;
  for (int r = 0; r < n; ++r) {
    pid_t p = fork();
    if (p < 0) { perror("fork"); return 2; }
    if (p == 0) _exit(child(r, n, id));
    kids.push_back(p);
  }
  int bad = 0;
  for (pid_t p : kids) {
    int st = 0;
    waitpid(p, &st, 0);
    if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) ++bad;
  }
  printf("one_device_per_process: %d process(es): %s\n", n, bad ? "FAILED" : "ok");
  return bad ? 1 : 0;
}
