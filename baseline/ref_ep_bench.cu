// Times the reference library's own expert-parallel extension (contrib/nccl_ep, low-latency mode, expert-major
// layout) on the workload this repository's ep_bench uses, so that the two can be compared on one machine.
// It is a plain client of the reference's public API: built against the reference's headers and linked with the
// libraries built from the reference sources (baseline/build_ref_ep.sh); nothing of this repository's library
// is on its path. One process per GPU, started by torchrun (RANK / WORLD_SIZE / LOCAL_RANK); the unique id
// travels through a file because the image has no MPI (the reference's own ep_bench needs it).
//   ref_ep_bench <id-file> [tokens hidden experts topk iters warmup fp8]
#include <cuda_runtime.h>
#include <nccl.h>
#include <nccl_ep.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>
#include <random>
#include <string>
#include <vector>

#define CK(cmd) do { cudaError_t e_ = (cmd); if (e_ != cudaSuccess) { printf("{\"impl\": \"reference\", \"unavailable\": \"CUDA error %s at line %d\"}\n", cudaGetErrorString(e_), __LINE__); return 0; } } while (0)
#define NK(cmd) do { ncclResult_t r_ = (cmd); if (r_ != ncclSuccess) { if (rank == 0) printf("{\"impl\": \"reference\", \"unavailable\": \"%s returned %d (%s)\"}\n", #cmd, (int)r_, ncclGetErrorString(r_)); return 0; } } while (0)

static cudaError_t devAlloc(void** p, size_t n, void*) { return cudaMalloc(p, n); }
static cudaError_t devFree(void* p, void*) { return cudaFree(p); }
static size_t esize(ncclDataType_t t) { return t == ncclInt64 ? 8 : t == ncclFloat32 || t == ncclInt32 ? 4 : t == ncclBfloat16 ? 2 : 1; }

static ncclResult_t tensor(ncclEpTensor_t** out, ncclDataType_t dt, std::vector<size_t> dims) {
  size_t total = esize(dt);
  for (size_t d : dims) total *= d;
  void* data = nullptr;
  if (cudaMalloc(&data, total) != cudaSuccess) return ncclSystemError;
  cudaMemset(data, 0, total);
  ncclResult_t r = ncclEpTensorAlloc(out, (unsigned)dims.size(), dt, dims.data(), nullptr);
  if (r == ncclSuccess) (*out)->data = data;
  return r;
}

int main(int argc, char** argv) {
  const int rank = atoi(getenv("RANK") ? getenv("RANK") : "0"), n = atoi(getenv("WORLD_SIZE") ? getenv("WORLD_SIZE") : "1");
  const int local = atoi(getenv("LOCAL_RANK") ? getenv("LOCAL_RANK") : "0");
  if (argc < 2) { printf("usage: ref_ep_bench <id-file> [tokens hidden experts topk iters warmup fp8]\n"); return 2; }
  const std::string idFile = argv[1];
  const int T = argc > 2 ? atoi(argv[2]) : 4096, H = argc > 3 ? atoi(argv[3]) : 7168, E = argc > 4 ? atoi(argv[4]) : 256;
  const int K = argc > 5 ? atoi(argv[5]) : 8, iters = argc > 6 ? atoi(argv[6]) : 10, warm = argc > 7 ? atoi(argv[7]) : 3;
  const bool fp8 = argc > 8 ? atoi(argv[8]) != 0 : false;
  const int El = E / n;

  ncclUniqueId id;
  if (rank == 0) {
    if (ncclGetUniqueId(&id) != ncclSuccess) return 1;
    FILE* f = fopen((idFile + ".tmp").c_str(), "wb");
    if (!f) return 1;
    fwrite(&id, sizeof(id), 1, f);
    fclose(f);
    rename((idFile + ".tmp").c_str(), idFile.c_str());
  } else {
    bool got = false;
    for (int i = 0; i < 600 && !got; ++i) {
      FILE* f = fopen(idFile.c_str(), "rb");
      if (f) { got = fread(&id, sizeof(id), 1, f) == 1; fclose(f); }
      if (!got) usleep(100000);
    }
    if (!got) return 1;
  }
  CK(cudaSetDevice(local));
  cudaStream_t s;
  CK(cudaStreamCreate(&s));
  ncclComm_t comm;
  NK(ncclCommInitRank(&comm, n, id, rank));

  ncclEpGroupConfig_t cfg = NCCL_EP_GROUP_CONFIG_INIT;
  cfg.algorithm = NCCL_EP_ALGO_LOW_LATENCY;
  cfg.num_experts = E;
  cfg.max_dispatch_tokens_per_rank = T;
  cfg.max_token_bytes = H * 2;
  cfg.rdma_buffer_size = NCCL_EP_AUTO;
  cfg.num_qp_per_rank = NCCL_EP_AUTO;
  cfg.num_channels = NCCL_EP_AUTO;
  cfg.alloc.alloc_fn = devAlloc;
  cfg.alloc.free_fn = devFree;
  cfg.alloc.context = nullptr;
  ncclEpGroup_t group;
  NK(ncclEpCreateGroup(&group, comm, &cfg));

  // routing: top-k of N(0,1) logits per token (the softmax keeps their order), seed 100 + rank
  std::mt19937 gen(100 + rank);
  std::normal_distribution<float> normal(0.f, 1.f);
  std::vector<int64_t> idx((size_t)T * K);
  std::vector<float> wts((size_t)T * K, 1.0f / K), logits(E);
  std::vector<int> order(E);
  for (int t = 0; t < T; ++t) {
    for (int e = 0; e < E; ++e) { logits[e] = normal(gen); order[e] = e; }
    std::partial_sort(order.begin(), order.begin() + K, order.end(), [&](int a, int b) { return logits[a] > logits[b]; });
    for (int k = 0; k < K; ++k) idx[(size_t)t * K + k] = order[k];
  }
  ncclEpTensor_t *tIdx, *tW, *tX, *tRecv, *tScales = nullptr, *tCnt, *tY, *tOut;
  NK(tensor(&tIdx, ncclInt64, {(size_t)T, (size_t)K}));
  NK(tensor(&tW, ncclFloat32, {(size_t)T, (size_t)K}));
  NK(tensor(&tX, ncclBfloat16, {(size_t)T, (size_t)H}));
  NK(tensor(&tRecv, fp8 ? ncclFloat8e4m3 : ncclBfloat16, {(size_t)El, (size_t)T * n, (size_t)H}));
  if (fp8) NK(tensor(&tScales, ncclFloat32, {(size_t)El, (size_t)T * n, (size_t)H / 128}));
  NK(tensor(&tCnt, ncclInt32, {(size_t)El}));
  NK(tensor(&tY, ncclBfloat16, {(size_t)El, (size_t)T * n, (size_t)H}));
  NK(tensor(&tOut, ncclBfloat16, {(size_t)T, (size_t)H}));
  CK(cudaMemcpy(tIdx->data, idx.data(), idx.size() * 8, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(tW->data, wts.data(), wts.size() * 4, cudaMemcpyHostToDevice));
  {
    std::vector<uint16_t> x((size_t)T * H);
    for (auto& v : x) { float f = normal(gen); uint32_t b; memcpy(&b, &f, 4); v = (uint16_t)(b >> 16); }
    CK(cudaMemcpy(tX->data, x.data(), x.size() * 2, cudaMemcpyHostToDevice));
  }

  ncclEpHandle_t handle;
  NK(ncclEpCreateHandle(&handle, group, NCCL_EP_LAYOUT_EXPERT_MAJOR, tIdx, nullptr, nullptr, s));
  CK(cudaStreamSynchronize(s));

  ncclEpDispatchInputs_t din = NCCL_EP_DISPATCH_INPUTS_INIT;
  ncclEpDispatchOutputs_t dout = NCCL_EP_DISPATCH_OUTPUTS_INIT;
  ncclEpLayoutInfo_t li = NCCL_EP_LAYOUT_INFO_INIT;
  ncclEpDispatchConfig_t dcfg = NCCL_EP_DISPATCH_CONFIG_INIT;
  din.tokens = tX;
  dout.tokens = tRecv;
  dout.scales = tScales;
  li.expert_counters = tCnt;
  ncclEpCombineInputs_t cin = NCCL_EP_COMBINE_INPUTS_INIT;
  ncclEpCombineOutputs_t cout = NCCL_EP_COMBINE_OUTPUTS_INIT;
  ncclEpCombineConfig_t ccfg = NCCL_EP_COMBINE_CONFIG_INIT;
  cin.tokens = tY;
  cout.tokens = tOut;
  cout.topk_weights = tW;

  float* dMax;
  CK(cudaMalloc(&dMax, 4));
  auto maxOverRanks = [&](float v, float* out) -> int {
    if (cudaMemcpy(dMax, &v, 4, cudaMemcpyHostToDevice) != cudaSuccess) return 1;
    if (ncclAllReduce(dMax, dMax, 1, ncclFloat32, ncclMax, comm, s) != ncclSuccess) return 1;
    if (cudaStreamSynchronize(s) != cudaSuccess) return 1;
    return cudaMemcpy(out, dMax, 4, cudaMemcpyDeviceToHost) != cudaSuccess;
  };
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  float ms[3] = {0, 0, 0};
  for (int what = 0; what < 3; ++what) {   // 0 dispatch, 1 combine, 2 both
    for (int phase = 0; phase < 2; ++phase) {
      const int reps = phase == 0 ? warm : iters;
      if (phase == 1) {
        CK(cudaStreamSynchronize(s));
        float dummy;
        if (maxOverRanks(0.f, &dummy)) return 1;   // all ranks start the timed loop together
        CK(cudaEventRecord(e0, s));
      }
      for (int i = 0; i < reps; ++i) {
        if (what != 1) { NK(ncclEpDispatch(handle, &din, &dout, &li, &dcfg, s)); NK(ncclEpComplete(handle, nullptr, s)); }
        if (what != 0) { NK(ncclEpCombine(handle, &cin, &cout, &ccfg, s)); NK(ncclEpComplete(handle, nullptr, s)); }
      }
      if (phase == 1) {
        CK(cudaEventRecord(e1, s));
        CK(cudaStreamSynchronize(s));
        float t;
        CK(cudaEventElapsedTime(&t, e0, e1));
        if (maxOverRanks(t / iters, &ms[what])) return 1;
      }
    }
  }
  std::vector<int> cnt(El);
  CK(cudaMemcpy(cnt.data(), tCnt->data, El * 4, cudaMemcpyDeviceToHost));
  long recv = 0;
  for (int c : cnt) recv += c;
  float recvMax;
  if (maxOverRanks((float)recv, &recvMax)) return 1;
  if (rank == 0)
    printf("{\"metric\": \"ep_dispatch_combine\", \"impl\": \"reference nccl_ep (low latency, expert major)\", \"n_gpus\": %d, \"tokens_per_rank\": %d, \"hidden\": %d, "
           "\"experts\": %d, \"topk\": %d, \"dispatch_dtype\": \"%s\", \"dispatch_us\": %.1f, \"combine_us\": %.1f, \"dispatch_plus_combine_us\": %.1f, \"recv_tokens_max\": %ld}\n",
           n, T, H, E, K, fp8 ? "fp8 e4m3 + scales" : "bf16", ms[0] * 1e3, ms[1] * 1e3, ms[2] * 1e3, (long)recvMax);
  ncclEpHandleDestroy(handle);
  ncclEpGroupDestroy(group);
  ncclCommDestroy(comm);
  return 0;
}
