"""Parallelism strategies over the library, for torch tensors on GPUs or on CPU ranks:

ddp       GradientBuckets: data-parallel gradient all-reduce in buckets, overlapped with backward
fsdp      FSDPEngine: ZeRO-3 sharding with prefetched all-gathers, reduce-scatter and a fused AdamW
pipeline  PipelineStage: GPipe stages exchanging activations with grouped send / receive
context   ring_attention, ulysses_*: sequence / context parallel communication recipes
train_bench  command-line benchmarks of the above
"""
