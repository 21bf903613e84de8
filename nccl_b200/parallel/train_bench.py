"""Training-step benchmarks over the library: ZeRO-3 / FSDP step of a Llama-shaped model and a
pipeline of ncclSend / ncclRecv activations.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m nccl_b200.parallel.train_bench --what fsdp --steps 5 --warmup 3
    ... --what pipeline --stages 4          # 4096 x 4096 bf16 activations between 4 stages
    ... --impl reference                    # the same engine over the library built from the reference sources

Each step's timed region includes the host-to-device copy of the step's token ids from pinned
memory and the device-to-host read of the loss. Times are CUDA-event durations, max over ranks.
One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF_LIB = os.path.join(ROOT, "baseline", "_ref", "build", "lib", "libnccl.so.2")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="fsdp", choices=("fsdp", "pipeline"))
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--stages", type=int, default=4)
    ap.add_argument("--micro", type=int, default=8)
    ap.add_argument("--tiny", action="store_true", help="tiny model (smoke runs)")
    a = ap.parse_args(argv)

    from nccl_b200 import Communicator, _lib, get_unique_id
    from nccl_b200.models.llama import LlamaConfig
    from nccl_b200.utils.perf import Dist
    d = Dist()
    torch.cuda.set_device(d.local_rank)
    if a.impl == "reference" and not os.path.exists(REF_LIB):
        if d.rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/build/lib/libnccl.so.2 is missing"}))
        return 0
    lib = _lib.load(REF_LIB) if a.impl == "reference" else _lib.load()
    uid = d.bcast_bytes(get_unique_id(lib) if d.rank == 0 else None)
    comm = Communicator(d.world, d.rank, uid, lib=lib)
    cfg = LlamaConfig.tiny(a.layers) if a.tiny else LlamaConfig(layers=a.layers)
    g = torch.Generator().manual_seed(1234 + d.rank)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    if a.what == "fsdp":
        from nccl_b200.parallel.fsdp import FSDPEngine
        eng = FSDPEngine(comm, cfg, device="cuda", seed=0, init_on_device=True)
        tok = torch.randint(0, cfg.vocab, (a.batch, a.seq), generator=g).pin_memory()
        tgt = torch.randint(0, cfg.vocab, (a.batch, a.seq), generator=g).pin_memory()
        loss = None
        for _ in range(a.warmup):
            loss = float(eng.step(tok, tgt))
        d.barrier()
        torch.cuda.synchronize()
        c0 = eng.collectives
        start.record()
        for _ in range(a.steps):
            loss = float(eng.step(tok, tgt))      # float(): device-to-host read of the loss, every step
        stop.record()
        torch.cuda.synchronize()
        d.barrier()
        ms = d.max(start.elapsed_time(stop)) / a.steps
        tokens = a.batch * a.seq * d.world
        out = {"metric": "fsdp_tokens_per_s", "value": tokens / (ms / 1e3), "unit": "tokens/s", "impl": a.impl, "n_gpus": d.world, "steps": a.steps,
               "warmup": a.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "dtype": "bf16", "data": "synthetic", "loss": loss,
               "collectives_per_step": (eng.collectives - c0) // a.steps, "h2d_bytes_per_step": 2 * tok.numel() * 8, "d2h_bytes_per_step": 4,
               "config": {"model": "llama3-8b-shaped" if not a.tiny and a.layers == 32 else "llama-%dL" % a.layers, "global_batch": a.batch * d.world,
                          "seq_len": a.seq, "parallelism": "zero3-dp%d" % d.world, "activation_checkpointing": True}}
        eng.close()
    else:
        from nccl_b200.parallel.pipeline import PipelineStage
        if d.world != a.stages:
            raise SystemExit("--stages must equal the number of ranks")
        st = PipelineStage(comm, cfg, device="cuda", seed=0)
        toks = [torch.randint(0, cfg.vocab, (a.batch, a.seq), generator=torch.Generator().manual_seed(i)) for i in range(a.micro)]
        for _ in range(a.warmup):
            st.forward_only(toks)
        d.barrier()
        torch.cuda.synchronize()
        s0 = st.sends
        start.record()
        for _ in range(a.steps):
            st.forward_only(toks)
        stop.record()
        torch.cuda.synchronize()
        d.barrier()
        ms = d.max(start.elapsed_time(stop)) / a.steps
        out = {"metric": "pipeline_tokens_per_s", "value": a.micro * a.batch * a.seq / (ms / 1e3), "unit": "tokens/s", "impl": a.impl, "n_gpus": d.world,
               "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
               "sends_per_step": (st.sends - s0) // max(a.steps, 1), "activation_bytes": a.batch * a.seq * cfg.hidden * 2,
               "config": {"model": "llama-%dL" % a.layers, "micro_batches": a.micro, "seq_len": a.seq, "parallelism": "pp%d" % d.world}}
    comm.destroy()
    if d.rank == 0:
        print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
