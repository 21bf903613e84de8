"""ZeRO-3 / FSDP training engine over the library's all-gather and reduce-scatter.

Every unit of the model (embedding, each decoder layer, output head) is one flat bf16 buffer cut
into equal shards, one per rank. A training step:

  forward    for unit u: all-gather(u+1) runs on the communication stream while unit u computes;
             only each unit's input is kept (activation checkpointing).
  backward   in reverse: all-gather(u-1) is prefetched, unit u is recomputed and differentiated,
             its flat gradient is reduce-scattered (sum, then scaled by 1/ranks inside AdamW) on the
             communication stream, and the fused AdamW kernel updates this rank's shard right
             behind it, all overlapped with the backward compute of unit u-1.

Shards, gather buffers and gradient buffers live in symmetric memory registered as windows, so
the collectives run zero-copy over NVLink. With a host-only communicator (no GPU) the same code
runs synchronously on CPU tensors, which is how the engine is tested against plain autograd.

Reference parity: the reference serves this pattern through ncclAllGather / ncclReduceScatter on
user-registered buffers (src/collectives.cc, src/register/register.cc: ncclCommWindowRegister).
"""
import ctypes

import torch

from .. import _lib
from ..core import mem_alloc, mem_free
from ..models import llama as M


def _align(n, a):
    return (n + a - 1) // a * a


class _Unit:
    pass


class FSDPEngine:
    def __init__(self, comm, cfg, device="cuda", seed=0, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, symmetric=True, init_on_device=False):
        self.comm, self.cfg, self.device = comm, cfg, torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.n, self.rank = comm.nranks, comm.rank
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.step_count = 0
        self.symmetric = symmetric and self.cuda
        self._allocs = []
        self._wins = []
        self.lib = comm.lib            # collectives and memory: the communicator's library
        self.own = _lib.load()         # the optimizer kernel always comes from this package's library
        if self.cuda:
            self.own.b200FusedAdamW.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_size_t] + [ctypes.c_float] * 6 + [ctypes.c_int, ctypes.c_void_p]
        specs = M.unit_specs(cfg)
        self.units = []
        gen = torch.Generator().manual_seed(seed)
        for name, shapes in specs:
            u = _Unit()
            u.name, u.shapes, u.numel = name, shapes, M.numel(shapes)
            u.padded = _align(u.numel, self.n * 128)
            u.shard = u.padded // self.n
            if init_on_device and self.cuda:
                # large models: draw the unit on the GPU (same seed on every rank), keep this rank's slice
                dgen = torch.Generator(device=self.device).manual_seed(seed * 1000003 + len(self.units))
                full = torch.zeros(u.padded, dtype=torch.bfloat16, device=self.device)
                off = 0
                for _, shape in shapes:
                    cnt = 1
                    for sdim in shape:
                        cnt *= sdim
                    if len(shape) == 1:
                        full[off:off + cnt] = 1.0
                    else:
                        full[off:off + cnt] = (torch.randn(cnt, generator=dgen, device=self.device) * 0.02).to(torch.bfloat16)
                    off += cnt
            else:
                full = torch.zeros(u.padded, dtype=torch.bfloat16)
                full[:u.numel] = M.init_flat(shapes, gen)      # every rank draws the same stream, keeps its slice
            mine = full[self.rank * u.shard:(self.rank + 1) * u.shard]
            u.param = self._buffer(u.shard, torch.bfloat16)
            u.param.copy_(mine)
            u.grad = self._buffer(u.shard, torch.bfloat16)
            u.master = mine.float().to(self.device)
            u.m = torch.zeros(u.shard, dtype=torch.float32, device=self.device)
            u.v = torch.zeros(u.shard, dtype=torch.float32, device=self.device)
            self.units.append(u)
        biggest = max(u.padded for u in self.units)
        self.gbuf = [self._buffer(biggest, torch.bfloat16) for _ in range(2)]
        self.ggrad = [self._buffer(biggest, torch.bfloat16) for _ in range(2)]
        if self.cuda:
            self.comm_stream = torch.cuda.Stream(device=self.device)
            ev = lambda: torch.cuda.Event()   # noqa: E731
            self.ev_gathered = [ev() for _ in range(2)]
            self.ev_free = [ev() for _ in range(2)]
            self.ev_grad_ready = [ev() for _ in range(2)]
            self.ev_grad_free = [ev() for _ in range(2)]
            for e in self.ev_free + self.ev_grad_free:
                e.record()
        self.collectives = 0      # all-gathers + reduce-scatters issued (for reporting)
        self.kernels = 0          # AdamW launches

    # ------------------------------------------------------------------ memory
    def _buffer(self, numel, dtype):
        if not self.symmetric:
            return torch.zeros(numel, dtype=dtype, device=self.device)
        from ..utils.perf import tensor_at
        es = torch.empty(0, dtype=dtype).element_size()
        nbytes = _align(numel * es, 4096)
        ptr = mem_alloc(nbytes, self.lib)
        raw = tensor_at(ptr, nbytes)
        raw.zero_()
        self._wins.append(self.comm.register_window(raw))
        self._allocs.append(ptr)
        return raw[:numel * es].view(dtype)

    def close(self):
        if self.cuda:
            torch.cuda.synchronize()
        for w in self._wins:
            self.comm.deregister_window(w)
        for p in self._allocs:
            mem_free(p, self.lib)
        self._wins, self._allocs = [], []

    # ------------------------------------------------------------------ communication
    def _gather(self, idx, slot):
        u = self.units[idx]
        dst = self.gbuf[slot][:u.padded]
        if self.cuda:
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(self.ev_free[slot])
                self.comm.all_gather(u.param, dst, stream=self.comm_stream)
                self.ev_gathered[slot].record(self.comm_stream)
        else:
            self.comm.all_gather(u.param, dst)
        self.collectives += 1

    def _wait_gathered(self, slot):
        if self.cuda:
            torch.cuda.current_stream().wait_event(self.ev_gathered[slot])

    def _release(self, slot):
        if self.cuda:
            self.ev_free[slot].record(torch.cuda.current_stream())

    def _reduce_and_update(self, idx, gslot):
        """Reduce-scatter of ggrad[gslot] into the unit's gradient shard, then AdamW on the shard."""
        u = self.units[idx]
        src = self.ggrad[gslot][:u.padded]
        if self.cuda:
            self.ev_grad_ready[gslot].record(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(self.ev_grad_ready[gslot])
                self.comm.reduce_scatter(src, u.grad, stream=self.comm_stream)
                self.ev_grad_free[gslot].record(self.comm_stream)
                self._adamw(u, self.comm_stream)
        else:
            self.comm.reduce_scatter(src, u.grad)
            self._adamw(u, None)
        self.collectives += 1

    def _adamw(self, u, stream):
        b1, b2 = self.betas
        step = self.step_count
        if self.cuda:
            rc = self.own.b200FusedAdamW(u.master.data_ptr(), u.m.data_ptr(), u.v.data_ptr(), u.grad.data_ptr(), u.param.data_ptr(), u.shard,
                                         self.lr, b1, b2, self.eps, self.wd, 1.0 / self.n, step, stream.cuda_stream)
            _lib.check(rc, "b200FusedAdamW", self.own)
            self.kernels += 1
            return
        g = u.grad.float() / self.n
        u.m.mul_(b1).add_(g, alpha=1 - b1)
        u.v.mul_(b2).addcmul_(g, g, value=1 - b2)
        mhat = u.m / (1 - b1 ** step)
        denom = u.v.sqrt() / (1 - b2 ** step) ** 0.5 + self.eps
        u.master.mul_(1 - self.lr * self.wd).addcdiv_(mhat, denom, value=-self.lr)
        u.param.copy_(u.master.to(torch.bfloat16))

    def _write_grads(self, idx, gslot, grads):
        u = self.units[idx]
        if self.cuda:
            torch.cuda.current_stream().wait_event(self.ev_grad_free[gslot])
        flat = self.ggrad[gslot]
        off = 0
        for g in grads:
            flat[off:off + g.numel()].copy_(g.reshape(-1))
            off += g.numel()
        if u.padded > off:
            flat[off:u.padded].zero_()

    # ------------------------------------------------------------------ one training step
    def step(self, tokens, targets):
        """tokens, targets: int64 [B, S] (host or device). Returns the loss of this rank as a 0-d tensor."""
        cfg, U = self.cfg, len(self.units)
        self.step_count += 1
        tokens = tokens.to(self.device, non_blocking=True)
        targets = targets.to(self.device, non_blocking=True)
        rope = M.rope_tables(cfg, tokens.shape[1], self.device)
        saved = [None] * U

        def params(idx, slot, need_grad):
            u = self.units[idx]
            flat = self.gbuf[slot][:u.numel]
            vs = M.views(flat, u.shapes)
            if need_grad:
                vs = {k: t.detach().requires_grad_(True) for k, t in vs.items()}
            return vs

        def run(idx, vs, x):
            if idx == 0:
                return M.embed(tokens, vs)
            if idx == U - 1:
                return M.head_loss(x, vs, cfg, targets)
            return M.decoder_layer(x, vs, cfg, rope)

        # forward (the head is differentiated at once: its recompute would be wasted work)
        self._gather(0, 0)
        x = None
        for idx in range(U - 1):
            self._gather(idx + 1, (idx + 1) % 2)
            self._wait_gathered(idx % 2)
            saved[idx] = x
            with torch.no_grad():
                x = run(idx, params(idx, idx % 2, False), x)
            self._release(idx % 2)
        # head: forward + backward
        idx = U - 1
        slot = idx % 2
        self._wait_gathered(slot)
        vs = params(idx, slot, True)
        xin = x.detach().requires_grad_(True)
        loss = run(idx, vs, xin)
        names = [n for n, _ in self.units[idx].shapes]
        grads = torch.autograd.grad(loss, [xin] + [vs[n] for n in names])
        self._gather(idx - 1, (idx - 1) % 2)
        self._release(slot)
        self._write_grads(idx, idx % 2, grads[1:])
        self._reduce_and_update(idx, idx % 2)
        gx = grads[0]
        del grads, vs, xin, x
        # backward through the layers and the embedding
        for idx in range(U - 2, -1, -1):
            slot = idx % 2
            if idx - 1 >= 0:
                self._gather(idx - 1, (idx - 1) % 2)
            self._wait_gathered(slot)
            vs = params(idx, slot, True)
            names = [n for n, _ in self.units[idx].shapes]
            with torch.enable_grad():
                if idx == 0:
                    out = run(idx, vs, None)
                    grads = (None,) + torch.autograd.grad(out, [vs[n] for n in names], gx)
                else:
                    xin = saved[idx].detach().requires_grad_(True)
                    out = run(idx, vs, xin)
                    grads = torch.autograd.grad(out, [xin] + [vs[n] for n in names], gx)
            self._release(slot)
            self._write_grads(idx, idx % 2, grads[1:])
            self._reduce_and_update(idx, idx % 2)
            gx = grads[0]
            saved[idx] = None
            del grads, vs, out
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        return loss.detach()

    # ------------------------------------------------------------------ inspection
    def full_params(self):
        """List of whole flat fp32 parameter buffers (gathers every unit; for tests)."""
        out = []
        for idx, u in enumerate(self.units):
            self._gather(idx, 0)
            self._wait_gathered(0)
            if self.cuda:
                torch.cuda.synchronize()
            out.append(self.gbuf[0][:u.numel].float().cpu().clone())
            self._release(0)
        return out
