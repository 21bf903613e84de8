"""Data parallelism: gradient all-reduce in buckets, overlapped with the backward pass.

Parameters are packed, in reverse order (the order in which backward produces gradients), into flat
buckets of about ``bucket_bytes``. Every parameter's ``.grad`` is a view into its bucket, so autograd
accumulates straight into the communication buffer and no copy is needed. A post-accumulate hook
counts the gradients of a bucket; when the last one has arrived the bucket is all-reduced on the
communication stream (ncclAvg, or ncclSum when ``average=False``) while backward goes on with the
next layers. ``finish()`` makes the compute stream wait for all buckets.

On a GPU the buckets come from ncclMemAlloc and are registered as symmetric windows, which is what
lets the library run its one-kernel peer-load / multimem all-reduce without staging copies.

Reference parity: the reference is the substrate (ncclAllReduce with ncclAvg / pre-multiplied sum,
src/collectives.cc, src/enqueue.cc); bucketing is what its users (DDP trainers) build on top of it.
"""
import torch

from ..core import mem_alloc, mem_free


class GradientBuckets:
    def __init__(self, comm, params, bucket_bytes=32 << 20, average=True, symmetric=True):
        self.comm = comm
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("no parameter requires a gradient")
        self.device = self.params[0].device
        self.cuda = self.device.type == "cuda"
        self.symmetric = symmetric and self.cuda
        self.op = "avg" if average else "sum"
        self._allocs, self._wins, self._hooks = [], [], []
        self.buckets = []          # dicts: flat, params, pending, launched, event
        self.launched = 0          # all-reduces issued (for reporting)
        cur, cur_bytes = [], 0
        for p in reversed(self.params):
            nbytes = p.numel() * p.element_size()
            if cur and (cur_bytes + nbytes > bucket_bytes or p.dtype != cur[0].dtype):
                self._make_bucket(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
        if cur:
            self._make_bucket(cur)
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        for b in self.buckets:
            for p in b["params"]:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(b)))

    # ------------------------------------------------------------------ set-up
    def _flat(self, numel, dtype):
        if not self.symmetric:
            return torch.zeros(numel, dtype=dtype, device=self.device)
        from ..utils.perf import tensor_at
        es = torch.empty(0, dtype=dtype).element_size()
        nbytes = (numel * es + 4095) // 4096 * 4096
        ptr = mem_alloc(nbytes, self.comm.lib)
        raw = tensor_at(ptr, nbytes)
        raw.zero_()
        self._wins.append(self.comm.register_window(raw))
        self._allocs.append(ptr)
        return raw[:numel * es].view(dtype)

    def _make_bucket(self, params):
        # every gradient starts on a 16-byte boundary: the vector width of the reduction kernels
        es = params[0].element_size()
        step = max(1, 16 // es)
        offs, total = [], 0
        for p in params:
            offs.append(total)
            total += (p.numel() + step - 1) // step * step
        flat = self._flat(total, params[0].dtype)
        for p, off in zip(params, offs):
            p.grad = flat[off:off + p.numel()].view_as(p)
        self.buckets.append({"flat": flat, "params": params, "pending": len(params), "launched": False,
                             "event": torch.cuda.Event() if self.cuda else None})

    def _make_hook(self, bucket):
        def hook(_param):
            bucket["pending"] -= 1
            if bucket["pending"] == 0:
                self._launch(bucket)
        return hook

    # ------------------------------------------------------------------ communication
    def _launch(self, bucket):
        if bucket["launched"]:
            return
        bucket["launched"] = True
        self.launched += 1
        if self.cuda:
            ready = torch.cuda.Event()
            ready.record()                                   # the gradients of this bucket are complete on the compute stream
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                self.comm.all_reduce(bucket["flat"], op=self.op, stream=self.comm_stream)
                bucket["event"].record(self.comm_stream)
        else:
            self.comm.all_reduce(bucket["flat"], op=self.op)

    def finish(self):
        """Call after backward: reduces buckets whose hooks did not all fire (unused parameters) and makes
        the compute stream wait for every bucket; re-arms the buckets for the next step."""
        for b in self.buckets:
            self._launch(b)
        for b in self.buckets:
            if self.cuda:
                torch.cuda.current_stream().wait_event(b["event"])
            b["pending"], b["launched"] = len(b["params"]), False

    def zero_grad(self):
        for b in self.buckets:
            b["flat"].zero_()

    def close(self):
        if self.cuda:
            torch.cuda.synchronize()
        for h in self._hooks:
            h.remove()
        for p in self.params:
            p.grad = None
        for w in self._wins:
            self.comm.deregister_window(w)
        for ptr in self._allocs:
            mem_free(ptr, self.comm.lib)
        self._hooks, self._wins, self._allocs = [], [], []
