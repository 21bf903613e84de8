"""Pipeline parallelism over ncclSend / ncclRecv: each rank owns a contiguous block of decoder
layers (rank 0 also the embedding, the last rank the head) and activations of shape
[batch, seq, hidden] travel between neighbours as point-to-point messages.

Schedule: all forwards of the micro-batches, then all backwards in reverse (GPipe). Receives for
micro-batch i+1 are posted on the communication stream while micro-batch i computes, so the
transfer overlaps compute; sends are issued on the communication stream behind an event.

Reference parity: ncclSend / ncclRecv (src/collectives.cc, grouped by ncclGroupStart/End in
src/group.cc) used the way pipeline-parallel trainers use them.
"""
import torch

from ..models import llama as M


class PipelineStage:
    def __init__(self, comm, cfg, device="cuda", seed=0):
        self.comm, self.cfg, self.device = comm, cfg, torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.n, self.rank = comm.nranks, comm.rank
        if cfg.layers % self.n:
            raise ValueError("layers must divide evenly over the stages")
        per = cfg.layers // self.n
        self.first, self.last = self.rank == 0, self.rank == self.n - 1
        gen = torch.Generator().manual_seed(seed)
        specs = M.unit_specs(cfg)
        flats = [M.init_flat(shapes, gen) for _, shapes in specs]   # same stream on every rank; keep only this stage's units
        lo = 1 + self.rank * per
        self.layer_ids = list(range(lo, lo + per))
        self.params = {}
        keep = self.layer_ids + ([0] if self.first else []) + ([len(specs) - 1] if self.last else [])
        for i in keep:
            self.params[i] = flats[i].to(self.device).requires_grad_(True)
        self.specs = specs
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self.sends = self.recvs = 0

    # ------------------------------------------------------------------ messaging
    def _recv(self, shape, peer):
        buf = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
        if self.cuda:
            with torch.cuda.stream(self.comm_stream):
                self.comm.recv(buf, peer, stream=self.comm_stream)
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
            buf.record_stream(self.comm_stream)
        else:
            self.comm.recv(buf, peer)
            ev = None
        self.recvs += 1
        return buf, ev

    def _send(self, t, peer):
        t = t.contiguous()
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ev)
                self.comm.send(t, peer, stream=self.comm_stream)
            t.record_stream(self.comm_stream)
        else:
            self.comm.send(t, peer)
        self.sends += 1

    @staticmethod
    def _wait(ev):
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    # ------------------------------------------------------------------ compute
    def _forward_block(self, x, tokens, targets, rope):
        cfg = self.cfg
        if self.first:
            x = M.embed(tokens, M.views(self.params[0], M.embed_shapes(cfg)))
        for i in self.layer_ids:
            x = M.decoder_layer(x, M.views(self.params[i], M.layer_shapes(cfg)), cfg, rope)
        if self.last:
            return M.head_loss(x, M.views(self.params[len(self.specs) - 1], M.head_shapes(cfg)), cfg, targets)
        return x

    def forward_backward(self, micro_tokens, micro_targets):
        """micro_tokens / micro_targets: lists of int64 [B, S] tensors (every rank passes the same lists).
        Runs all forwards then all backwards; gradients accumulate in this stage's parameters.
        Returns the mean loss on the last stage, None elsewhere."""
        cfg = self.cfg
        mb = len(micro_tokens)
        B, S = micro_tokens[0].shape
        shape = (B, S, cfg.hidden)
        rope = M.rope_tables(cfg, S, self.device)
        inputs, outputs = [], []
        pending = self._recv(shape, self.rank - 1) if not self.first else None
        for i in range(mb):
            tok = micro_tokens[i].to(self.device)
            tgt = micro_targets[i].to(self.device)
            x = None
            if not self.first:
                x, ev = pending
                pending = self._recv(shape, self.rank - 1) if i + 1 < mb else None
                self._wait(ev)
                x.requires_grad_(True)
            y = self._forward_block(x, tok, tgt, rope)
            inputs.append(x)
            outputs.append(y)
            if not self.last:
                self._send(y.detach(), self.rank + 1)
        losses = []
        pending = self._recv(shape, self.rank + 1) if not self.last else None
        for i in range(mb - 1, -1, -1):
            if self.last:
                losses.append(outputs[i].detach())
                (outputs[i] / mb).backward()
            else:
                g, ev = pending
                pending = self._recv(shape, self.rank + 1) if i > 0 else None
                self._wait(ev)
                outputs[i].backward(g)
            if not self.first:
                self._send(inputs[i].grad, self.rank - 1)
            outputs[i] = None
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        return torch.stack(losses).mean() if self.last else None

    def forward_only(self, micro_tokens):
        """Inference-style pass: activations flow first -> last stage; returns final hidden states on the last stage."""
        cfg = self.cfg
        B, S = micro_tokens[0].shape
        rope = M.rope_tables(cfg, S, self.device)
        outs = []
        with torch.no_grad():
            for tok in micro_tokens:
                x = None
                if not self.first:
                    x, ev = self._recv((B, S, cfg.hidden), self.rank - 1)
                    self._wait(ev)
                else:
                    x = M.embed(tok.to(self.device), M.views(self.params[0], M.embed_shapes(cfg)))
                for i in self.layer_ids:
                    x = M.decoder_layer(x, M.views(self.params[i], M.layer_shapes(cfg)), cfg, rope)
                if not self.last:
                    self._send(x, self.rank + 1)
                else:
                    outs.append(x)
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        return outs
