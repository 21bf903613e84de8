"""Context (sequence) parallelism recipes over the library's point-to-point and all-to-all calls.

ring_attention   every rank holds a contiguous slice of the sequence. Key / value blocks travel
                 round the ring with one grouped ncclSend + ncclRecv per step into a second buffer
                 while the current block is being used (double buffering; on a GPU the exchange runs
                 on a communication stream). Partial results are merged with the running-maximum
                 ("online softmax") update, so the result equals attention over the whole sequence.
ulysses_*        all-to-all that swaps the sharded dimension: from "sequence sharded, all heads"
                 to "all of the sequence, heads sharded" before attention and back after it.

The attention arithmetic is plain PyTorch: these are recipes for the communication pattern, not
attention kernels. Reference parity: the reference ships the primitives only (grouped ncclSend /
ncclRecv ring of docs/examples/02_point_to_point/01_ring_pattern, ncclAlltoAll of src/collectives.cc).
"""
import math

import torch

from ..core import group


def _block(q, k, v, scale, mask):
    """Scores of one key / value block: returns (block maximum, exp-sum, unnormalised output), fp32."""
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale          # [B, H, Sq, Sk]
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    m = s.amax(dim=-1, keepdim=True)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)                    # fully masked rows
    p = torch.exp(s - m)
    if mask is not None:
        p = p.masked_fill(~mask, 0.0)
    return m, p.sum(dim=-1, keepdim=True), torch.matmul(p, v.float())


def ring_attention(comm, q, k, v, causal=False, stream=None):
    """q, k, v: [batch, heads, local sequence, head dim]; rank r holds positions [r * S, (r + 1) * S).
    Returns this rank's slice of softmax(q k^T / sqrt(d)) v over the whole sequence, in q's dtype."""
    n, rank = comm.nranks, comm.rank
    cuda = q.is_cuda
    scale = 1.0 / math.sqrt(q.shape[-1])
    S = q.shape[2]
    kv = [torch.stack((k, v)).contiguous(), None]
    kv[1] = torch.empty_like(kv[0])
    comm_stream = stream if stream is not None else (torch.cuda.Stream(device=q.device) if cuda and n > 1 else None)
    m_run = torch.full(q.shape[:3] + (1,), float("-inf"), dtype=torch.float32, device=q.device)
    l_run = torch.zeros_like(m_run)
    o_run = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    tri = torch.ones(S, S, dtype=torch.bool, device=q.device).tril() if causal else None
    nxt, prv = (rank + 1) % n, (rank - 1) % n
    for step in range(n):
        cur, other = kv[step % 2], kv[(step + 1) % 2]
        done = None
        if step + 1 < n:
            # pass the block on while it is being used here
            if cuda:
                ready = torch.cuda.Event()
                ready.record()                      # `other` is no longer read, `cur` is complete
                with torch.cuda.stream(comm_stream):
                    comm_stream.wait_event(ready)
                    with group(comm.lib):
                        comm.send(cur, nxt, stream=comm_stream)
                        comm.recv(other, prv, stream=comm_stream)
                    done = torch.cuda.Event()
                    done.record(comm_stream)
            else:
                with group(comm.lib):
                    comm.send(cur, nxt)
                    comm.recv(other, prv)
        src = (rank - step) % n                     # the rank whose keys / values are in `cur`
        if not causal or src <= rank:
            mask = tri if causal and src == rank else None
            m_blk, l_blk, o_blk = _block(q, cur[0], cur[1], scale, mask)
            m_new = torch.maximum(m_run, m_blk)
            a_old = torch.exp(m_run - m_new)
            a_blk = torch.exp(m_blk - m_new)
            l_run = l_run * a_old + l_blk * a_blk
            o_run = o_run * a_old + o_blk * a_blk
            m_run = m_new
        if done is not None:
            torch.cuda.current_stream().wait_event(done)
    return (o_run / l_run).to(q.dtype)


def ulysses_scatter_heads(comm, x, stream=None):
    """[batch, local sequence, heads, dim] on every rank -> [batch, sequence, heads / n, dim]:
    rank r ends up with heads [r * H / n, (r + 1) * H / n) of every position. One ncclAlltoAll."""
    n = comm.nranks
    B, S, H, D = x.shape
    if H % n:
        raise ValueError("the number of heads must be a multiple of the number of ranks")
    if n == 1:
        return x
    send = x.reshape(B, S, n, H // n, D).permute(2, 0, 1, 3, 4).contiguous()    # [n, B, S, H/n, D]: block p goes to rank p
    recv = torch.empty_like(send)
    comm.all_to_all(send, recv, stream=stream)                                   # block p now holds rank p's positions
    return recv.permute(1, 0, 2, 3, 4).reshape(B, n * S, H // n, D)


def ulysses_gather_heads(comm, x, stream=None):
    """Inverse of ulysses_scatter_heads: [batch, sequence, heads / n, dim] -> [batch, local sequence, heads, dim]."""
    n = comm.nranks
    B, S_all, Hl, D = x.shape
    if S_all % n:
        raise ValueError("the sequence length must be a multiple of the number of ranks")
    if n == 1:
        return x
    S = S_all // n
    send = x.reshape(B, n, S, Hl, D).permute(1, 0, 2, 3, 4).contiguous()         # [n, B, S, H/n, D]: block p = rank p's positions
    recv = torch.empty_like(send)
    comm.all_to_all(send, recv, stream=stream)                                   # block p now holds rank p's heads
    return recv.permute(1, 2, 0, 3, 4).reshape(B, S, n * Hl, D)


def ulysses_attention(comm, q, k, v, causal=False):
    """q, k, v: [batch, local sequence, heads, dim]. Swaps to head sharding, runs full-sequence attention on
    this rank's heads, swaps back. Returns [batch, local sequence, heads, dim]."""
    qh, kh, vh = (ulysses_scatter_heads(comm, t).transpose(1, 2) for t in (q, k, v))     # [B, H/n, S_all, D]
    o = torch.nn.functional.scaled_dot_product_attention(qh.float(), kh.float(), vh.float(), is_causal=causal).to(q.dtype)
    return ulysses_gather_heads(comm, o.transpose(1, 2).contiguous())
