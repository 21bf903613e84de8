"""Llama-shaped decoder written as pure functions over flat parameter buffers.

Each FSDP unit (embedding, one decoder layer, output head) owns one flat bf16 buffer; `layer_views`
cuts a gathered buffer into the weight matrices without copying, so the sharding engine can
all-gather / reduce-scatter whole units with one collective each. The maths is standard
pre-norm Llama: RMSNorm, rotary embeddings, grouped-query causal attention, SwiGLU.

The communication pattern this model exists to drive (per-layer parameter all-gather and gradient
reduce-scatter, overlapped with compute) is the one the reference documents for FSDP users in
docs/userguide (buffer registration for all-gather / reduce-scatter) and serves through
ncclAllGather / ncclReduceScatter (src/collectives.cc).
"""
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class LlamaConfig:
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    eps: float = 1e-5

    @property
    def head_dim(self):
        return self.hidden // self.heads

    @staticmethod
    def llama3_8b():
        return LlamaConfig()

    @staticmethod
    def tiny(layers=2):
        return LlamaConfig(layers=layers, hidden=64, heads=4, kv_heads=2, ffn=128, vocab=256, rope_theta=10000.0)


def layer_shapes(cfg):
    """Ordered (name, shape) of one decoder layer's parameters inside its flat buffer."""
    h, kv, f = cfg.hidden, cfg.kv_heads * cfg.head_dim, cfg.ffn
    return [("norm1", (h,)), ("wq", (h, h)), ("wk", (kv, h)), ("wv", (kv, h)), ("wo", (h, h)),
            ("norm2", (h,)), ("w_gate", (f, h)), ("w_up", (f, h)), ("w_down", (h, f))]


def embed_shapes(cfg):
    return [("tok", (cfg.vocab, cfg.hidden))]


def head_shapes(cfg):
    return [("norm", (cfg.hidden,)), ("out", (cfg.vocab, cfg.hidden))]


def numel(shapes):
    return sum(math.prod(s) for _, s in shapes)


def views(flat, shapes):
    """Dict of weight views into `flat` (no copies)."""
    out, off = {}, 0
    for name, shape in shapes:
        n = math.prod(shape)
        out[name] = flat[off:off + n].view(shape)
        off += n
    return out


def init_flat(shapes, generator, std=0.02, dtype=torch.bfloat16):
    """Random-init flat buffer: N(0, std) matrices, unit norm gains."""
    parts = []
    for name, shape in shapes:
        if len(shape) == 1:
            parts.append(torch.ones(shape, dtype=torch.float32))
        else:
            parts.append(torch.randn(shape, generator=generator, dtype=torch.float32) * std)
    return torch.cat([p.reshape(-1) for p in parts]).to(dtype)


def rmsnorm(x, gain, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * gain


def rope_tables(cfg, seq, device, dtype=torch.float32):
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=device, dtype=torch.float32) / cfg.head_dim))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x, cos, sin):
    # x [B, S, H, D]; rotate pairs (first half, second half)
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def decoder_layer(x, p, cfg, rope):
    """x [B, S, hidden] -> [B, S, hidden]; p = views(flat, layer_shapes(cfg))."""
    B, S, _ = x.shape
    cos, sin = rope
    h = rmsnorm(x, p["norm1"], cfg.eps)
    q = F.linear(h, p["wq"]).view(B, S, cfg.heads, cfg.head_dim)
    k = F.linear(h, p["wk"]).view(B, S, cfg.kv_heads, cfg.head_dim)
    v = F.linear(h, p["wv"]).view(B, S, cfg.kv_heads, cfg.head_dim)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, enable_gqa=True)
    x = x + F.linear(a.transpose(1, 2).reshape(B, S, cfg.hidden), p["wo"])
    h = rmsnorm(x, p["norm2"], cfg.eps)
    return x + F.linear(F.silu(F.linear(h, p["w_gate"])) * F.linear(h, p["w_up"]), p["w_down"])


def embed(tokens, p):
    return F.embedding(tokens, p["tok"])


def head_loss(x, p, cfg, targets):
    """Mean next-token cross entropy (fp32 log-softmax) of the final hidden states."""
    logits = F.linear(rmsnorm(x, p["norm"], cfg.eps), p["out"])
    return F.cross_entropy(logits.float().view(-1, cfg.vocab), targets.reshape(-1))


def unit_specs(cfg):
    """The FSDP units of the model in execution order: (name, shapes)."""
    return [("embed", embed_shapes(cfg))] + [("layer%d" % i, layer_shapes(cfg)) for i in range(cfg.layers)] + [("head", head_shapes(cfg))]


def reference_loss(flats, cfg, tokens, targets):
    """Plain autograd forward over whole (unsharded) flat buffers; the oracle of the sharded engine."""
    x = embed(tokens, views(flats[0], embed_shapes(cfg)))
    rope = rope_tables(cfg, tokens.shape[1], tokens.device)
    for i in range(cfg.layers):
        x = decoder_layer(x, views(flats[1 + i], layer_shapes(cfg)), cfg, rope)
    return head_loss(x, views(flats[-1], head_shapes(cfg)), cfg, targets)
