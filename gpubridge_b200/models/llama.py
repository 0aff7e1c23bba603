"""Llama-style decoder: RMSNorm, rotary positions, grouped-query attention, SwiGLU.

The FSDP2 / HSDP benchmark models.  Named shapes: the reference's ``llama-tiny/125m/350m/1b``
(scripts/gpu/llama.py:49-58) plus the two large benchmark shapes - ``llama-1.3b`` (24 layers,
d_model 2048, 16 heads, FFN 5632, vocabulary 32000) and ``llama3-8b`` (32 layers, d_model 4096,
32 query / 8 KV heads, FFN 14336, vocabulary 128256).  Weights are N(0, 0.02) from a CPU
generator with a fixed seed, so every rank (and a single-process oracle) builds the same model.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from gpubridge_b200.models.attention import causal_attention


@dataclass(frozen=True)
class LlamaConfig:
    layers: int
    width: int
    heads: int
    kv_heads: int
    ffn: int
    vocab: int
    context: int = 2048
    rope_base: float = 10000.0
    eps: float = 1e-5


CONFIGS = {
    "llama-tiny": LlamaConfig(2, 64, 4, 2, 176, 256, 64),
    "llama-mini": LlamaConfig(4, 64, 4, 2, 176, 256, 64),          # four blocks: pipelines of up to four stages on CPU
    "llama-125m": LlamaConfig(12, 768, 12, 12, 2048, 32000, 2048),
    "llama-350m": LlamaConfig(24, 1024, 16, 16, 2816, 32000, 2048),
    "llama-1b": LlamaConfig(16, 2048, 32, 8, 8192, 32000, 2048),
    "llama-1.3b": LlamaConfig(24, 2048, 16, 16, 5632, 32000, 2048),
    "llama3-8b": LlamaConfig(32, 4096, 32, 8, 14336, 128256, 4096, rope_base=500000.0),
}


class RMSNorm(nn.Module):
    def __init__(self, width: int, eps: float) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def rope_tables(head_dim: int, length: int, base: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / base ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim)
    angle = torch.outer(torch.arange(length, device=device, dtype=torch.float32), inv)
    return angle.cos(), angle.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x``: [batch, heads, time, head_dim]; rotates pairs (even, odd halves)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half].float(), x[..., half:].float()
    c, s = cos[: x.shape[-2]], sin[: x.shape[-2]]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1).to(x.dtype)


class Block(nn.Module):
    def __init__(self, c: LlamaConfig) -> None:
        super().__init__()
        self.heads, self.kv_heads, self.head_dim = c.heads, c.kv_heads, c.width // c.heads
        self.attn_norm, self.ffn_norm = RMSNorm(c.width, c.eps), RMSNorm(c.width, c.eps)
        self.wq = nn.Linear(c.width, c.heads * self.head_dim, bias=False)
        self.wk = nn.Linear(c.width, c.kv_heads * self.head_dim, bias=False)
        self.wv = nn.Linear(c.width, c.kv_heads * self.head_dim, bias=False)
        self.wo = nn.Linear(c.heads * self.head_dim, c.width, bias=False)
        self.gate = nn.Linear(c.width, c.ffn, bias=False)
        self.up = nn.Linear(c.width, c.ffn, bias=False)
        self.down = nn.Linear(c.ffn, c.width, bias=False)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        b, t, _ = x.shape
        h = self.attn_norm(x)
        q = self.wq(h).view(b, t, self.heads, self.head_dim).transpose(1, 2)
        k = self.wk(h).view(b, t, self.kv_heads, self.head_dim).transpose(1, 2)
        v = self.wv(h).view(b, t, self.kv_heads, self.head_dim).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        y = causal_attention(q, k, v, enable_gqa=self.kv_heads != self.heads)
        x = x + self.wo(y.transpose(1, 2).reshape(b, t, -1))
        h = self.ffn_norm(x)
        return x + self.down(F.silu(self.gate(h)) * self.up(h))


class Llama(nn.Module):
    def __init__(self, c: LlamaConfig) -> None:
        super().__init__()
        self.config = c
        self.embed = nn.Embedding(c.vocab, c.width)
        self.blocks = nn.ModuleList(Block(c) for _ in range(c.layers))
        self.norm = RMSNorm(c.width, c.eps)
        self.head = nn.Linear(c.width, c.vocab, bias=False)
        self.unit_grad = False

    def forward(self, idx: torch.Tensor) -> torch.Tensor:
        cos, sin = rope_tables(self.config.width // self.config.heads, idx.shape[1],
                               self.config.rope_base, idx.device)
        x = self.embed(idx)
        for block in self.blocks:
            x = block(x, cos, sin)
        return self.head(self.norm(x))

    def loss(self, idx: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        from gpubridge_b200.ops.xent import fused_cross_entropy
        logits = self(idx)
        return fused_cross_entropy(logits.view(-1, logits.shape[-1]), targets.reshape(-1),
                                   self.config.vocab, unit_grad=self.unit_grad)


def build(name: str, seed: int = 0, device="cpu", dtype=torch.float32, rng: str = "cpu") -> Llama:
    """The named model with deterministic N(0, 0.02) weights (norm weights stay 1).  Built on
    the meta device and materialised on ``device`` so an 8 B model never sits in host memory
    twice.  ``rng="cpu"`` draws the weights from a CPU generator (the same values on any
    machine, as the reference's models do); ``rng="device"`` draws them on ``device`` (seconds
    instead of minutes for billions of parameters; the same values on the same kind of GPU)."""
    config = CONFIGS[name]
    with torch.device("meta"):
        model = Llama(config)
    model.to_empty(device=device)
    generator = torch.Generator(device="cpu").manual_seed(seed)
    on_device = rng == "device" and torch.device(device).type == "cuda"
    if on_device:
        generator = torch.Generator(device=device).manual_seed(seed)
    with torch.no_grad():
        for parameter in model.parameters():
            if parameter.dim() == 1:
                parameter.fill_(1.0)
            elif on_device:
                parameter.normal_(0.0, 0.02, generator=generator)
            else:
                values = torch.empty(parameter.shape, dtype=torch.float32)
                values.normal_(0.0, 0.02, generator=generator)
                parameter.copy_(values)
    return model.to(dtype)


def synthetic_tokens(config: LlamaConfig, batch: int, seq: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(config.vocab, (batch, seq + 1), generator=g)
    return tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()


def rule_batch(config: LlamaConfig, step: int, rows: int, seq: int, seed: int = 0):
    """The whole batch of training step ``step``: ``rows`` (input, target) sequences that are
    the same whatever the world size, so runs at different scales see the same data and
    their loss curves can be laid over each other.  The tokens follow a rule a model can
    learn - each token is an affine function of the one before it plus one of four small
    offsets - so the loss falls instead of sitting at log(vocab) as it does on uniform
    noise.  Same purpose as the reference's ``global_batch`` (scripts/gpu/llama.py:170-184)."""
    g = torch.Generator().manual_seed(seed * 1_000_003 + step)
    first = torch.randint(config.vocab, (rows, 1), generator=g)
    jitter = torch.randint(4, (rows, seq), generator=g)
    columns = [first[:, 0]]
    for i in range(seq):
        columns.append((columns[-1] * 7 + 13 + jitter[:, i]) % config.vocab)
    tokens = torch.stack(columns, dim=1)
    return tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()
