"""GPT-2 shaped decoder (the DDP benchmark model).

Architecture of the reference's ``train_bench.py`` model (scripts/gpu/train_bench.py:158-189):
pre-LayerNorm blocks of causal self-attention and a 4x GELU(tanh) MLP, learned positions,
tied input/output embedding.  ``gpt2-small``: 12 layers, 12 heads, width 768, vocabulary
50257, context 1024 (124 M parameters).  Weights are initialised N(0, 0.02), biases zero,
LayerNorm to identity.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from gpubridge_b200.models.attention import causal_attention
from gpubridge_b200.ops.layernorm import FusedLayerNorm


@dataclass(frozen=True)
class GPTConfig:
    layers: int = 12
    heads: int = 12
    width: int = 768
    vocab: int = 50257
    context: int = 1024
    mlp: int = 3072


CONFIGS = {
    "gpt2-small": GPTConfig(),
    "gpt2-tiny": GPTConfig(layers=2, heads=2, width=64, vocab=257, context=64, mlp=256),
}


class Block(nn.Module):
    def __init__(self, c: GPTConfig) -> None:
        super().__init__()
        self.heads = c.heads
        self.ln1, self.ln2 = FusedLayerNorm(c.width), FusedLayerNorm(c.width)
        self.qkv, self.proj = nn.Linear(c.width, 3 * c.width), nn.Linear(c.width, c.width)
        self.fc, self.out = nn.Linear(c.width, c.mlp), nn.Linear(c.mlp, c.width)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, t, w = x.shape
        qkv = self.qkv(self.ln1(x)).view(b, t, 3, self.heads, w // self.heads)
        q, k, v = (z.transpose(1, 2) for z in qkv.unbind(2))
        y = causal_attention(q, k, v)
        x = x + self.proj(y.transpose(1, 2).reshape(b, t, w))
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class GPT(nn.Module):
    def __init__(self, c: GPTConfig) -> None:
        super().__init__()
        self.config = c
        self.padded_vocab = -(-c.vocab // 64) * 64
        self.tok = nn.Embedding(self.padded_vocab, c.width)
        self.pos = nn.Embedding(c.context, c.width)
        self.blocks = nn.ModuleList(Block(c) for _ in range(c.layers))
        self.ln = FusedLayerNorm(c.width)
        self.head = nn.Linear(c.width, self.padded_vocab, bias=False)
        self.head.weight = self.tok.weight          # tied, as in GPT-2
        self.apply(self._init)
        with torch.no_grad():
            self.tok.weight[c.vocab:].zero_()
        #: set by a trainer that calls ``loss.backward()`` itself (see fused_cross_entropy)
        self.unit_grad = False

    @staticmethod
    def _init(module: nn.Module) -> None:
        if isinstance(module, (nn.Linear, nn.Embedding)):
            nn.init.normal_(module.weight, mean=0.0, std=0.02)
            if getattr(module, "bias", None) is not None:
                nn.init.zeros_(module.bias)

    def hidden(self, idx: torch.Tensor) -> torch.Tensor:
        x = self.tok(idx) + self.pos(torch.arange(idx.shape[1], device=idx.device))
        for block in self.blocks:
            x = block(x)
        return self.ln(x)

    def forward(self, idx: torch.Tensor) -> torch.Tensor:
        return self.head(self.hidden(idx))[..., :self.config.vocab]

    def loss(self, idx: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        from gpubridge_b200.ops.xent import fused_cross_entropy
        logits = self.head(self.hidden(idx))
        return fused_cross_entropy(logits.view(-1, logits.shape[-1]), targets.reshape(-1),
                                   self.config.vocab, unit_grad=self.unit_grad)


def build(name: str = "gpt2-small") -> GPT:
    return GPT(CONFIGS[name])


def synthetic_tokens(config: GPTConfig, batch: int, seq: int, seed: int = 0,
                     count: int = 1) -> list[tuple[torch.Tensor, torch.Tensor]]:
    """``count`` (input, target) pairs of uniform token ids in [0, vocab), on the host."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(count):
        tokens = torch.randint(config.vocab, (batch, seq + 1), generator=g)
        out.append((tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()))
    return out
