"""Seeded synthetic inputs with the Qwen3 layer shapes (real checkpoints are not available offline).

Weights N(0, 0.02), activations N(0, 1), both rounded to bf16, from a torch CPU generator so that
the CPU checker and the GPU see identical values.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class LayerShape:
    name: str
    hidden: int
    inter: int
    experts: int
    topk: int


QWEN3_30B_A3B = LayerShape("Qwen3-30B-A3B", 2048, 768, 128, 8)
QWEN3_235B_A22B = LayerShape("Qwen3-235B-A22B", 4096, 1536, 128, 8)
TINY = LayerShape("tiny", 256, 128, 32, 4)


def make_weights(shape: LayerShape, seed: int = 0, experts_slice=None, std: float = 0.02):
    """(gate [E,H], w13 [E,2I,H], w2 [E,H,I]) bf16 on CPU.  `experts_slice` = (first, count) keeps only
    that contiguous shard of the expert weights (expert parallelism); the gate is always whole."""
    g = torch.Generator().manual_seed(seed)
    gate = (torch.randn(shape.experts, shape.hidden, generator=g) * std).to(torch.bfloat16)
    first, count = experts_slice if experts_slice else (0, shape.experts)
    w13 = torch.empty(count, 2 * shape.inter, shape.hidden, dtype=torch.bfloat16)
    w2 = torch.empty(count, shape.hidden, shape.inter, dtype=torch.bfloat16)
    for e in range(shape.experts):
        # one generator stream per expert so that a shard equals the same experts of the whole
        ge = torch.Generator().manual_seed(seed * 1000003 + 17 + e)
        if first <= e < first + count:
            w13[e - first] = (torch.randn(2 * shape.inter, shape.hidden, generator=ge) * std).to(torch.bfloat16)
            w2[e - first] = (torch.randn(shape.hidden, shape.inter, generator=ge) * std).to(torch.bfloat16)
    return gate, w13, w2


def make_tokens(shape: LayerShape, tokens: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed * 7919 + 1)
    return torch.randn(tokens, shape.hidden, generator=g).to(torch.bfloat16)


def add_zipf_bias(shape: LayerShape, gate: torch.Tensor, tokens: torch.Tensor, s: float = 1.2,
                  scale: float = 1.0, seed: int = 0):
    """Skews routing without touching the interface: the last activation column becomes exactly 1 and
    the gate weight of expert e in that column becomes scale * (-s * ln rank_e), the ranks being a
    seeded permutation of the experts.  Returns (gate, tokens) copies."""
    g = torch.Generator().manual_seed(seed + 4242)
    perm = torch.randperm(shape.experts, generator=g)
    rank = torch.empty(shape.experts, dtype=torch.float32)
    rank[perm] = torch.arange(1, shape.experts + 1, dtype=torch.float32)
    gate = gate.clone()
    tokens = tokens.clone()
    gate[:, -1] = (scale * (-s) * torch.log(rank)).to(torch.bfloat16)
    tokens[:, -1] = 1.0
    return gate, tokens
