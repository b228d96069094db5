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
# one rank's share of the Qwen3-235B-A22B layer when its 128 experts are spread over 8 GPUs: same
# hidden and intermediate sizes (the shape-dependent code paths), 16 experts, so that tests stay light
QWEN3_235B_E16 = LayerShape("Qwen3-235B-A22B-16-experts", 4096, 1536, 16, 8)
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


def zipf_inclusion_target(experts: int, topk: int, s: float) -> torch.Tensor:
    """Share of the tokens that select the expert of popularity rank r = 1..E when popularity follows
    Zipf(s) and every token selects `topk` distinct experts: proportional to r^-s, capped at 1 (an
    expert cannot be selected more than once per token), summing to topk."""
    w = torch.arange(1, experts + 1, dtype=torch.float64) ** (-s)
    pi = torch.zeros(experts, dtype=torch.float64)
    capped = torch.zeros(experts, dtype=torch.bool)
    for _ in range(experts):
        free = ~capped
        scale = (topk - capped.sum().item()) / w[free].sum().item()
        pi[free] = w[free] * scale
        pi[capped] = 1.0
        over = (pi > 1.0) & free
        if not over.any():
            break
        capped |= over
    return pi.to(torch.float32)


def zipf_routing(shape: LayerShape, gate: torch.Tensor, tokens: torch.Tensor, s: float = 1.2, seed: int = 0):
    """Gate and tokens biased so that expert popularity follows Zipf(s): the last activation column
    becomes exactly 1 and the gate weight of every expert in that column a bias (the reference's way of
    steering the routing without touching the interface, test/common/moeTools.h:187-207).  The biases
    start from -s * ln(rank), the ranks being a seeded permutation of the experts, and are then fitted
    on a fixed seeded token sample so that the share of tokens selecting each expert approaches the
    target (zipf_inclusion_target).  The same inputs give the same biases on every rank.
    Returns (gate, tokens, info); info holds the realised shares."""
    E, K = shape.experts, shape.topk
    g = torch.Generator().manual_seed(seed + 977)
    sample = torch.randn(4096, shape.hidden, generator=g).to(torch.bfloat16)
    sample[:, -1] = 1.0
    perm = torch.randperm(E, generator=torch.Generator().manual_seed(seed + 4242))
    rank = torch.empty(E, dtype=torch.float32)
    rank[perm] = torch.arange(1, E + 1, dtype=torch.float32)
    target = zipf_inclusion_target(E, K, s)[(rank - 1).long()]  # per expert
    base = sample[:, :-1].float() @ gate[:, :-1].float().t()
    bias = -s * torch.log(rank)
    eps = 1.0 / (2 * sample.shape[0])
    logit = lambda p: torch.log(p.clamp(eps, 1 - eps)) - torch.log1p(-p.clamp(eps, 1 - eps))  # noqa: E731
    for _ in range(40):
        b16 = bias.to(torch.bfloat16).float()
        idx = (base + b16).topk(K, dim=1).indices
        share = torch.bincount(idx.flatten(), minlength=E).float() / sample.shape[0]
        bias = bias + 0.5 * (logit(target) - logit(share)).clamp(-2.0, 2.0)
        bias = bias - bias.max()
    b16 = bias.to(torch.bfloat16)
    idx = (base + b16.float()).topk(K, dim=1).indices
    share = torch.bincount(idx.flatten(), minlength=E).float() / sample.shape[0]
    order = torch.argsort(rank)
    gate_b, tokens_b = gate.clone(), tokens.clone()
    gate_b[:, -1] = b16
    tokens_b[:, -1] = 1.0
    info = {"zipf_s": s, "l1_distance_to_target": round((share - target).abs().sum().item(), 4),
            "selection_share_realised_top8": [round(v, 4) for v in share[order][:8].tolist()],
            "selection_share_target_top8": [round(v, 4) for v in target[order][:8].tolist()]}
    return gate_b, tokens_b, info
