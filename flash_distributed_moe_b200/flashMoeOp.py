"""Drop-in module wrapper: runs a Qwen3 sparse-MoE block's forward through the launcher, in place.

Mirrors the reference's FlashMoeBlockWrapper (test/singleGPU/python/flashMoeOp.py:7-38) without
importing vLLM: any module exposing `gate.weight` [E,H], `experts.w13_weight` [E,2I,H] and
`experts.w2_weight` [E,H,I] works (vLLM's Qwen3MoeSparseMoeBlock has exactly these).
"""
from __future__ import annotations

import torch

from .flashMoeLauncher import MoeKernelLauncher


class FlashMoeBlockWrapper(torch.nn.Module):
    def __init__(self, qwen3MoeSparseMoeBlockModule: torch.nn.Module, maxTokens: int, topk: int = 8):
        super().__init__()
        self.qwen3MoeSparseMoeBlockModule = qwen3MoeSparseMoeBlockModule
        self.launcher = MoeKernelLauncher()
        gateWeights = qwen3MoeSparseMoeBlockModule.gate.weight
        ffn1ExpertWeights = qwen3MoeSparseMoeBlockModule.experts.w13_weight
        ffn2ExpertWeights = qwen3MoeSparseMoeBlockModule.experts.w2_weight
        uniqueid = self.launcher.getDistributedUniqueId(empty=True)
        self.launcher.create(gateWeights.detach(), ffn1ExpertWeights.detach(), ffn2ExpertWeights.detach(),
                             maxTokens, uniqueid, 0, 1, topk=topk)
        self.maxTokens = maxTokens

    def __del__(self):
        try:
            self.launcher.destroy()
        except Exception:
            pass

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        num_tokens, _ = hidden_states.shape
        if num_tokens <= self.maxTokens:
            # in-place: output memory = input memory
            self.launcher.launch(hidden_states, hidden_states)
            return hidden_states
        # larger batches go to the wrapped block (the reference calls a non-existent super().forward here)
        return self.qwen3MoeSparseMoeBlockModule(hidden_states)
