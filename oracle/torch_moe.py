"""Plain-torch CPU restatement of the layer, the "CPU/torch path" timed beside the GPU numbers.

TEST INFRASTRUCTURE ONLY, like everything under oracle/: imported by tests/ (where it is checked
against the C restatement) and by the cpu_baseline leg of bench.py.  The shipped package never
imports it.

Same math as the reference's CPU layer (test/singleGPU/cpp/moe/reference/refFullMoe.h:9-69): gate
logits `x @ Wg^T` (refMoeGate.h:16-33), the top-k logits in descending order (refTopk.h:36-58),
softmax over the kept logits in double (refSoftmax.h:23-50), per expert
`silu(x @ W1^T) * (x @ W3^T)` with the gate projection in rows 0..I-1 of W13 (refExpertFFN1.h:31-65),
`@ W2^T`, and the weighted sum over the slots (refFullMoe.h:62-65).  The GEMMs run expert by expert
over all rows routed to the expert, in torch's own accumulation order, so results agree with the
reference's to fp32 rounding, not bit for bit, and two experts whose logits differ by less than that
rounding may swap places.
"""
from __future__ import annotations

import torch


def torch_moe(tokens: torch.Tensor, gate_w: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk: int):
    """tokens [T,H], gate_w [E,H], w13 [E,2I,H], w2 [E,H,I], all fp32 on the CPU.
    Returns (out [T,H], topk_w [T,K], topk_idx [T,K])."""
    E = gate_w.shape[0]
    inter = w2.shape[2]
    logits = tokens @ gate_w.t()
    top_v, top_i = torch.topk(logits, topk, dim=1, largest=True, sorted=True)
    top_w = torch.softmax(top_v.double(), dim=1).float()
    out = torch.zeros_like(tokens)
    for e in range(E):
        tok, slot = (top_i == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = tokens[tok] @ w13[e].t()
        act = torch.nn.functional.silu(h[:, :inter]) * h[:, inter:]
        out.index_add_(0, tok, (act @ w2[e].t()) * top_w[tok, slot].unsqueeze(1))
    return out, top_w, top_i.to(torch.int32)
