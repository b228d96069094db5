"""Shared helpers of the parity tests: seeded inputs, the CPU oracle, and a thin driver around the
launcher that also pulls the stage buffers (routing, activations, weighted expert outputs)."""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import cpu_oracle  # noqa: E402
from flash_distributed_moe_b200 import synth  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden")

# north-star tolerances for bf16 outputs against the reference's own CPU MoE
MAX_ABS = 2e-2
REL_L2 = 1e-2


def f32(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.to(torch.float32).numpy())


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.int16).numpy().tobytes()).hexdigest()[:16]


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) /
                 max(np.linalg.norm(b.astype(np.float64)), 1e-30))


def assert_close_bf16(got: np.ndarray, ref: np.ndarray, what: str) -> None:
    """North-star bound for bf16 results: max-abs 2e-2 and rel-L2 1e-2.  bf16 keeps 8 significant bits, so
    one ulp of a value v is up to 2^-7 |v|; the result and the K staged per-slot rows it is summed from
    are all rounded to bf16, which for |v| > 2.56 alone exceeds 2e-2.  For such elements the absolute
    bound is widened to two bf16 ulps of the value (2^-6 |v|).  The synthetic N(0,0.02) layers of the benchmark never reach that size, so there the plain
    2e-2 bound is what is enforced; the widening matters only for the reference's U(-0.1,0.1) test stream."""
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    tol = np.maximum(MAX_ABS, np.abs(ref) * 2.0 ** -6)
    worst = float((err / tol).max()) if err.size else 0.0
    rl2 = rel_l2(got, ref)
    assert worst <= 1.0 and rl2 <= REL_L2, f"{what}: max-abs {err.max():.3e} ({worst:.2f}x tolerance), rel-L2 {rl2:.3e}"


def reference_stream_inputs(tokens: int, shape=synth.QWEN3_30B_A3B):
    """The reference tests' own inputs: one libc rand() stream seeded with 7907, tokens U(-1,1) then
    gate, FFN1 and FFN2 weights U(-0.1,0.1) (reference test/common/moeTools.h:45-69,
    test/common/utils.h:9,62-86), here rounded to bf16 because that is what the B200 path consumes."""
    p = cpu_oracle.PortOracle()
    H, I, E = shape.hidden, shape.inter, shape.experts
    x = p.rand_uniform(tokens * H, -1.0, 1.0, True).reshape(tokens, H)
    gate = p.rand_uniform(E * H, -0.1, 0.1, False).reshape(E, H)
    w13 = p.rand_uniform(E * H * I * 2, -0.1, 0.1, False).reshape(E, 2 * I, H)
    w2 = p.rand_uniform(E * H * I, -0.1, 0.1, False).reshape(E, H, I)
    to = lambda a: torch.from_numpy(a).to(torch.bfloat16)  # noqa: E731
    return to(x), to(gate), to(w13), to(w2)


def near_tie_mask(logits: np.ndarray, k: int, gap: float = 1e-6) -> np.ndarray:
    """True for tokens whose top-(k+1) logits contain an adjacent pair closer than `gap`."""
    top = -np.sort(-logits.astype(np.float64), axis=1)[:, :k + 1]
    return (np.abs(np.diff(top, axis=1)) < gap).any(axis=1)


class GpuLayer:
    """One launcher on cuda:0 with its weights; run() returns the output and the stage buffers."""

    def __init__(self, shape, gate, w13, w2, max_tokens, rank=0, world=1, uid=None, device="cuda:0"):
        from flash_distributed_moe_b200 import MoeKernelLauncher
        self.shape = shape
        self.dev = torch.device(device)
        self.gate = gate.to(self.dev)
        self.w13 = w13.to(self.dev)
        self.w2 = w2.to(self.dev)
        self.max_tokens = max_tokens
        self.launcher = MoeKernelLauncher()
        uid = uid if uid is not None else MoeKernelLauncher.getDistributedUniqueId(empty=True)
        self.launcher.create(self.gate, self.w13, self.w2, max_tokens, uid, rank, world, topk=shape.topk)
        info = np.frombuffer(self.launcher.debug_read(7, 16), np.int32)
        self.cap_rows, self.e_local, self.grid, self.smem = [int(v) for v in info]

    def run(self, x: torch.Tensor, inplace: bool = False) -> torch.Tensor:
        xd = x.to(self.dev)
        out = xd if inplace else torch.empty_like(xd)
        self.launcher.launch(xd, out)
        torch.cuda.synchronize(self.dev)
        code, info = self.launcher.last_status()
        assert code == 0, f"device-side error {code} info 0x{info:x}"
        return out.cpu()

    def stages(self, T: int) -> dict:
        s, L = self.shape, self.launcher
        K, H, I = s.topk, s.hidden, s.inter
        rows = self.e_local * self.cap_rows
        d = {}
        d["idx"] = np.frombuffer(L.debug_read(0, T * K * 4), np.int32).reshape(T, K).copy()
        d["w"] = np.frombuffer(L.debug_read(1, T * K * 4), np.float32).reshape(T, K).copy()
        d["cnt"] = np.frombuffer(L.debug_read(2, self.e_local * 4), np.uint32).copy()
        d["meta"] = np.frombuffer(L.debug_read(4, rows * 16), np.int32).reshape(rows, 4).copy()
        bf = lambda b, shp: torch.frombuffer(bytearray(b), dtype=torch.bfloat16).reshape(shp)  # noqa: E731
        d["packed"] = bf(L.debug_read(3, rows * H * 2), (rows, H))
        d["act"] = bf(L.debug_read(5, rows * I * 2), (rows, I))
        d["y"] = bf(L.debug_read(6, T * K * H * 2), (T, K, H))
        return d

    def close(self):
        self.launcher.destroy()
