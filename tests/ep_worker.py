"""One expert-parallel rank of the multi-GPU parity tests (run as a child process, one per GPU).

    python tests/ep_worker.py <rank> <world> <uid hex> <case> [tokens per rank ...]

Mirrors the reference's fork-per-rank fixture (test/multiGPU/cpp/moe/moeDistBaseTest.h:30-104): the
parent creates the unique id, every child pins its GPU, creates a launcher on its expert shard, runs
its own token slice and compares with its slice of the CPU result
(test/multiGPU/cpp/moe/moeMultiGPUTests.cpp:31-67).  Exit code 0 = parity holds.
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import moe_testlib as tl  # noqa: E402
from moe_testlib import cpu_oracle, synth  # noqa: E402


def main():
    # Ranks check their slices against the CPU oracle between launches and so reach the next (collective)
    # launch seconds apart, a rank without tokens at once: the library's own budget for peers to enter a
    # launch (FLASHMOE_PEER_TIMEOUT_MS, 60 s by default) covers that; the waits inside a launch keep theirs.
    rank, world = int(sys.argv[1]), int(sys.argv[2])
    uid = bytes.fromhex(sys.argv[3])
    case = sys.argv[4]
    counts = [int(v) for v in sys.argv[5:5 + world]]
    torch.cuda.set_device(rank)
    shape = (synth.TINY if case.startswith("tiny") else
             synth.QWEN3_235B_E16 if case.startswith("q235") else synth.QWEN3_30B_A3B)
    std = 0.05 if shape is synth.TINY else 0.02
    gate, w13, w2 = synth.make_weights(shape, seed=11, std=std)
    xs = [synth.make_tokens(shape, n, seed=100 + r) for r, n in enumerate(counts)]
    if case.endswith("zipf"):
        # the fourth benchmark configuration's routing: the most popular experts take a row from every
        # token of every rank, so their buffers on the owning rank are filled to exactly their capacity
        allx = torch.cat(xs)
        gate, allx, _ = synth.zipf_routing(shape, gate, allx)
        xs = list(torch.split(allx, counts))
    if case.endswith("local"):
        # the reference's forced routing (test/common/moeTools.h:187-207): token t is a one-hot at
        # column t and its K experts get gate weight 100 there, all inside one rank's shard
        gate = torch.zeros_like(gate)
        el = shape.experts // world
        col = 0
        for r, n in enumerate(counts):
            for t in range(n):
                xs[r][t] = 0
                xs[r][t, col] = 1.0
                first = ((r + 1) % world) * el  # experts of ANOTHER rank: every row crosses NVLink
                gate[first:first + shape.topk, col] = 100.0
                col += 1
    el = shape.experts // world
    layer = tl.GpuLayer(shape, gate, w13[rank * el:(rank + 1) * el].contiguous(),
                        w2[rank * el:(rank + 1) * el].contiguous(),
                        max_tokens=counts[rank] if case.endswith("zipf") else max(counts) + 2,
                        rank=rank, world=world, uid=uid, device=f"cuda:{rank}")
    port = cpu_oracle.PortOracle()
    ok = True
    for rep in range(3):  # several launches: epochs, counter reset and queue carry-over across ranks
        x = xs[rank]
        out = tl.f32(layer.run(x, inplace=(rep == 2)))
        if x.shape[0]:
            ref, rw, ri, _, _ = port.full_moe(tl.f32(x), tl.f32(gate), tl.f32(w13), tl.f32(w2), shape.topk,
                                              threads=4, stages=True)
            idx = np.frombuffer(layer.launcher.debug_read(0, x.shape[0] * shape.topk * 4), np.int32).reshape(ri.shape)
            if not np.array_equal(idx, ri):
                print(f"rank {rank} rep {rep}: top-k mismatch", flush=True)
                ok = False
            try:
                tl.assert_close_bf16(out, ref, f"rank {rank} rep {rep} output")
            except AssertionError as e:
                print(e, flush=True)
                ok = False
    layer.close()
    print(f"rank {rank}: {'ok' if ok else 'FAILED'}", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
