"""CPU, world size 2 over gloo: the host-side logic of the multi-GPU path that needs no device: the
unique id travels from rank 0 to the others (as the reference's vLLM patch does with
broadcast_object_list, test/multiGPU/python/flash_moe_patch.py:73-87), expert shards of the synthetic
weights equal the same experts of the unsharded weights, the benchmark's max-over-ranks reduction, and
the benchmark's parity check at N > 1 (all ranks' shards in one memory-mapped file, every rank against the
oracle on all experts)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import moe_testlib as tl
from moe_testlib import synth


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from flash_distributed_moe_b200 import MoeKernelLauncher
    box = [MoeKernelLauncher.getDistributedUniqueId() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    uid = box[0]
    s = synth.TINY
    el = s.experts // world
    gate, w13, w2 = synth.make_weights(s, seed=5, std=0.05, experts_slice=(rank * el, el))
    t = torch.tensor([1.0 + rank, 10.0 - rank])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    q.put((rank, uid, tl.sha(gate), tl.sha(w13), tl.sha(w2), t.tolist()))
    dist.barrier()
    dist.destroy_process_group()


def test_uid_broadcast_shards_and_max_reduction():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29400 + os.getpid() % 500
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, seed=5, std=0.05)
    el = s.experts // world
    assert got[0][1] == got[1][1] and len(got[0][1]) == 128 and got[0][1] != bytes(128)
    for rank, _, g_sha, w13_sha, w2_sha, red in got:
        assert g_sha == tl.sha(gate)
        assert w13_sha == tl.sha(w13[rank * el:(rank + 1) * el].contiguous())
        assert w2_sha == tl.sha(w2[rank * el:(rank + 1) * el].contiguous())
        assert red == [2.0, 10.0]


def _shared_weights_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, tl.ROOT)
    import bench
    from moe_testlib import cpu_oracle
    s = synth.TINY
    el = s.experts // world
    gate, w13, w2 = synth.make_weights(s, seed=5, std=0.05, experts_slice=(rank * el, el))
    shared = bench.SharedWeights(s, rank, world, w13, w2, dist.barrier)
    paths = list(shared.paths)
    x = synth.make_tokens(s, 24, seed=70 + rank)
    port_oracle = cpu_oracle.PortOracle()
    out, _, idx = port_oracle.full_moe_bf16_weights(tl.f32(x), tl.f32(gate), shared.maps[0], shared.maps[1], s.topk)
    shared.close(dist.barrier)
    dist.barrier()
    q.put((rank, out.tobytes(), idx.tobytes(), [os.path.exists(p) for p in paths]))
    dist.barrier()
    dist.destroy_process_group()


def test_benchmark_ranks_share_one_copy_of_all_expert_shards():
    # bench.py at N > 1: every rank writes the shard its GPU uses into one memory-mapped file and checks
    # its own tokens against the oracle on ALL experts; the result must be what the oracle gives on the
    # unsharded weights, and the files must be gone afterwards
    from moe_testlib import cpu_oracle
    cpu_oracle.build()
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + os.getpid() % 90
    procs = [ctx.Process(target=_shared_weights_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    import numpy as np
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, seed=5, std=0.05)
    port_oracle = cpu_oracle.PortOracle()
    for rank, out_b, idx_b, exists in got:
        x = synth.make_tokens(s, 24, seed=70 + rank)
        ref, _, ref_idx, _, _ = port_oracle.full_moe(tl.f32(x), tl.f32(gate), tl.f32(w13), tl.f32(w2), s.topk, stages=True)
        assert np.frombuffer(out_b, np.float32).reshape(ref.shape).tobytes() == ref.tobytes()
        assert np.frombuffer(idx_b, np.int32).reshape(ref_idx.shape).tobytes() == ref_idx.tobytes()
        assert exists == [False, False]
