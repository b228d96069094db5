"""One rank of the peer-arrival time-out test (child process, one per GPU).

    python tests/timeout_worker.py <rank> <world> <uid hex>

Both ranks create a launcher on the tiny layer.  Rank 0 launches; rank 1 never does.  Rank 0's kernel
gives up waiting for its peer after FLASHMOE_PEER_TIMEOUT_MS, records FDMOE_ERR_TIMEOUT_PEER and
returns; the next launch is refused.  Then both ranks destroy their launchers (a collective step that
needs no kernel) and exit 0.  No kernel of rank 1 is ever in flight, nothing faults."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import moe_testlib as tl  # noqa: E402
from moe_testlib import synth  # noqa: E402


def main():
    rank, world = int(sys.argv[1]), int(sys.argv[2])
    uid = bytes.fromhex(sys.argv[3])
    torch.cuda.set_device(rank)
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, seed=5, std=0.05)
    el = s.experts // world
    layer = tl.GpuLayer(s, gate, w13[rank * el:(rank + 1) * el].contiguous(), w2[rank * el:(rank + 1) * el].contiguous(),
                        max_tokens=16, rank=rank, world=world, uid=uid, device=f"cuda:{rank}")
    ok = True
    if rank == 0:
        x = synth.make_tokens(s, 16, seed=1).to(layer.dev)
        out = torch.empty_like(x)
        layer.launcher.launch(x, out)
        torch.cuda.synchronize(layer.dev)  # returns after the peer budget: no hang
        code, info = layer.launcher.last_status()
        print(f"rank 0: status {code} info {info}", flush=True)
        ok = code == 5
        try:
            layer.launcher.launch(x, out)
            ok = False  # must be refused
        except RuntimeError:
            pass
    layer.close()
    print(f"rank {rank}: {'ok' if ok else 'FAILED'}", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
