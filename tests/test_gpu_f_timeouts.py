"""GPU: device-side waits that run out.  Every wait in the kernel is bounded; when one runs out the
kernel records a status code, all of its roles leave normally and the host reads the code without a
fault, a trap or a hang.  The launcher then refuses further launches until it is destroyed and created
again.  (The reference's device waits are unbounded, src/hip/taskSystem/taskManager.h:208-215; its
communication test delays one rank by two seconds on purpose,
test/multiGPU/cpp/rocshmem/moeLikeCommPattern.cpp:318-326, which the peer-arrival budget covers.)"""
import ctypes as C
import os
import subprocess
import sys

import pytest
import torch

import moe_testlib as tl
from moe_testlib import synth
from flash_distributed_moe_b200 import MoeKernelLauncher, _lib

pytestmark = pytest.mark.gpu

FDMOE_ERR_TIMEOUT_QUEUE = 1
FDMOE_ERR_TIMEOUT_PEER = 5
WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "timeout_worker.py")


def test_queue_wait_runs_out_and_the_launcher_recovers_after_recreation(monkeypatch):
    monkeypatch.setenv("FLASHMOE_TIMEOUT_MS", "50")
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, std=0.05)
    layer = tl.GpuLayer(s, gate, w13, w2, max_tokens=32)
    try:
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert _lib.lib().FlashMoeTestStall(layer.launcher._h, stream) == 0  # the launch itself succeeds
        torch.cuda.synchronize()  # the kernel returned: no hang, the context is alive
        code, _ = layer.launcher.last_status()
        assert code == FDMOE_ERR_TIMEOUT_QUEUE
        x = synth.make_tokens(s, 8).cuda()
        with pytest.raises(RuntimeError):  # refused: cudaErrorUnknown
            layer.launcher.launch(x, torch.empty_like(x))
    finally:
        layer.close()
    monkeypatch.delenv("FLASHMOE_TIMEOUT_MS")
    # destroy + create again: back to normal
    layer = tl.GpuLayer(s, gate, w13, w2, max_tokens=32)
    try:
        x = synth.make_tokens(s, 8, seed=3)
        out = layer.run(x)
        assert torch.isfinite(out.float()).all()
        assert layer.launcher.last_status() == (0, 0)
    finally:
        layer.close()


def test_peer_that_never_launches_times_out_on_the_waiting_rank():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    uid = MoeKernelLauncher.getDistributedUniqueId().hex()
    env = dict(os.environ, FLASHMOE_PEER_TIMEOUT_MS="300", NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, WORKER, str(r), "2", uid], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timeout]"
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r}:\n{out[-2000:]}"
    assert f"status {FDMOE_ERR_TIMEOUT_PEER}" in outs[0]
