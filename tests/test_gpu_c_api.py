"""GPU: life cycle and edge cases through the launcher interface (twin of the reference's
test/singleGPU/python/test_pythonBinding.py:5-40 and test_flashMoeOp.py:12-76)."""
import numpy as np
import pytest
import torch

import moe_testlib as tl
from moe_testlib import cpu_oracle, synth
from flash_distributed_moe_b200 import FlashMoeBlockWrapper, MoeKernelLauncher

pytestmark = pytest.mark.gpu


def test_python_binding_life_cycle():
    s = synth.TINY
    gate, w13, w2 = [t.cuda() for t in synth.make_weights(s, std=0.05)]
    tokens = synth.make_tokens(s, 16).cuda()
    output = torch.empty_like(tokens)
    launcher = MoeKernelLauncher()
    assert launcher.valid is False
    uid = launcher.getDistributedUniqueId(empty=True)
    launcher.create(gate, w13, w2, 16, uid, 0, 1, topk=s.topk)
    assert launcher.valid is True
    launcher.launch(tokens, output)
    torch.cuda.synchronize()
    assert output.shape == (16, s.hidden) and output.dtype == torch.bfloat16
    assert launcher.last_status() == (0, 0)
    with pytest.raises(RuntimeError):
        launcher.launch(torch.zeros(17, s.hidden, dtype=torch.bfloat16, device="cuda"),
                        torch.zeros(17, s.hidden, dtype=torch.bfloat16, device="cuda"))  # > maxTokens
    launcher.destroy()
    assert launcher.valid is False
    with pytest.raises(RuntimeError):
        launcher.launch(tokens, output)


def test_zero_tokens_and_repeated_launches():
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, std=0.05)
    port = cpu_oracle.PortOracle()
    layer = tl.GpuLayer(s, gate, w13, w2, max_tokens=96)
    try:
        empty = torch.empty(0, s.hidden, dtype=torch.bfloat16)
        assert layer.run(empty).shape == (0, s.hidden)
        for T, seed in ((1, 5), (96, 6), (33, 7), (0, 0), (64, 8)):
            x = synth.make_tokens(s, T, seed=seed)
            out = tl.f32(layer.run(x))
            if T == 0:
                continue
            ref = port.full_moe(tl.f32(x), tl.f32(gate), tl.f32(w13), tl.f32(w2), s.topk)
            assert np.abs(out - ref).max() <= tl.MAX_ABS and tl.rel_l2(out, ref) <= tl.REL_L2, (T, seed)
    finally:
        layer.close()


def test_host_buffer_entry_point_matches_device_entry_point():
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, std=0.05)
    layer = tl.GpuLayer(s, gate, w13, w2, max_tokens=64)
    try:
        x = synth.make_tokens(s, 50, seed=9)
        dev = layer.run(x)
        xin = x.clone().pin_memory()
        out = torch.empty_like(xin).pin_memory()
        layer.launcher.launch_host(xin, out)
        torch.cuda.synchronize()
        assert torch.equal(out, dev)
    finally:
        layer.close()


def test_host_entry_point_pipelines_back_to_back_calls():
    # calls made back to back overlap the copies of one with the kernel of the other (two sets of
    # staging buffers on internal streams); device-pointer launches in between share the scratch
    # arena and must stay ordered with them
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, std=0.05)
    layer = tl.GpuLayer(s, gate, w13, w2, max_tokens=64)
    try:
        xs = [synth.make_tokens(s, T, seed=20 + i) for i, T in enumerate((64, 17, 0, 50, 64, 33))]
        want = [layer.run(x).cpu() for x in xs]
        ins = [x.clone().pin_memory() for x in xs]
        outs = [torch.empty_like(x).pin_memory() for x in ins]
        dev_x = xs[3].cuda()
        dev_out = torch.empty_like(dev_x)
        for i, (xin, out) in enumerate(zip(ins, outs)):
            layer.launcher.launch_host(xin, out)
            if i == 2:
                layer.launcher.launch(dev_x, dev_out)  # a direct launch in the middle of the pipeline
        torch.cuda.synchronize()
        for i, (out, ref) in enumerate(zip(outs, want)):
            assert torch.equal(out, ref), i
        assert torch.equal(dev_out.cpu(), want[3])
    finally:
        layer.close()


def test_fp32_io_adapter():
    # the reference interface is fp32; weights are converted once, tokens/output cast at the boundary
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, std=0.05)
    x = synth.make_tokens(s, 24, seed=3)
    port = cpu_oracle.PortOracle()
    ref = port.full_moe(tl.f32(x), tl.f32(gate), tl.f32(w13), tl.f32(w2), s.topk)
    l = MoeKernelLauncher()
    g32, a32, b32 = gate.float().cuda(), w13.float().cuda(), w2.float().cuda()
    l.create(g32, a32, b32, 24, l.getDistributedUniqueId(empty=True), 0, 1, topk=s.topk)
    xin = x.float().cuda()
    out = torch.empty_like(xin)
    l.launch(xin, out)
    torch.cuda.synchronize()
    l.destroy()
    o = out.cpu().numpy()
    assert out.dtype == torch.float32
    assert np.abs(o - ref).max() <= tl.MAX_ABS and tl.rel_l2(o, ref) <= tl.REL_L2


class _Experts(torch.nn.Module):
    def __init__(self, w13, w2):
        super().__init__()
        self.w13_weight = torch.nn.Parameter(w13, requires_grad=False)
        self.w2_weight = torch.nn.Parameter(w2, requires_grad=False)


class _Block(torch.nn.Module):
    """Stand-in with the attribute layout of vLLM's Qwen3MoeSparseMoeBlock."""

    def __init__(self, gate, w13, w2):
        super().__init__()
        self.gate = torch.nn.Linear(gate.shape[1], gate.shape[0], bias=False, dtype=gate.dtype, device=gate.device)
        self.gate.weight = torch.nn.Parameter(gate, requires_grad=False)
        self.experts = _Experts(w13, w2)


def test_block_wrapper_in_place():
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, std=0.05)
    port = cpu_oracle.PortOracle()
    wrapper = FlashMoeBlockWrapper(_Block(gate.cuda(), w13.cuda(), w2.cuda()), maxTokens=48, topk=s.topk)
    for batch in (1, 16, 48):  # batch sizes of the reference's wrapper test
        x = synth.make_tokens(s, batch, seed=batch)
        hidden = x.cuda()
        got = wrapper(hidden)
        torch.cuda.synchronize()
        assert got.data_ptr() == hidden.data_ptr()
        ref = port.full_moe(tl.f32(x), tl.f32(gate), tl.f32(w13), tl.f32(w2), s.topk)
        o = tl.f32(got.cpu())
        assert np.abs(o - ref).max() <= tl.MAX_ABS and tl.rel_l2(o, ref) <= tl.REL_L2
    wrapper.launcher.destroy()


def test_single_gpu_launch_replays_from_a_cuda_graph():
    # On one GPU a launch is a memset and a kernel launch on the caller's stream, so it can be captured
    # into a CUDA graph (the reference's launch cannot: its micro-benchmark says so,
    # test/singleGPU/python/qwen3MoeMicroBenchmark.py:84); the replay reads whatever the captured
    # token buffer holds at that time.
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, std=0.05)
    port = cpu_oracle.PortOracle()
    g, a, b = gate.cuda(), w13.cuda(), w2.cuda()
    launcher = MoeKernelLauncher()
    launcher.create(g, a, b, 64, launcher.getDistributedUniqueId(empty=True), 0, 1, topk=s.topk)
    try:
        x_dev = synth.make_tokens(s, 48, seed=60).cuda()
        out_dev = torch.empty_like(x_dev)
        launcher.launch(x_dev, out_dev)  # first launch outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            launcher.launch(x_dev, out_dev)
        for seed in (61, 62, 63):
            x = synth.make_tokens(s, 48, seed=seed)
            x_dev.copy_(x)
            out_dev.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert launcher.last_status() == (0, 0)
            ref = port.full_moe(tl.f32(x), tl.f32(gate), tl.f32(w13), tl.f32(w2), s.topk)
            tl.assert_close_bf16(tl.f32(out_dev.cpu()), ref, f"graph replay, seed {seed}")
        del graph
    finally:
        torch.cuda.synchronize()
        launcher.destroy()
