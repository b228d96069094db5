"""GPU: the allocation-free entry point against the regular launcher.

FlashMoeLaunchNoAlloc exists for hosts that are not allowed to allocate device memory when the layer
runs (a serving engine with a frozen memory pool, code running under an allocator it must not
disturb): it takes all scratch from a fixed array inside the library.  Here it is called twice in a
row through the C ABI, the second time on different tokens, and each result must equal what
create/launch/destroy produce for the same inputs (the kernel is deterministic, so the comparison
is exact, which is well inside the bf16 tolerances the other tests use).  This file sorts last so
that a failure here cannot hide the other tests in a run that stops at the first failure."""
import ctypes as C

import numpy as np
import pytest
import torch

import moe_testlib as tl
from moe_testlib import synth
from flash_distributed_moe_b200 import _lib

pytestmark = pytest.mark.gpu


def _no_alloc(gate, w13, w2, x, shape):
    cfg = _lib.FlashMoeConfig(shape.hidden, shape.inter, shape.experts, shape.topk, 0, (C.c_int32 * 3)())
    out = torch.full_like(x, float("nan"))
    code = _lib.lib().FlashMoeLaunchNoAlloc(gate.data_ptr(), w13.data_ptr(), w2.data_ptr(), x.data_ptr(),
                                            out.data_ptr(), x.shape[0], C.byref(cfg),
                                            C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert code == 0, _lib.error_string(code)
    return out


def test_no_alloc_entry_point_matches_launcher_on_two_calls_in_a_row():
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, seed=4, std=0.05)
    layer = tl.GpuLayer(s, gate, w13, w2, max_tokens=300)
    try:
        xs = [synth.make_tokens(s, 300, seed=21), synth.make_tokens(s, 77, seed=22)]
        want = [layer.run(x) for x in xs]
        got = [_no_alloc(layer.gate, layer.w13, layer.w2, x.cuda(), s).cpu() for x in xs]
    finally:
        layer.close()
    for i, (g, w) in enumerate(zip(got, want)):
        assert torch.isfinite(g.float()).all(), f"call {i}"
        tl.assert_close_bf16(tl.f32(g), tl.f32(w), f"call {i} vs launcher")
        assert torch.equal(g, w), f"call {i}: deterministic kernel, results should be identical"


def test_no_alloc_rejects_what_does_not_fit():
    s = synth.QWEN3_30B_A3B  # 128 experts x 128-row minimum already exceed the fixed array
    cfg = _lib.FlashMoeConfig(s.hidden, s.inter, s.experts, s.topk, 0, (C.c_int32 * 3)())
    dummy = torch.zeros(16, device="cuda")
    code = _lib.lib().FlashMoeLaunchNoAlloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                            dummy.data_ptr(), 4096, C.byref(cfg), None)
    assert code == 1  # cudaErrorInvalidValue, before anything is dereferenced or launched
