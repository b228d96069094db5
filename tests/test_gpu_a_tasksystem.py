"""GPU: the device task system on its own (no tensor cores involved).

Twin of the reference's saxpy coherence test (test/singleGPU/cpp/taskSystem/
saxpyCoherenceTest.hip:43-143): every element goes through two dependent tasks, x*2 pushed from the
host, then +1 pushed by the first task through the global ticket queue; the result must be 2i+1."""
import ctypes as C

import numpy as np
import pytest
import torch

import moe_testlib as tl
from moe_testlib import synth
from flash_distributed_moe_b200 import _lib

pytestmark = pytest.mark.gpu


def test_two_stage_tasks_through_the_queue():
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, std=0.05)
    layer = tl.GpuLayer(s, gate, w13, w2, max_tokens=64)
    try:
        n = 262144  # as in the reference test
        for rep in range(2):  # twice: queue state carries over between launches
            data = torch.arange(n, dtype=torch.int32, device="cuda:0")
            code = _lib.lib().FlashMoeTestTaskSystem(layer.launcher._h, data.data_ptr(), n,
                                                     C.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert code == 0, _lib.error_string(code)
            torch.cuda.synchronize()
            assert layer.launcher.last_status() == (0, 0)
            got = data.cpu().numpy()
            want = 2 * np.arange(n, dtype=np.int32) + 1
            bad = np.nonzero(got != want)[0]
            assert bad.size == 0, f"rep {rep}: {bad.size} wrong, first at {bad[:5]}: {got[bad[:5]]}"
    finally:
        layer.close()
