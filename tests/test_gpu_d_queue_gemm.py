"""GPU: tile GEMM driven through the task queue against the CPU GEMM (twin of the reference's
test/singleGPU/cpp/taskSystem/gemmTest/gemmTest.cpp:69-73), on the tcgen05 FFN2 tile path with unit
routing weights, ragged row counts per expert."""
import ctypes as C

import numpy as np
import pytest
import torch

import moe_testlib as tl
from moe_testlib import cpu_oracle, synth
from flash_distributed_moe_b200 import _lib

pytestmark = pytest.mark.gpu


def test_queue_gemm_matches_cpu():
    s = synth.LayerShape("gemm", 512, 256, 8, 2)
    gate, w13, w2 = synth.make_weights(s, seed=2, std=0.05)
    rows = np.array([128, 1, 0, 130, 77, 256, 5, 127], np.uint32)
    total = int(rows.sum())
    g = torch.Generator().manual_seed(11)
    A = torch.randn(total, s.inter, generator=g).to(torch.bfloat16)
    layer = tl.GpuLayer(s, gate, w13, w2, max_tokens=256)
    try:
        Ad = A.cuda()
        out = torch.zeros(total, s.hidden, dtype=torch.bfloat16, device="cuda")
        code = _lib.lib().FlashMoeTestQueueGemm(layer.launcher._h, rows.ctypes.data_as(C.POINTER(C.c_uint32)),
                                                Ad.data_ptr(), out.data_ptr(),
                                                C.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert code == 0, _lib.error_string(code)
        torch.cuda.synchronize()
        assert layer.launcher.last_status() == (0, 0)
    finally:
        layer.close()
    port = cpu_oracle.PortOracle()
    got = tl.f32(out.cpu())
    r0 = 0
    for e, n in enumerate(rows):
        n = int(n)
        if n == 0:
            continue
        ref = port.gemm_nt(tl.f32(A[r0:r0 + n]), tl.f32(w2[e]))
        err = np.abs(got[r0:r0 + n] - ref).max()
        assert err <= 2e-2 and tl.rel_l2(got[r0:r0 + n], ref) <= 1e-2, f"expert {e}: max-abs {err}"
        r0 += n
