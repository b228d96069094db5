"""GPU: the CTA-pair tensor-core primitive under the FFN tiles (tcgen05.mma.cta_group::2 fed by TMA
from both CTAs of a cluster) against a plain fp32 matrix product, for several token counts N (the
B operand, split half and half over the pair) and TMA box heights."""
import ctypes as C

import pytest
import torch

from flash_distributed_moe_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,K,box", [(256, 256, 128), (256, 2048, 16), (64, 512, 32), (16, 64, 8), (208, 768, 8)])
def test_pair_gemm_matches_fp32_product(N, K, box):
    g = torch.Generator().manual_seed(N * 7 + K)
    W = torch.randn(256, K, generator=g).to(torch.bfloat16).cuda()
    X = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    D = torch.full((256, N), float("nan"), dtype=torch.float32, device="cuda")
    code = _lib.lib().FlashMoeTestPairGemm(W.data_ptr(), X.data_ptr(), D.data_ptr(), N, K, box, None,
                                           C.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(code, "FlashMoeTestPairGemm")
    ref = W.float() @ X.float().T
    err = (D - ref).abs().max().item()
    assert err <= 1e-3 * max(1.0, ref.abs().max().item()), err
