"""B200-native FlashDMoE layer behind the reference launcher interface.

`flashMoeLauncher.MoeKernelLauncher` mirrors the reference's torch extension class
(python/pyMoeLauncherTorch.cpp:115-133 in the reference project); `flashMoeOp.FlashMoeBlockWrapper`
mirrors its vLLM wrapper (test/singleGPU/python/flashMoeOp.py:7-38).  All compute runs in
libflashMoe.so (CUDA, sm_100a); there is no CPU or PyTorch fallback.
"""
from . import flashMoeLauncher  # noqa: F401
from .flashMoeLauncher import MoeKernelLauncher  # noqa: F401
from .flashMoeOp import FlashMoeBlockWrapper  # noqa: F401

__all__ = ["MoeKernelLauncher", "FlashMoeBlockWrapper", "flashMoeLauncher"]
