"""ctypes binding of libflashMoe.so (the flat C ABI of include/flashmoe_c.h).

The library is the product; if it is missing this module raises at import of the first symbol
rather than falling back to anything else.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflashMoe.so")

# Every symbol include/iMoeKernelLauncher.h and include/flashmoe_c.h declare.
EXPORTED_SYMBOLS = [
    "GetDistributedUniqueId", "CreateLauncher", "CreateLauncherEx", "DestroyLauncher",
    "FlashMoeGetUniqueId", "FlashMoeCreate", "FlashMoeLaunch", "FlashMoeLaunchHost",
    "FlashMoeDestroy", "FlashMoeGetLastStatus", "FlashMoeDebugRead", "FlashMoeTestTaskSystem",
    "FlashMoeTestQueueGemm", "FlashMoeTestStall", "FlashMoeErrorString", "FlashMoeLaunchNoAlloc",
]


class FlashMoeConfig(C.Structure):
    _fields_ = [("hiddenSize", C.c_int32), ("expertIntermediateSize", C.c_int32),
                ("expertsNum", C.c_int32), ("topk", C.c_int32), ("dtype", C.c_int32),
                ("reserved", C.c_int32 * 3)]


_lib = None


def lib() -> C.CDLL:
    """Loads the library once.  Raises if it has not been built (python -m flash_distributed_moe_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m flash_distributed_moe_b200.build`. "
            "There is no fallback path.")
    L = C.CDLL(LIB_PATH)
    vp = C.c_void_p
    L.FlashMoeGetUniqueId.argtypes = [C.c_int, C.POINTER(C.c_uint8)]
    L.FlashMoeCreate.argtypes = [C.POINTER(vp), vp, vp, vp, C.c_int, vp, C.POINTER(C.c_uint8), C.c_int,
                                 C.c_int, C.POINTER(FlashMoeConfig)]
    L.FlashMoeLaunch.argtypes = [vp, vp, vp, C.c_int, vp]
    L.FlashMoeLaunchHost.argtypes = [vp, vp, vp, C.c_int, vp]
    L.FlashMoeDestroy.argtypes = [vp, vp]
    L.FlashMoeGetLastStatus.argtypes = [vp, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
    L.FlashMoeDebugRead.argtypes = [vp, C.c_int, vp, C.c_size_t, C.c_size_t]
    L.FlashMoeTestTaskSystem.argtypes = [vp, vp, C.c_int, vp]
    L.FlashMoeTestQueueGemm.argtypes = [vp, C.POINTER(C.c_uint32), vp, vp, vp]
    L.FlashMoeTestStall.argtypes = [vp, vp]
    L.FlashMoeTestStall.restype = C.c_int
    L.FlashMoeLaunchNoAlloc.argtypes = [vp, vp, vp, vp, vp, C.c_int, C.POINTER(FlashMoeConfig), vp]
    L.FlashMoeLaunchNoAlloc.restype = C.c_int
    L.FlashMoeErrorString.argtypes = [C.c_int]
    L.FlashMoeErrorString.restype = C.c_char_p
    for fn in ("FlashMoeGetUniqueId", "FlashMoeCreate", "FlashMoeLaunch", "FlashMoeLaunchHost",
               "FlashMoeDestroy", "FlashMoeGetLastStatus", "FlashMoeDebugRead",
               "FlashMoeTestTaskSystem", "FlashMoeTestQueueGemm"):
        getattr(L, fn).restype = C.c_int
    _lib = L
    return L


def error_string(code: int) -> str:
    return lib().FlashMoeErrorString(int(code)).decode()


def check(code: int, what: str) -> None:
    """Non-zero return codes become exceptions, as the reference binding does with TORCH_CHECK
    (python/pyMoeLauncherTorch.cpp:14-22)."""
    if code != 0:
        raise RuntimeError(f"{what} failed: CUDA error {code} ({error_string(code)})")
