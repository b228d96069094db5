"""Host-side checks that need no GPU: the C-ABI library loads and exports what the headers declare,
unique ids, and the create-time error paths (which by contract run before any CUDA call)."""
import ctypes as C
import os
import re

import pytest

import moe_testlib as tl  # noqa: F401  (sets sys.path)
from flash_distributed_moe_b200 import _lib, build as build_mod
from flash_distributed_moe_b200.flashMoeLauncher import MoeKernelLauncher

CUDA_ERROR_INVALID_VALUE = 1
CUDA_ERROR_UNKNOWN = 999


@pytest.fixture(scope="module")
def lib():
    build_mod.build()
    return _lib.lib()


def test_library_exports_every_declared_symbol(lib):
    inc = os.path.join(tl.ROOT, "include")
    declared = set()
    for name in os.listdir(inc):
        text = open(os.path.join(inc, name)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        declared |= set(re.findall(r"\b((?:FlashMoe|CreateLauncher|DestroyLauncher|GetDistributedUniqueId)\w*)\s*\(", text))
    declared -= {"FlashMoeHandle"}
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    for sym in declared:
        assert hasattr(lib, sym), sym


def test_only_the_interface_is_exported():
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    names = {line.split()[-1].split("@")[0] for line in out.splitlines() if " T " in line}
    assert names == set(_lib.EXPORTED_SYMBOLS)


def test_unique_id():
    empty = MoeKernelLauncher.getDistributedUniqueId(empty=True)
    assert empty == bytes(128)
    a = MoeKernelLauncher.getDistributedUniqueId()
    b = MoeKernelLauncher.getDistributedUniqueId()
    assert len(a) == 128 and a != bytes(128) and a != b


def _create(lib, cfg, max_tokens, weights=(None, None, None), rank=0, world=1):
    h = C.c_void_p(None)
    uid = (C.c_uint8 * 128)()
    code = lib.FlashMoeCreate(C.byref(h), weights[0], weights[1], weights[2], max_tokens, None, uid, rank, world,
                              C.byref(cfg) if cfg is not None else None)
    return code, h


def test_create_rejects_null_weights_like_the_reference_api_test(lib):
    # reference test/singleGPU/cpp/moe/moeApiTest.cpp:5-12: CreateLauncher(nullptr weights, 1024 tokens)
    # must fail with the "unknown" error code and leave the launcher pointer untouched.
    code, h = _create(lib, None, 1024)
    assert code == CUDA_ERROR_UNKNOWN and not h.value


def test_create_rejects_over_capacity(lib, monkeypatch):
    monkeypatch.setenv("FLASHMOE_MAX_SCRATCH_GB", "1")
    code, h = _create(lib, None, 1 << 20)
    assert code == CUDA_ERROR_UNKNOWN and not h.value


@pytest.mark.parametrize("cfg", [
    (2048 + 64, 768, 128, 8, 0),  # hidden not a multiple of 256
    (2048, 700, 128, 8, 0),       # intermediate not a multiple of 128
    (2048, 768, 256, 8, 0),       # too many experts
    (2048, 768, 128, 9, 0),       # top-k too large
    (2048, 768, 128, 8, 7),       # unknown dtype
])
def test_create_rejects_unsupported_shapes(lib, cfg):
    c = _lib.FlashMoeConfig(*cfg, (C.c_int32 * 3)())
    code, h = _create(lib, c, 16)
    assert code == CUDA_ERROR_INVALID_VALUE and not h.value


def test_create_rejects_bad_rank(lib):
    assert _create(lib, None, 16, rank=2, world=2)[0] == CUDA_ERROR_INVALID_VALUE
    assert _create(lib, None, 16, rank=0, world=9)[0] == CUDA_ERROR_INVALID_VALUE
    c = _lib.FlashMoeConfig(2048, 768, 128, 8, 0, (C.c_int32 * 3)())
    assert _create(lib, c, 16, rank=0, world=3)[0] == CUDA_ERROR_INVALID_VALUE  # 128 % 3 != 0


def test_launch_on_destroyed_launcher_raises():
    import torch
    l = MoeKernelLauncher()
    assert l.valid is False
    with pytest.raises(RuntimeError):
        l.launch(torch.zeros(1, 2048), torch.zeros(1, 2048))
    l.destroy()  # no-op on an empty launcher, as in the reference binding
