"""A C++ program that binds the reference-shaped entry points the way the reference's own callers do
(test/singleGPU/cpp/moe/moeTest.cpp:28-70, moeApiTest.cpp:5-12): `GetDistributedUniqueId` returning a
struct by value, `CreateLauncher` taking the id by C++ reference, `Launch` through the vtable,
`DestroyLauncher`.  `CreateLauncher` means what it means in the reference: the Qwen3-30B-A3B layer with
fp32 tensors.  The error paths need no GPU; the run is checked against the CPU oracle."""
import os
import subprocess

import numpy as np
import pytest

import moe_testlib as tl
from moe_testlib import cpu_oracle
from flash_distributed_moe_b200 import _lib, build as build_mod

CPP = os.path.join(tl.ROOT, "tests", "cpp", "launcher_api_test.cpp")
BIN = os.path.join(tl.ROOT, "tests", "cpp", "launcher_api_test.bin")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


@pytest.fixture(scope="module")
def binary():
    build_mod.build()
    pkg = os.path.dirname(_lib.LIB_PATH)
    subprocess.run(["g++", "-std=c++17", "-O1", "-o", BIN, CPP, f"-I{CUDA}/include", f"-L{pkg}", "-l:libflashMoe.so",
                    f"-L{CUDA}/lib64", "-lcudart", f"-Wl,-rpath,{pkg}", f"-Wl,-rpath,{CUDA}/lib64"], check=True)
    return BIN


def test_create_time_error_paths_from_cpp(binary):
    r = subprocess.run([binary, "errors"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


def _tensor(n, salt, scale):
    i = np.arange(n, dtype=np.uint64).astype(np.uint32)
    u = i * np.uint32(2654435761) + np.uint32(salt)
    u ^= u >> np.uint32(15)
    u *= np.uint32(2246822519)
    u ^= u >> np.uint32(13)
    return ((u >> np.uint32(24)).astype(np.float32) - np.float32(128.0)) / np.float32(128.0) * np.float32(scale)


@pytest.mark.gpu
def test_create_launch_destroy_from_cpp_matches_the_oracle(binary, tmp_path):
    tokens, E, H, I, K = 24, 128, 2048, 768, 8
    out_file = str(tmp_path / "out.f32")
    r = subprocess.run([binary, "run", str(tokens), out_file], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    got = np.fromfile(out_file, np.float32).reshape(tokens, H)
    gate = _tensor(E * H, 1, 0.03125).reshape(E, H)
    w13 = _tensor(E * 2 * I * H, 2, 0.03125).reshape(E, 2 * I, H)
    w2 = _tensor(E * H * I, 3, 0.03125).reshape(E, H, I)
    x = _tensor(tokens * H, 4, 2.0).reshape(tokens, H)
    port = cpu_oracle.PortOracle()
    ref = port.full_moe(x, gate, w13, w2, K, threads=port.max_threads())
    tl.assert_close_bf16(got, ref, "C++ CreateLauncher/Launch output")
