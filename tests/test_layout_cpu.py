"""Host arithmetic of the scratch arena (csrc/host_layout.h) at the benchmark configurations, checked
by a small C++ program: region order and alignment, queue capacity against the tasks one launch can
publish, the limit of the dispatch word, totals against a B200's memory.  No GPU."""
import os
import subprocess

import moe_testlib as tl

CPP = os.path.join(tl.ROOT, "tests", "cpp", "layout_test.cpp")
BIN = os.path.join(tl.ROOT, "tests", "cpp", "layout_test.bin")
CSRC = os.path.join(tl.ROOT, "flash_distributed_moe_b200", "csrc")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def test_arena_layout_holds_at_the_benchmark_configurations():
    subprocess.run(["g++", "-std=c++17", "-O1", "-o", BIN, CPP, f"-I{CUDA}/include", f"-I{CSRC}"], check=True)
    r = subprocess.run([BIN], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all checks hold" in r.stdout and "cfg5 235B 8x16384: fits=1" in r.stdout
