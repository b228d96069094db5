"""GPU (2+ devices): expert parallelism over NVLink, one process per rank.

Twin of the reference's multi-GPU test (test/multiGPU/cpp/moe/moeMultiGPUTests.cpp:80-91: ranks with
different token counts, one of them with zero tokens) and of its dispatch/return pattern test
(test/multiGPU/cpp/rocshmem/moeLikeCommPattern.cpp:257-351: every token leaves its rank).  Unlike the
reference product, rows really travel to the rank that owns the expert and the results come back."""
import os
import subprocess
import sys

import pytest
import torch

import moe_testlib as tl
from flash_distributed_moe_b200 import MoeKernelLauncher

pytestmark = pytest.mark.gpu

WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ep_worker.py")


def run_ranks(case, counts, timeout=600):
    world = len(counts)
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    uid = MoeKernelLauncher.getDistributedUniqueId().hex()  # created by the parent, as in the reference fixture
    procs = [subprocess.Popen([sys.executable, WORKER, str(r), str(world), uid, case] + [str(c) for c in counts],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timeout]"
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{out[-3000:]}"


def test_two_ranks_random_routing():
    run_ranks("tiny", [70, 33])


def test_two_ranks_one_without_tokens():
    run_ranks("tiny", [40, 0])


def test_two_ranks_every_row_remote():
    run_ranks("tiny_local", [2, 1])


def test_two_ranks_qwen3_30b_shape():
    run_ranks("qwen", [160, 96])


def test_two_ranks_qwen3_235b_sizes():
    # hidden 4096 / intermediate 1536 with 8 experts per rank
    run_ranks("q235", [150, 70])


def test_two_ranks_zipf_routing_buffers_exactly_full():
    # maxTokens equals each rank's token count: the hottest experts' buffers hold exactly one row per token
    run_ranks("qwen_zipf", [200, 184])


def test_four_ranks_uneven_tokens():
    run_ranks("tiny", [3, 50, 0, 129])


def test_four_ranks_qwen3_235b_sizes():
    run_ranks("q235", [64, 0, 200, 33])


def test_eight_ranks_qwen3_30b_shape():
    # every rank owns 16 of the 128 experts; uneven token counts, one rank without tokens
    run_ranks("qwen", [96, 17, 0, 130, 64, 1, 200, 33])
