"""GPU: vLLM with data parallelism and expert parallelism, with and without the patch that routes its
Qwen3-MoE block through the launcher (tests/vllm_dp_harness.py; twin of the reference's
test/multiGPU/python/benchmark_dp.py:412-435, which compares the token ids of both runs).  Skipped where
vLLM, or the patched engine, cannot be brought up (exit codes 77 and 78 of the harness); fails when both
runs finish and their token ids disagree (or, in the harness's verify mode, when the rows of the patched
block lie too far from vLLM's own block's on the same input)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HARNESS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "vllm_dp_harness.py")


def _run(dp, mode="tokens"):
    if os.environ.get("FLASHMOE_TEST_VLLM") != "1":
        pytest.skip("opt-in (FLASHMOE_TEST_VLLM=1): bringing vLLM engines up twice takes many minutes")
    if torch.cuda.device_count() < dp:
        pytest.skip(f"needs {dp} GPUs")
    r = subprocess.run([sys.executable, HARNESS, "--dp", str(dp), "--mode", mode], capture_output=True, text=True, timeout=1500)
    tail = (r.stdout[-1500:] + "\n" + r.stderr[-2500:])
    if r.returncode == 77:
        pytest.skip("vLLM could not run here: " + tail[-600:])
    if r.returncode == 78:
        pytest.skip("the patched vLLM engine did not come up here: " + tail[-900:])
    assert r.returncode == 0, tail


def test_single_rank_every_call_matches_vllm_block():
    # one engine, the patch's checking mode: vLLM's own block and the kernel on the same input, call by call
    _run(1, "verify")


def test_single_rank_token_ids_match_vllm():
    _run(1)


def test_two_ranks_dp_ep_token_ids_match_vllm():
    _run(2)
