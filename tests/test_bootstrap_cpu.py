"""CPU: the host-side rendezvous of the multi-rank launcher (TCP star around rank 0, addressed by the
unique id) with forked ranks, including the failure paths: a rank that never joins (time-out error
instead of a hang), ranks that disagree about the world size, an empty id."""
import os
import subprocess

import pytest

import moe_testlib as tl

CSRC = os.path.join(tl.ROOT, "flash_distributed_moe_b200", "csrc")
BIN = os.path.join(tl.ROOT, "tests", "cpp", "bootstrap_test.bin")


@pytest.fixture(scope="module")
def binary():
    subprocess.run(["g++", "-std=c++17", "-O1", "-o", BIN, os.path.join(tl.ROOT, "tests", "cpp", "bootstrap_test.cpp"),
                    os.path.join(CSRC, "bootstrap.cpp")], check=True)
    return BIN


@pytest.mark.parametrize("world", [2, 4, 8])
def test_all_ranks_join(binary, world):
    assert subprocess.run([binary, "ok", str(world)], timeout=60).returncode == 0


def test_missing_rank_times_out_on_every_rank(binary):
    assert subprocess.run([binary, "missing", "3"], timeout=60).returncode == 0


def test_world_size_mismatch_is_refused(binary):
    assert subprocess.run([binary, "mismatch"], timeout=60).returncode == 0


def test_empty_id_is_rejected_for_multi_rank(binary):
    assert subprocess.run([binary, "empty"], timeout=60).returncode == 0
