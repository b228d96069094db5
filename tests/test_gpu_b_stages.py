"""GPU parity, stage by stage, from one full launch per case: gate (top-k indices exact, weights),
routing/pack (row counts, sideband, payload), FFN1 activations, FFN2 weighted rows, final output.

Twins of the reference's stage tests (test/singleGPU/cpp/moe/internal/moeGateTest.hip:62-109,
moeRoutingTest.hip:286-353, moeExpertFFN1Test.hip:58-106, moeExpertsTests.hip:389-475) and of its
integration test (test/singleGPU/cpp/moe/moeTest.cpp:28-70).  Everything is checked against the CPU
oracle on the same bf16-rounded inputs; bf16 tolerances are the north-star ones (max-abs 2e-2,
rel-L2 1e-2)."""
import os

import numpy as np
import pytest
import torch

import moe_testlib as tl
from moe_testlib import cpu_oracle, synth

pytestmark = pytest.mark.gpu


def check_routing_and_output(shape, x, gate, w13, w2, max_tokens):
    """Top-k indices (exact, in order), routing weights and the output of one launch against the oracle,
    without pulling the row buffers: for token counts whose stage buffers run to gigabytes."""
    port = cpu_oracle.PortOracle()
    T, K = x.shape[0], shape.topk
    o_out, o_w, o_idx, _, _ = port.full_moe(tl.f32(x), tl.f32(gate), tl.f32(w13), tl.f32(w2), K,
                                            threads=port.max_threads(), stages=True)
    layer = tl.GpuLayer(shape, gate, w13, w2, max_tokens)
    try:
        out = tl.f32(layer.run(x))
        idx = np.frombuffer(layer.launcher.debug_read(0, T * K * 4), np.int32).reshape(T, K)
        w = np.frombuffer(layer.launcher.debug_read(1, T * K * 4), np.float32).reshape(T, K)
        cnt = np.frombuffer(layer.launcher.debug_read(2, layer.e_local * 4), np.uint32)
    finally:
        layer.close()
    assert np.array_equal(idx, o_idx), f"top-k mismatch on {(idx != o_idx).any(1).sum()} tokens"
    assert np.abs(w - o_w).max() <= 1e-5
    assert np.array_equal(cnt, np.bincount(o_idx.ravel(), minlength=shape.experts))
    tl.assert_close_bf16(out, o_out, "layer output")


def check_layer(shape, x, gate, w13, w2, max_tokens, golden=None, inplace=False, check_stages=True):
    port = cpu_oracle.PortOracle()
    T = x.shape[0]
    K, H, I = shape.topk, shape.hidden, shape.inter
    xf, gf, w13f, w2f = tl.f32(x), tl.f32(gate), tl.f32(w13), tl.f32(w2)
    o_out, o_w, o_idx, o_act, o_y = port.full_moe(xf, gf, w13f, w2f, K, threads=port.max_threads(), stages=True)
    if golden is not None:
        g = np.load(os.path.join(tl.GOLDEN, golden))
        assert np.array_equal(o_idx, g["topk_idx"]) and np.array_equal(o_out, g["out"])

    layer = tl.GpuLayer(shape, gate, w13, w2, max_tokens)
    try:
        out = tl.f32(layer.run(x, inplace=inplace))
        st = layer.stages(T) if check_stages else None
    finally:
        layer.close()

    if check_stages:
        # --- gate: indices bit-exact, in the reference's order, with no near-tie exclusion (nearly tied
        # tokens are recomputed in the reference's fp32 order on the device); weights to 1e-5, the
        # tolerance of the reference's own gate test (test/common/utils.h:27, moeGateTest.hip:62-109)
        assert np.array_equal(st["idx"], o_idx), f"top-k mismatch on {(st['idx'] != o_idx).any(1).sum()} tokens"
        assert np.abs(st["w"] - o_w).max() <= 1e-5
        # --- routing: per-expert row counts and the (token, slot) set of each expert
        cap = layer.cap_rows
        for e in range(shape.experts):
            want = {(t, k) for t, k in zip(*np.nonzero(o_idx == e))}
            assert st["cnt"][e] == len(want), f"expert {e}: {st['cnt'][e]} rows, expected {len(want)}"
            m = st["meta"][e * cap:e * cap + len(want)]
            got = {(int(t), int(hs) & 0xff) for t, hs in zip(m[:, 0], m[:, 1])}
            assert got == want, f"expert {e}: wrong (token, slot) set"
        # --- per-row checks on every packed row
        act_got, act_ref = [], []
        for e in range(shape.experts):
            n = int(st["cnt"][e])
            if n == 0:
                continue
            m = st["meta"][e * cap:e * cap + n]
            toks, slots = m[:, 0], m[:, 1] & 0xff
            wts = m[:, 2].copy().view(np.float32)
            assert torch.equal(st["packed"][e * cap:e * cap + n], x[torch.from_numpy(toks.astype(np.int64))])
            assert np.abs(wts - o_w[toks, slots]).max() <= 1e-5
            act_got.append(tl.f32(st["act"][e * cap:e * cap + n]))
            act_ref.append(o_act[toks, slots])
        tl.assert_close_bf16(np.concatenate(act_got), np.concatenate(act_ref), "FFN1 activations")
        tl.assert_close_bf16(tl.f32(st["y"]), o_y * o_w[:, :, None], "FFN2 weighted rows")

    assert np.isfinite(out).all()
    tl.assert_close_bf16(out, o_out, "layer output")
    max_abs, rl2 = float(np.abs(out - o_out).max()), tl.rel_l2(out, o_out)
    return max_abs, rl2


def test_tiny_layer_ragged_tokens():
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, seed=0, std=0.05)
    check_layer(s, synth.make_tokens(s, 40, seed=0), gate, w13, w2, max_tokens=48, golden="tiny_t40.npz")


def test_tiny_layer_many_tiles_per_expert():
    # 1000 tokens x 4 slots over 32 experts: about 125 rows per expert, some experts cross a 128-row tile
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, seed=1, std=0.05)
    check_layer(s, synth.make_tokens(s, 1000, seed=1), gate, w13, w2, max_tokens=1000)


def test_qwen3_30b_first_config_128_tokens():
    s = synth.QWEN3_30B_A3B
    gate, w13, w2 = synth.make_weights(s, seed=0)
    check_layer(s, synth.make_tokens(s, 128, seed=0), gate, w13, w2, max_tokens=128,
                golden="qwen3_30b_t128_seed0.npz")


def test_qwen3_30b_reference_test_stream_48_tokens_in_place():
    # the reference's own moeTest: 48 tokens of its srand(7907) stream, maxTokens = tokens + 2,
    # output aliasing the input as its vLLM wrapper does
    x, gate, w13, w2 = tl.reference_stream_inputs(48)
    check_layer(synth.QWEN3_30B_A3B, x, gate, w13, w2, max_tokens=50, golden="qwen3_30b_t48_refstream.npz",
                inplace=True)


def test_all_logits_tied_every_token_takes_the_exact_path():
    # zero gate weights: every logit is 0, every token is a tie and is re-gated in the reference's fp32
    # order; the reference keeps the lower expert index first (refTopk.h:36-58), so experts 0..K-1 win
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, seed=2, std=0.05)
    gate = torch.zeros_like(gate)
    check_layer(s, synth.make_tokens(s, 150, seed=2), gate, w13, w2, max_tokens=150)


def test_identical_tokens_one_hot_expert_set():
    # every token is the same row: K experts receive every row (the per-expert buffer is filled to its
    # capacity of one row per token), all other experts none
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, seed=3, std=0.05)
    x = synth.make_tokens(s, 1, seed=3).repeat(300, 1).contiguous()
    check_layer(s, x, gate, w13, w2, max_tokens=300)


def test_zipf_skewed_routing():
    # expert popularity skewed by a per-expert gate bias injected through a constant activation column
    # (the fourth benchmark configuration's construction), 700 tokens
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, seed=4, std=0.05)
    x = synth.make_tokens(s, 700, seed=4)
    gate, x = synth.add_zipf_bias(s, gate, x, s=1.2, scale=1.0, seed=4)
    check_layer(s, x, gate, w13, w2, max_tokens=700)


def test_qwen3_235b_sizes_ragged_tokens():
    # hidden 4096 / intermediate 1536: the exact gate path stages an 8 KB token row, a dispatch stage holds
    # 6 rows instead of 12, COMBINE takes two passes over the hidden columns; 200 tokens, maxTokens above
    s = synth.QWEN3_235B_E16
    gate, w13, w2 = synth.make_weights(s, seed=5)
    check_layer(s, synth.make_tokens(s, 200, seed=6), gate, w13, w2, max_tokens=208)


def test_qwen3_235b_sizes_golden_24_tokens_in_place():
    s = synth.QWEN3_235B_E16
    gate, w13, w2 = synth.make_weights(s, seed=5)
    check_layer(s, synth.make_tokens(s, 24, seed=5), gate, w13, w2, max_tokens=24,
                golden="qwen3_235b_e16_t24_seed5.npz", inplace=True)


def test_qwen3_235b_sizes_many_tiles_per_expert():
    # 1100 tokens x 8 slots over 16 experts: about 550 rows, five m-tiles, per expert
    s = synth.QWEN3_235B_E16
    gate, w13, w2 = synth.make_weights(s, seed=5)
    check_layer(s, synth.make_tokens(s, 1100, seed=7), gate, w13, w2, max_tokens=1100)


def test_qwen3_30b_second_config_4096_tokens_routing_and_output():
    # the benchmark's single-GPU configuration: all 4096 tokens, top-k exact for every one of them
    s = synth.QWEN3_30B_A3B
    gate, w13, w2 = synth.make_weights(s, seed=0)
    check_routing_and_output(s, synth.make_tokens(s, 4096, seed=9), gate, w13, w2, max_tokens=4096)


def test_qwen3_30b_zipf_routing_hottest_expert_takes_every_token():
    # the fourth benchmark configuration's routing: the two most popular experts are selected by every
    # token, so their row buffers are filled to exactly their capacity of one row per token
    s = synth.QWEN3_30B_A3B
    gate, w13, w2 = synth.make_weights(s, seed=0)
    gate, x, info = synth.zipf_routing(s, gate, synth.make_tokens(s, 640, seed=10))
    assert info["selection_share_realised_top8"][0] == 1.0
    check_routing_and_output(s, x, gate, w13, w2, max_tokens=640)
