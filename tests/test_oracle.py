"""Pins the CPU oracle (oracle/moe_oracle.c): against the reference project's own CPU MoE compiled
here (oracle/_ref, when the reference sources are present) and against the committed golden vectors
that were generated from it.  All comparisons are bit-exact."""
import os

import numpy as np
import pytest

import moe_testlib as tl
from moe_testlib import cpu_oracle, synth


@pytest.fixture(scope="module")
def port():
    cpu_oracle.build()
    return cpu_oracle.PortOracle()


def _rand(shape, scale, seed):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def test_gemm_matches_definition(port):
    A, B = _rand((5, 37), 1.0, 1), _rand((7, 37), 1.0, 2)
    C = port.gemm_nt(A, B)
    ref = np.zeros((5, 7), np.float32)
    for i in range(5):
        for j in range(7):
            acc = np.float32(0)
            for k in range(37):
                acc = np.float32(acc + np.float32(A[i, k] * B[j, k]))
            ref[i, j] = acc
    assert np.array_equal(C, ref)


def test_topk_order_and_ties(port):
    # descending, lower index first among equals (reference refTopk.h:36-58 uses strict '>')
    x = np.array([[1, 5, 5, 3, 5, 0, -1, 2, 9, 9]], np.float32)
    v, i = port.topk_rows(x, 4)
    assert i.tolist() == [[8, 9, 1, 2]]
    assert v.tolist() == [[9, 9, 5, 5]]
    # fewer columns than k: padded with lowest()/-1 (refTopk.h:13-15)
    v, i = port.topk_rows(np.array([[2, 1]], np.float32), 4)
    assert i.tolist() == [[0, 1, -1, -1]]


def test_softmax_rows_sum_to_one(port):
    x = _rand((9, 8), 3.0, 3)
    y = port.softmax_rows(x)
    assert np.allclose(y.sum(1), 1.0, atol=1e-6)
    ref = np.exp(x.astype(np.float64) - x.max(1, keepdims=True))
    assert np.allclose(y, ref / ref.sum(1, keepdims=True), atol=1e-7)


def test_empty_input(port):
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, std=0.05)
    out = port.full_moe(np.zeros((0, s.hidden), np.float32), tl.f32(gate), tl.f32(w13), tl.f32(w2), s.topk)
    assert out.shape == (0, s.hidden)


def test_threads_do_not_change_result(port):
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, std=0.05)
    x = tl.f32(synth.make_tokens(s, 11))
    a = port.full_moe(x, tl.f32(gate), tl.f32(w13), tl.f32(w2), s.topk, threads=1)
    b = port.full_moe(x, tl.f32(gate), tl.f32(w13), tl.f32(w2), s.topk, threads=4)
    assert np.array_equal(a, b)


def test_stage_outputs_compose(port):
    s = synth.TINY
    gate, w13, w2 = [tl.f32(t) for t in synth.make_weights(s, std=0.05)]
    x = tl.f32(synth.make_tokens(s, 7))
    out, tw, ti, act, y = port.full_moe(x, gate, w13, w2, s.topk, stages=True)
    for t in range(7):
        acc = np.zeros(s.hidden, np.float32)
        for k in range(s.topk):
            e = ti[t, k]
            assert np.array_equal(act[t, k], port.ffn1(x[t:t + 1], w13[e])[0])
            assert np.array_equal(y[t, k], port.gemm_nt(act[t, k:k + 1], w2[e])[0])
            acc = (acc + y[t, k] * tw[t, k]).astype(np.float32)
        assert np.array_equal(acc, out[t])


@pytest.mark.skipif(not cpu_oracle.RefOracle.available(), reason="oracle/_ref not built")
def test_port_equals_reference_build(port):
    ref = cpu_oracle.RefOracle()
    s = synth.TINY
    gate, w13, w2 = [tl.f32(t) for t in synth.make_weights(s, seed=3, std=0.05)]
    x = tl.f32(synth.make_tokens(s, 19, seed=3))
    assert np.array_equal(port.gemm_nt(x, gate), ref.gemm_nt(x, gate))
    pw, pi = port.gate(x, gate, s.topk)
    rw, ri = ref.gate(x, gate, s.topk)
    assert np.array_equal(pi, ri) and np.array_equal(pw, rw)
    assert np.array_equal(port.ffn1(x, w13[5]), ref.ffn1(x, w13[5]))
    assert np.array_equal(port.full_moe(x, gate, w13, w2, s.topk), ref.full_moe(x, gate, w13, w2, s.topk))
    assert np.array_equal(ref.full_moe(x, gate, w13, w2, s.topk, threads=3), ref.full_moe(x, gate, w13, w2, s.topk))


def _check_golden(port, name, x, gate, w13, w2, topk):
    g = np.load(os.path.join(tl.GOLDEN, name))
    assert [tl.sha(t) for t in (x, gate, w13, w2)] == list(g["hashes"]), "input generators drifted"
    xf, gf = tl.f32(x), tl.f32(gate)
    tw, ti = port.gate(xf, gf, topk)
    assert np.array_equal(ti, g["topk_idx"])
    assert np.array_equal(tw, g["topk_w"])
    out = port.full_moe(xf, gf, tl.f32(w13), tl.f32(w2), topk, threads=port.max_threads())
    assert np.array_equal(out, g["out"])


def test_golden_tiny(port):
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, seed=0, std=0.05)
    _check_golden(port, "tiny_t40.npz", synth.make_tokens(s, 40, seed=0), gate, w13, w2, s.topk)


def test_golden_qwen3_30b_first_config(port):
    s = synth.QWEN3_30B_A3B
    gate, w13, w2 = synth.make_weights(s, seed=0)
    _check_golden(port, "qwen3_30b_t128_seed0.npz", synth.make_tokens(s, 128, seed=0), gate, w13, w2, s.topk)


def test_golden_reference_test_stream(port):
    x, gate, w13, w2 = tl.reference_stream_inputs(48)
    _check_golden(port, "qwen3_30b_t48_refstream.npz", x, gate, w13, w2, 8)


def test_golden_qwen3_235b_sizes(port):
    s = synth.QWEN3_235B_E16
    gate, w13, w2 = synth.make_weights(s, seed=5)
    _check_golden(port, "qwen3_235b_e16_t24_seed5.npz", synth.make_tokens(s, 24, seed=5), gate, w13, w2, s.topk)


def test_bf16_weight_variant_equals_widened_weights(port):
    # the variant the benchmark's multi-rank parity check uses (one bf16 copy of all expert weights
    # shared between the ranks): bit-identical to the fp32 entry point on the widened weights
    import torch
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, seed=6, std=0.05)
    x = tl.f32(synth.make_tokens(s, 33, seed=6))
    out, tw, ti, _, _ = port.full_moe(x, tl.f32(gate), tl.f32(w13), tl.f32(w2), s.topk, threads=3, stages=True)
    bits = lambda t: t.view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    out2, tw2, ti2 = port.full_moe_bf16_weights(x, tl.f32(gate), bits(w13), bits(w2), s.topk, threads=2)
    assert np.array_equal(out, out2) and np.array_equal(tw, tw2) and np.array_equal(ti, ti2)


def test_torch_restatement_agrees_with_the_port(port):
    # the plain-torch CPU path that the benchmark times beside the reference's own CPU code
    import torch
    from oracle.torch_moe import torch_moe
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, std=0.05)
    x = synth.make_tokens(s, 200, seed=3)
    out, tw, ti, _, _ = port.full_moe(tl.f32(x), tl.f32(gate), tl.f32(w13), tl.f32(w2), s.topk, stages=True)
    got, gw, gi = torch_moe(x.float(), gate.float(), w13.float(), w2.float(), s.topk)
    logits = port.gemm_nt(tl.f32(x), tl.f32(gate))
    srt = -np.sort(-logits, axis=1)[:, :s.topk + 1]
    clear = (srt[:, :-1] - srt[:, 1:]).min(axis=1) > 1e-5      # rows whose routing no rounding can change
    assert clear.mean() > 0.9
    assert (gi.numpy()[clear] == ti[clear]).all()
    np.testing.assert_allclose(gw.numpy()[clear], tw[clear], atol=1e-6)
    np.testing.assert_allclose(got.numpy()[clear], out[clear], atol=1e-5)
