"""Generates the golden vectors under tests/golden/ from the REFERENCE project's own CPU MoE
(oracle/_ref/libref_moe.so, compiled by oracle/Makefile from the reference sources where they lie).

    python tests/golden/make_golden.py

Needs the reference sources (it runs where they exist); the .npz files it writes are committed and
are what travels.  Inputs are not stored (they are regenerated from seeds); their hashes are, so a
drift of the generators is detected instead of silently changing the test.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import moe_testlib as tl  # noqa: E402
from moe_testlib import cpu_oracle, synth  # noqa: E402


def run_ref(ref, x, gate, w13, w2, topk, threads):
    xf, gf, w13f, w2f = tl.f32(x), tl.f32(gate), tl.f32(w13), tl.f32(w2)
    tw, ti = ref.gate(xf, gf, topk)
    out = ref.full_moe(xf, gf, w13f, w2f, topk, threads=threads)
    return dict(topk_idx=ti, topk_w=tw, out=out,
                hashes=np.array([tl.sha(x), tl.sha(gate), tl.sha(w13), tl.sha(w2)]))


def main():
    cpu_oracle.build()
    ref = cpu_oracle.RefOracle()
    threads = ref.max_threads()

    # 1. tiny layer, ragged token count
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, seed=0, std=0.05)
    x = synth.make_tokens(s, 40, seed=0)
    np.savez_compressed(os.path.join(HERE, "tiny_t40.npz"), **run_ref(ref, x, gate, w13, w2, s.topk, threads))

    # 2. Qwen3-30B-A3B layer, 128 tokens, seed 0 (first benchmark configuration)
    s = synth.QWEN3_30B_A3B
    gate, w13, w2 = synth.make_weights(s, seed=0)
    x = synth.make_tokens(s, 128, seed=0)
    np.savez_compressed(os.path.join(HERE, "qwen3_30b_t128_seed0.npz"),
                        **run_ref(ref, x, gate, w13, w2, s.topk, threads))

    # 3. the reference tests' own input stream (srand(7907) uniform), 48 tokens as in its moeTest
    x, gate, w13, w2 = tl.reference_stream_inputs(48)
    np.savez_compressed(os.path.join(HERE, "qwen3_30b_t48_refstream.npz"),
                        **run_ref(ref, x, gate, w13, w2, 8, threads))
    # 4. Qwen3-235B-A22B hidden/intermediate sizes with 16 experts (one rank's share at 8 GPUs), 24 tokens
    s = synth.QWEN3_235B_E16
    gate, w13, w2 = synth.make_weights(s, seed=5)
    x = synth.make_tokens(s, 24, seed=5)
    np.savez_compressed(os.path.join(HERE, "qwen3_235b_e16_t24_seed5.npz"),
                        **run_ref(ref, x, gate, w13, w2, s.topk, threads))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
