"""Data-parallel + expert-parallel vLLM run of a one-layer Qwen3-MoE model with and without the patch
that routes its MoE block through the launcher (twin of the reference's
test/multiGPU/python/benchmark_dp.py:137-252,412-435 and flash_moe_patch.py:42-112).

    python tests/vllm_dp_harness.py --dp 2 [--mode tokens|verify] [--out result.json]

One process per data-parallel rank (one GPU each), expert parallelism on, eager mode, no tokenizer.
The model is written to a temporary directory with seeded weights (a checkpoint of a few MB; vLLM's
own dummy weights are so small that every logit is a tie), so greedy decoding is well defined.  The
script runs the job twice, patch off and patch on, and compares the generated token ids: the first
generated token of every prompt must agree, and at least 90 % of all generated tokens (after a
first difference, caused by bf16 rounding of nearly tied logits, the two runs decode different
histories).  `--mode verify` brings up the patched job only, in the patch's checking mode: every call
of the MoE block runs vLLM's own block and the kernel on the same input inside the engine, and the
script requires that the job generates its tokens and that at least 95 % of all rows of all calls lie
within a relative L2 distance of 2e-2 of vLLM's rows (vLLM routes on bf16 logits, so a few per cent of
the rows pick another last expert than the kernel's exact routing and differ more).  Unlike the reference's patch, which falls back to vLLM's block when ep_size > 1
(flash_moe_patch.py:104), the patched run dispatches rows between the ranks inside the kernel.

Exit codes: 0 agreement, 1 the token ids disagree, 77 vLLM itself could not run here, 78 the patched
engine did not come up (the caller skips on both, with the message).
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import socket
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, HEADS, KV_HEADS, EXPERTS, TOPK, INTER, VOCAB = 256, 4, 2, 32, 4, 128, 512


def make_model_dir(path: str, seed: int = 0) -> str:
    """config.json + model.safetensors of a one-layer Qwen3-MoE model with seeded weights."""
    import torch
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    head_dim = HIDDEN // HEADS
    config = {
        "architectures": ["Qwen3MoeForCausalLM"], "model_type": "qwen3_moe", "hidden_size": HIDDEN,
        "intermediate_size": HIDDEN * 2, "num_hidden_layers": 1, "vocab_size": VOCAB,
        "max_position_embeddings": 256, "num_attention_heads": HEADS, "num_key_value_heads": KV_HEADS,
        "head_dim": head_dim, "attention_bias": False, "attention_dropout": 0.0, "num_experts": EXPERTS,
        "num_experts_per_tok": TOPK, "moe_intermediate_size": INTER, "decoder_sparse_step": 1,
        "norm_topk_prob": True, "output_router_logits": False, "router_aux_loss_coef": 0.001,
        "mlp_only_layers": [], "hidden_act": "silu", "initializer_range": 0.02, "rms_norm_eps": 1e-6,
        "use_cache": True, "tie_word_embeddings": False, "rope_theta": 10000.0, "rope_scaling": None,
        "use_sliding_window": False, "sliding_window": None, "torch_dtype": "bfloat16", "dtype": "bfloat16",
        "transformers_version": "4.51.0", "bos_token_id": 1, "eos_token_id": 2,
    }
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    g = torch.Generator().manual_seed(seed)

    def w(*shape, std=0.05):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16).contiguous()

    ones = lambda n: torch.ones(n, dtype=torch.bfloat16)  # noqa: E731
    t = {"model.embed_tokens.weight": w(VOCAB, HIDDEN, std=1.0), "model.norm.weight": ones(HIDDEN),
         "lm_head.weight": w(VOCAB, HIDDEN, std=0.3)}
    p = "model.layers.0."
    t[p + "input_layernorm.weight"] = ones(HIDDEN)
    t[p + "post_attention_layernorm.weight"] = ones(HIDDEN)
    t[p + "self_attn.q_proj.weight"] = w(HEADS * head_dim, HIDDEN)
    t[p + "self_attn.k_proj.weight"] = w(KV_HEADS * head_dim, HIDDEN)
    t[p + "self_attn.v_proj.weight"] = w(KV_HEADS * head_dim, HIDDEN)
    t[p + "self_attn.o_proj.weight"] = w(HIDDEN, HEADS * head_dim)
    t[p + "self_attn.q_norm.weight"] = ones(head_dim)
    t[p + "self_attn.k_norm.weight"] = ones(head_dim)
    t[p + "mlp.gate.weight"] = w(EXPERTS, HIDDEN, std=0.2)
    for e in range(EXPERTS):
        t[p + f"mlp.experts.{e}.gate_proj.weight"] = w(INTER, HIDDEN, std=0.1)
        t[p + f"mlp.experts.{e}.up_proj.weight"] = w(INTER, HIDDEN, std=0.1)
        t[p + f"mlp.experts.{e}.down_proj.weight"] = w(HIDDEN, INTER, std=0.1)
    save_file(t, os.path.join(path, "model.safetensors"))
    return path


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(dp_size, rank, port, model_dir, patched, prompts, max_tokens, queue, extra_env=None):
    try:
        os.environ.update(extra_env or {})
        os.environ.update({"VLLM_DP_RANK": str(rank), "VLLM_DP_RANK_LOCAL": str(rank), "VLLM_DP_SIZE": str(dp_size),
                           "VLLM_DP_MASTER_IP": "127.0.0.1", "VLLM_DP_MASTER_PORT": str(port),
                           "HF_HUB_OFFLINE": "1", "TRANSFORMERS_OFFLINE": "1", "VLLM_LOGGING_LEVEL": "WARNING",
                           "FLASH_MOE_MAX_TOKENS": "512"})
        if dp_size == 1:
            for k in ("VLLM_DP_RANK", "VLLM_DP_RANK_LOCAL", "VLLM_DP_SIZE", "VLLM_DP_MASTER_IP", "VLLM_DP_MASTER_PORT"):
                os.environ.pop(k, None)
            os.environ["CUDA_VISIBLE_DEVICES"] = os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0]
        if patched:
            from flash_distributed_moe_b200.vllm_patch import enable_flash_moe_patching
            enable_flash_moe_patching()  # before the engine spawns its core process
        from vllm import LLM, SamplingParams
        t0 = time.time()
        llm = LLM(model=model_dir, skip_tokenizer_init=True, enforce_eager=True, enable_expert_parallel=True,
                  gpu_memory_utilization=0.2, max_model_len=128, max_num_batched_tokens=256, max_num_seqs=16,
                  dtype="bfloat16", disable_log_stats=True, seed=0)
        init_s = time.time() - t0
        mine = prompts[rank::dp_size] or [prompts[0]]
        sp = SamplingParams(temperature=0.0, top_p=1.0, ignore_eos=True, max_tokens=max_tokens, detokenize=False)
        t0 = time.time()
        outs = llm.generate([{"prompt_token_ids": p} for p in mine], sp, use_tqdm=False)
        gen_s = time.time() - t0
        queue.put({"rank": rank, "ok": True, "tokens": [list(o.outputs[0].token_ids) for o in outs],
                   "init_s": init_s, "gen_s": gen_s})
        time.sleep(1.0)  # let the other ranks finish their last (collective) steps
    except Exception as e:  # reported to the parent, which decides between failure and skip
        import traceback
        queue.put({"rank": rank, "ok": False, "error": f"{type(e).__name__}: {e}", "trace": traceback.format_exc()[-3000:]})


def run_job(dp_size, model_dir, patched, prompts, max_tokens, timeout_s=900, extra_env=None):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(dp_size, r, port, model_dir, patched, prompts, max_tokens, queue, extra_env))
             for r in range(dp_size)]
    for p in procs:
        p.start()
    results, deadline = {}, time.time() + timeout_s
    while len(results) < dp_size and time.time() < deadline:
        try:
            r = queue.get(timeout=5)
            results[r["rank"]] = r
        except Exception:
            if not any(p.is_alive() for p in procs):
                break
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.kill()
    return results


def verify_mode(args, model_dir, prompts) -> int:
    """The patched job alone, in the patch's checking mode; returns the exit code."""
    import glob
    log = os.path.join(tempfile.mkdtemp(prefix="flash_moe_verify_"), "calls")
    res = run_job(args.dp, model_dir, True, prompts, args.max_tokens, args.job_timeout,
                  {"FLASH_MOE_VERIFY": "1", "FLASH_MOE_VERIFY_LOG": log})
    bad = [r for r in res.values() if not r.get("ok")]
    if len(res) < args.dp or bad:
        print(json.dumps({"status": "vllm could not run", "patched": True, "dp": args.dp,
                          "errors": [b.get("error") for b in bad], "trace": (bad[0].get("trace") if bad else "")}))
        return 78
    calls = [json.loads(line) for f in glob.glob(log + ".*") for line in open(f) if line.strip()]
    rows = sum(c["rows"] for c in calls)
    beyond = sum(c["rows_beyond"] for c in calls)
    generated = sum(len(t) for r in res.values() for t in r["tokens"])
    report = {"status": "ok", "mode": "verify", "dp": args.dp, "processes_with_calls": len(glob.glob(log + ".*")),
              "calls": len(calls), "rows": rows, "rows_beyond_2e-2": beyond,
              "median_of_call_medians": (sorted(c["median"] for c in calls)[len(calls) // 2] if calls else None),
              "max_row_distance": max((c["max"] for c in calls), default=None), "tokens_generated": generated,
              "init_s": max(r["init_s"] for r in res.values()), "gen_s": max(r["gen_s"] for r in res.values())}
    print(json.dumps(report))
    if args.out:
        with open(args.out, "w") as f:
            json.dump(report, f)
    want = len(prompts) * args.max_tokens if args.dp <= len(prompts) else None
    ok = len(calls) > 0 and rows > 0 and beyond <= 0.05 * rows and (want is None or generated == want)
    return 0 if ok else 1


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--prompts", type=int, default=8)
    ap.add_argument("--input-len", type=int, default=24)
    ap.add_argument("--max-tokens", type=int, default=6)
    ap.add_argument("--out", default="")
    ap.add_argument("--mode", choices=("tokens", "verify"), default="tokens")
    ap.add_argument("--job-timeout", type=int, default=900)
    args = ap.parse_args()
    import numpy as np
    rng = np.random.RandomState(0)
    prompts = [rng.randint(3, VOCAB, size=args.input_len).tolist() for _ in range(args.prompts)]
    model_dir = make_model_dir(tempfile.mkdtemp(prefix="qwen3moe_tiny_"))
    if args.mode == "verify":
        sys.exit(verify_mode(args, model_dir, prompts))
    runs = {}
    for patched in (False, True):
        res = run_job(args.dp, model_dir, patched, prompts, args.max_tokens, args.job_timeout)
        bad = [r for r in res.values() if not r.get("ok")]
        if len(res) < args.dp or bad:
            print(json.dumps({"status": "vllm could not run", "patched": patched, "dp": args.dp,
                              "errors": [b.get("error") for b in bad], "trace": (bad[0].get("trace") if bad else "")}))
            sys.exit(77 if not patched else 78)
        runs[patched] = res
    base = [t for r in range(args.dp) for t in runs[False][r]["tokens"]]
    ours = [t for r in range(args.dp) for t in runs[True][r]["tokens"]]
    first_equal = all(a[0] == b[0] for a, b in zip(base, ours))
    total = sum(len(a) for a in base)
    equal = sum(int(x == y) for a, b in zip(base, ours) for x, y in zip(a, b))
    tok_s = {p: sum(len(t) for r in runs[p].values() for t in r["tokens"]) / max(r2["gen_s"] for r2 in runs[p].values())
             for p in (False, True)}
    report = {"status": "ok", "dp": args.dp, "prompts": len(base), "first_token_equal": first_equal,
              "tokens_equal": equal, "tokens_total": total, "tokens_per_s_vllm": tok_s[False],
              "tokens_per_s_patched": tok_s[True]}
    print(json.dumps(report))
    if args.out:
        with open(args.out, "w") as f:
            json.dump(report, f)
    sys.exit(0 if first_equal and equal >= 0.9 * total else 1)


if __name__ == "__main__":
    main()
