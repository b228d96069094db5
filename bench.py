#!/usr/bin/env python
"""MoE-layer throughput benchmark (tokens/s) for the B200 FlashDMoE launcher.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--shape 30b|235b] [--tokens T] [--skew none|zipf]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one `Launch` of the layer over one batch of synthetic tokens (seeded N(0,1) bf16
activations, N(0,0.02) bf16 weights; real Qwen3 checkpoints are not available offline).  Default
workload: the Qwen3-30B-A3B layer shape (hidden 2048, 128 experts, top-8, intermediate 768) at 4096
tokens per GPU; with N > 1 the experts are sharded over the ranks (expert parallelism) and the
tokens per GPU stay fixed (weak scaling).  `--skew zipf` biases the gate so that expert popularity
follows Zipf(1.2).  Before anything is timed, every rank checks a sample of its tokens against the
CPU oracle (top-k indices exact, output within max-abs 2e-2 / rel-L2 1e-2).  Rank 0 prints ONE JSON
line.  At N = 1 its `cpu_baseline` holds the reference project's CPU MoE on all host threads (`value`),
the same code on one thread (`single_thread`) and a plain-torch restatement of the same math on the
host cores (`torch_cpu`), each timed on a bounded sample of the step's tokens.

`--impl reference` times the reference project's own CPU MoE (oracle/_ref when it was built from
the reference sources, else the C restatement under oracle/) on the host cores, on a bounded sample
of the same workload per step.
"""
from __future__ import annotations

import argparse
import atexit
import json
import os
import statistics
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from flash_distributed_moe_b200 import synth  # noqa: E402

SHAPES = {"30b": synth.QWEN3_30B_A3B, "235b": synth.QWEN3_235B_A22B}
L2_BYTES = 126e6
MAX_ABS, REL_L2 = 2e-2, 1e-2


def flops_per_token(s) -> float:
    return 2.0 * s.hidden * s.experts + s.topk * 6.0 * s.hidden * s.inter


def algorithmic_bytes(s, tokens, world) -> float:
    """HBM bytes one launch has to move on one GPU: active expert weights once, token rows in, packed rows
    written and read, activations written and read, weighted rows written and read, output rows out, gate."""
    pairs = tokens * s.topk
    weights = (s.experts // world) * 3 * s.hidden * s.inter * 2
    return (weights + 2 * s.hidden * s.experts + 2 * s.hidden * tokens * 2
            + 2 * (2 * s.hidden * pairs) + 2 * (2 * s.inter * pairs) + 2 * (2 * s.hidden * pairs))


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the persistent kernel from ncu, for the
# workloads that were captured (profiles/): (shape, tokens per GPU, GPUs) -> bytes
MEASURED_TRAFFIC = {("30b", 4096, 1): 1.637e9 + 0.328e9}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) in a background thread
    while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.001):
        import threading
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            phys = index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None
            return
        self._period = period_s
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        nv = self._nv
        flags = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "sw_power_cap": 0x4}
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for name, bit in flags.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self._period)

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def workload_name(shape, tokens, world, skew) -> str:
    routing = "random gate" if skew == "none" else "gate biased to Zipf(1.2) expert popularity"
    return (f"{shape.name} MoE layer, {tokens} tokens per GPU, top-{shape.topk} of {shape.experts} experts, "
            f"{routing}, experts sharded over {world} GPU(s)")


def make_gate_and_tokens(shape, tokens, rank, device, skew):
    """Gate weights (identical on all ranks) and this rank's tokens, bf16 on the device.  With
    skew == "zipf" the last activation column is 1 and the gate column holds a per-expert bias
    (reference construction: test/common/moeTools.h:187-207); returns the realised popularity too."""
    g = torch.Generator(device=device).manual_seed(0)
    gate = (torch.randn(shape.experts, shape.hidden, generator=g, device=device) * 0.02).to(torch.bfloat16)
    gt = torch.Generator(device=device).manual_seed(7 + rank)
    x = torch.randn(tokens, shape.hidden, generator=gt, device=device).to(torch.bfloat16)
    info = None
    if skew == "zipf":
        gate_c, x_c, info = synth.zipf_routing(shape, gate.cpu(), x.cpu(), s=1.2, seed=0)
        gate, x = gate_c.to(device), x_c.to(device)
    return gate, x, info


def make_expert_shard(shape, rank, world, device):
    """This rank's contiguous shard of the expert weights, generated on the device (one seed per rank;
    the parity check reads back what the GPUs really hold, so the set need not be independent of the
    sharding)."""
    el = shape.experts // world
    ge = torch.Generator(device=device).manual_seed(1000 + rank)
    w13 = (torch.randn(el, 2 * shape.inter, shape.hidden, generator=ge, device=device) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(el, shape.hidden, shape.inter, generator=ge, device=device) * 0.02).to(torch.bfloat16)
    return w13, w2


class SharedWeights:
    """All ranks' expert shards as bf16 bit patterns in one memory-mapped file that every rank can read
    (each rank writes the shard its GPU really uses), for the CPU oracle's parity check."""

    def __init__(self, shape, rank, world, w13, w2, barrier):
        base = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else "/tmp"
        tag = os.environ.get("MASTER_PORT", "0") + "_" + str(os.getppid() if world > 1 else os.getpid())
        self.paths = [os.path.join(base, f"flashmoe_bench_{tag}_{n}.bin") for n in ("w13", "w2")]
        E, H, I = shape.experts, shape.hidden, shape.inter
        el = E // world
        shapes = [(E, 2 * I, H), (E, H, I)]
        self.rank = rank
        if rank == 0:
            for p, shp in zip(self.paths, shapes):
                np.lib.format.open_memmap(p, mode="w+", dtype=np.uint16, shape=shp).flush()
        barrier()
        self.maps = [np.load(p, mmap_mode="r+") for p in self.paths]
        atexit.register(self._unlink)  # a rank that dies before close() must not leave gigabytes behind
        for m, t in zip(self.maps, (w13, w2)):
            m[rank * el:(rank + 1) * el] = t.cpu().view(torch.int16).numpy().view(np.uint16)
            m.flush()
        barrier()

    def _unlink(self):
        # (removing a file that other ranks still have mapped leaves their mappings valid)
        for p in self.paths:
            try:
                os.remove(p)
            except OSError:
                pass

    def close(self, barrier):
        self.maps = None
        barrier()
        if self.rank == 0:
            self._unlink()


def parity_check(shape, launcher, shared, gate, x, out, n_check, threads):
    """Top-k indices (exact) and output (north-star tolerances) of a sample of this rank's tokens
    against the CPU oracle.  This and cpu_baseline_leg are the only places the b200 arm touches oracle/."""
    from oracle import cpu_oracle
    port = cpu_oracle.PortOracle()
    T = x.shape[0]
    n = min(n_check, T)
    if n == 0:
        return {"tokens_checked": 0, "topk_mismatch_tokens": 0, "max_abs": 0.0, "rel_l2": 0.0, "pass": True}
    sel = np.unique(np.linspace(0, T - 1, n).astype(np.int64))
    xs = np.ascontiguousarray(x[torch.from_numpy(sel).to(x.device)].float().cpu().numpy())
    ref, _, ref_idx = port.full_moe_bf16_weights(xs, np.ascontiguousarray(gate.float().cpu().numpy()),
                                                 shared.maps[0], shared.maps[1], shape.topk, threads=threads)
    idx = np.frombuffer(launcher.debug_read(0, T * shape.topk * 4), np.int32).reshape(T, shape.topk)[sel]
    got = out[torch.from_numpy(sel).to(out.device)].float().cpu().numpy()
    mism = int((idx != ref_idx).any(axis=1).sum())
    max_abs = float(np.abs(got - ref).max())
    rel = float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))
    return {"tokens_checked": int(len(sel)), "topk_mismatch_tokens": mism, "max_abs": max_abs, "rel_l2": rel,
            "pass": bool(mism == 0 and max_abs <= MAX_ABS and rel <= REL_L2)}


def cpu_reference_run(oracle, xf, gf, w13f, w2f, topk, threads):
    t0 = time.perf_counter()
    out = oracle.full_moe(xf, gf, w13f, w2f, topk, threads=threads)
    return out, time.perf_counter() - t0


def cpu_baseline_leg(shape, gate, w13, w2, x, budget_s=12.0):
    """Times the CPU reference on a bounded sample of the step's tokens with all host threads."""
    from oracle import cpu_oracle
    cpu_oracle.build()
    oracle = cpu_oracle.best_oracle()
    threads = oracle.max_threads()
    gf = gate.float().cpu().numpy()
    w13f = w13.float().cpu().numpy()
    w2f = w2.float().cpu().numpy()
    xs = x[:4096].float().cpu().numpy()
    probe = min(threads, xs.shape[0])
    _, dt = cpu_reference_run(oracle, xs[:probe], gf, w13f, w2f, shape.topk, threads)
    per_round = max(dt, 1e-3)
    n = int(min(xs.shape[0], max(probe, probe * int(budget_s / per_round))))
    _, dt = cpu_reference_run(oracle, xs[:n], gf, w13f, w2f, shape.topk, threads)
    # the same code on one thread (tokens are independent, the cost per token is constant)
    n1 = max(1, min(32, int(1.5 / max(per_round, 1e-3))))
    _, dt1 = cpu_reference_run(oracle, xs[:n1], gf, w13f, w2f, shape.topk, 1)
    # the plain-torch restatement of the same math on the host cores (library GEMMs, expert by expert)
    from oracle.torch_moe import torch_moe
    tg, t13, t2 = (torch.from_numpy(a) for a in (gf, w13f, w2f))
    xt = x[:min(x.shape[0], 2048)].float().cpu()
    torch_moe(xt[:64], tg, t13, t2, shape.topk)
    t0 = time.perf_counter()
    torch_moe(xt, tg, t13, t2, shape.topk)
    dtt = time.perf_counter() - t0
    return {"value": n / dt, "unit": "tokens/s", "cores": threads, "kind": oracle.kind,
            "sample": f"first {n} tokens of the step's batch, fp32, all host threads, {dt:.1f} s",
            "single_thread": {"value": n1 / dt1, "unit": "tokens/s", "cores": 1,
                              "sample": f"first {n1} tokens, {dt1:.1f} s"},
            "torch_cpu": {"value": xt.shape[0] / dtt, "unit": "tokens/s", "cores": torch.get_num_threads(),
                          "kind": "port",
                          "sample": f"first {xt.shape[0]} tokens of the step's batch through the plain-torch "
                                    f"restatement (fp32, library GEMMs per expert), {dtt:.2f} s"}}


def run_reference_arm(args, shape):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from oracle import cpu_oracle
    cpu_oracle.build()
    oracle = cpu_oracle.best_oracle()
    threads = oracle.max_threads()
    gate, w13, w2 = synth.make_weights(shape, seed=0)
    x = synth.make_tokens(shape, min(args.tokens, 2048), seed=0)
    if args.skew == "zipf":
        gate, x, _ = synth.zipf_routing(shape, gate, x, s=1.2, seed=0)
    gf, w13f, w2f, xf = [t.float().numpy() for t in (gate, w13, w2, x)]
    # bounded sample per step: calibrate one round of `threads` tokens, then size the step so that the
    # whole run stays within about two minutes
    probe = min(threads, xf.shape[0])
    _, dt = cpu_reference_run(oracle, xf[:probe], gf, w13f, w2f, shape.topk, threads)
    total_steps = args.steps + args.warmup
    per_step_budget = max(0.5, 120.0 / max(total_steps, 1))
    n = int(min(xf.shape[0], max(probe, probe * int(per_step_budget / max(dt, 1e-3)))))
    for _ in range(args.warmup):
        cpu_reference_run(oracle, xf[:n], gf, w13f, w2f, shape.topk, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_run(oracle, xf[:n], gf, w13f, w2f, shape.topk, threads)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    value = n / dt
    sample = f"{n} tokens per step of the {args.tokens}-token batch, fp32, {threads} host threads"
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(shape, args.tokens, args.gpus, args.skew),
                   "hidden": shape.hidden, "inter": shape.inter, "tokens_per_gpu": args.tokens},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": oracle.kind, "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--shape", default="30b", choices=sorted(SHAPES))
    ap.add_argument("--tokens", type=int, default=4096, help="tokens per GPU per step")
    ap.add_argument("--skew", default="none", choices=["none", "zipf"], help="expert popularity")
    ap.add_argument("--parity-tokens", type=int, default=512, help="tokens per rank checked against the CPU oracle")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    shape = SHAPES[args.shape]
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args, shape)
        return

    rank, world, local = dist_env()
    if world != args.gpus:
        if args.gpus != 1 or world != 1:
            raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)

    from flash_distributed_moe_b200 import MoeKernelLauncher
    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    T = args.tokens
    gate, x, skew_info = make_gate_and_tokens(shape, T, rank, device, args.skew)
    w13, w2 = make_expert_shard(shape, rank, world, device)
    launcher = MoeKernelLauncher()
    if world > 1:
        box = [MoeKernelLauncher.getDistributedUniqueId() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        uid = box[0]
    else:
        uid = MoeKernelLauncher.getDistributedUniqueId(empty=True)
    launcher.create(gate, w13, w2, T, uid, rank, world, topk=shape.topk)
    out = torch.empty_like(x)

    # ---- parity gate, before anything is timed: a sample of every rank's tokens against the CPU oracle
    from oracle import cpu_oracle
    if rank == 0:
        cpu_oracle.build()
    barrier()
    shared = SharedWeights(shape, rank, world, w13, w2, barrier)
    launcher.launch(x, out)
    barrier()
    code, info = launcher.last_status()
    if code != 0:
        raise SystemExit(f"device-side error {code} (info 0x{info:x}) in the parity launch")
    threads = max(1, (os.cpu_count() or 1) // world)
    par = parity_check(shape, launcher, shared, gate, x, out, args.parity_tokens, threads)
    if world > 1:
        t = torch.tensor([float(par["topk_mismatch_tokens"]), par["max_abs"], par["rel_l2"],
                          0.0 if par["pass"] else 1.0], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst = [float(v) for v in t.tolist()]
    else:
        worst = [float(par["topk_mismatch_tokens"]), par["max_abs"], par["rel_l2"], 0.0 if par["pass"] else 1.0]
    parity = {"tokens_checked_per_rank": par["tokens_checked"], "ranks": world,
              "topk_mismatch_tokens_worst_rank": int(worst[0]), "max_abs": worst[1], "rel_l2": worst[2],
              "tolerance": {"topk": "exact", "max_abs": MAX_ABS, "rel_l2": REL_L2}, "pass": worst[3] == 0.0}
    shared.close(barrier)

    for _ in range(args.warmup):
        launcher.launch(x, out)
    barrier()
    code, info = launcher.last_status()
    if code != 0:
        raise SystemExit(f"device-side error {code} (info 0x{info:x}) during warm-up")

    # ---- device-resident timing: K launches, one event pair per launch (inputs stay in HBM; the
    # expert weights read each step plus the row buffers written and read exceed L2, so no flush is needed)
    sampler = ClockSampler(local) if rank == 0 else None
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for i in range(args.steps):
        starts[i].record()
        launcher.launch(x, out)
        stops[i].record()
    t_end.record()
    barrier()
    total_ms = t_begin.elapsed_time(t_end)
    per_launch_ms = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    code, info = launcher.last_status()
    if code != 0:
        raise SystemExit(f"device-side error {code} (info 0x{info:x}) during the timed region")

    # ---- end to end through the host-buffer entry point: pinned host tokens in, pinned host result out
    h_in = x.cpu().pin_memory()
    h_out = torch.empty_like(h_in).pin_memory()
    for _ in range(2):
        launcher.launch_host(h_in, h_out)
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        launcher.launch_host(h_in, h_out)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None  # covers both timed regions
    e2e_ok = torch.equal(h_out, out.cpu())

    if world > 1:
        t = torch.tensor([total_ms, e2e_ms, max(per_launch_ms), statistics.mean(per_launch_ms),
                          0.0 if e2e_ok else 1.0], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms, _, mean_launch_ms, e2e_bad = [float(v) for v in t.tolist()]
        e2e_ok = e2e_bad == 0.0
    else:
        mean_launch_ms = statistics.mean(per_launch_ms)

    result = None
    if rank == 0:
        peaks = measured_peaks()
        tokens_total = T * world
        ms_per_step = total_ms / args.steps
        value = tokens_total / (ms_per_step * 1e-3)
        flop_launch = flops_per_token(shape) * T  # per GPU (every rank computes T*K pairs on average)
        achieved_tflops = flop_launch / (mean_launch_ms * 1e-3) / 1e12
        expert_tflops = shape.topk * 6.0 * shape.hidden * shape.inter * T / (mean_launch_ms * 1e-3) / 1e12
        alg_bytes = algorithmic_bytes(shape, T, world)
        hbm_gbs = alg_bytes / (mean_launch_ms * 1e-3) / 1e9
        # The launch has two floors: its expert GEMMs at the measured tensor peak and its algorithmic bytes
        # at the measured copy bandwidth.  The bound reported is the higher floor (the larger fraction);
        # both fractions are given.
        tensor_frac = achieved_tflops / peaks["bf16_tflops"]
        hbm_frac = hbm_gbs / peaks["hbm_gbs"]
        roofline = {"kernel": "moe_persistent_kernel", "kernel_ms": mean_launch_ms,
                    "peak_source": peaks["source"] + " (tensor: burst)",
                    "tensor_tflops": achieved_tflops, "tensor_peak_tflops": peaks["bf16_tflops"], "tensor_frac": tensor_frac,
                    "expert_gemm_tflops": expert_tflops, "expert_gemm_frac": expert_tflops / peaks["bf16_tflops"],
                    "hbm_algorithmic_gbs": hbm_gbs, "hbm_peak_gbs": peaks["hbm_gbs"], "hbm_frac": hbm_frac,
                    "algorithmic_bytes": alg_bytes, "algorithmic_flop": flop_launch,
                    "traffic": MEASURED_TRAFFIC.get((args.shape, T, world)),
                    "traffic_unit": "bytes/launch (ncu dram read+write)"}
        if hbm_frac > tensor_frac:
            roofline.update({"bound": "hbm", "achieved": hbm_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": hbm_frac})
        else:
            roofline.update({"bound": "tensor", "achieved": achieved_tflops, "peak": peaks["bf16_tflops"],
                             "unit": "TFLOP/s", "frac": tensor_frac})
        config = {"workload": workload_name(shape, T, world, args.skew),
                  "hidden": shape.hidden, "inter": shape.inter, "tokens_per_gpu": T,
                  "l2_policy": "inputs larger than L2 (expert weights and row buffers touched per step exceed 126 MB)"}
        if skew_info is not None:
            config["routing_skew"] = skew_info
        result = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config,
            "roofline": roofline,
            "e2e": {"value": tokens_total / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(h_in.numel() * 2), "d2h_bytes_per_step": int(h_out.numel() * 2),
                    "matches_device_path": bool(e2e_ok)},
            "gpu_launches": args.steps,
            "clocks": clocks,
            "parity": parity,
        }
        if world == 1 and not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline_leg(shape, gate, w13, w2, x)
    launcher.destroy()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
