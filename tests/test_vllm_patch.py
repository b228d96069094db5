"""The vLLM patch (twin of the reference's test/multiGPU/python/flash_moe_patch.py): the wrapper class
around a block with vLLM's attribute layout, and the mechanism that applies the patch in every process
of a job (a sitecustomize.py on PYTHONPATH plus an import hook)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import moe_testlib as tl
from moe_testlib import cpu_oracle, synth
from flash_distributed_moe_b200 import vllm_patch


def _vllm_importable():
    try:
        import importlib.util
        return importlib.util.find_spec("vllm") is not None
    except Exception:
        return False


@pytest.mark.skipif(not _vllm_importable(), reason="vLLM is not installed")
def test_patch_reaches_a_freshly_started_process():
    # a process started after enable_flash_moe_patching() (as vLLM's spawned workers are) gets the
    # wrapper class as soon as it imports vLLM's qwen3_moe module
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "from flash_distributed_moe_b200.vllm_patch import enable_flash_moe_patching\n"
        "import os, subprocess\n"
        "os.environ.pop('FLASH_MOE_ENABLED', None)\n"
        "import vllm.model_executor.models.qwen3_moe as q0\n"
        "assert not getattr(q0.Qwen3MoeSparseMoeBlock, '_flash_moe_wrapper', False)\n"
        "enable_flash_moe_patching()\n"
        "assert q0.Qwen3MoeSparseMoeBlock._flash_moe_wrapper\n"
        "child = 'import vllm.model_executor.models.qwen3_moe as q; "
        "print(\"CHILD\", getattr(q.Qwen3MoeSparseMoeBlock, \"_flash_moe_wrapper\", False), "
        "q.Qwen3MoeSparseMoeBlock.__mro__[1].__name__)'\n"
        "print(subprocess.run([sys.executable, '-c', child], capture_output=True, text=True).stdout)\n"
    ) % tl.ROOT
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    assert "CHILD True Qwen3MoeSparseMoeBlock" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_checking_mode_records_row_distances(tmp_path, monkeypatch):
    # FLASH_MOE_VERIFY=1: one JSON line per call with the rows beyond the relative distance of 2e-2
    import json
    monkeypatch.setenv("FLASH_MOE_VERIFY_LOG", str(tmp_path / "calls"))
    theirs = torch.randn(6, 32)
    ours = theirs.clone()
    ours[1] *= 1.5      # far
    ours[4] += 1e-4     # near
    vllm_patch.record_row_distances(ours.to(torch.bfloat16).float(), theirs)
    vllm_patch.record_row_distances(theirs[:0], theirs[:0])  # empty calls leave no line
    lines = [json.loads(x) for x in open(f"{tmp_path / 'calls'}.{os.getpid()}")]
    assert len(lines) == 1 and lines[0]["rows"] == 6 and lines[0]["rows_beyond"] == 1
    assert 0.4 < lines[0]["max"] < 0.6 and lines[0]["median"] < vllm_patch.VERIFY_ROW_TOLERANCE


class _Experts(torch.nn.Module):
    def __init__(self, w13, w2):
        super().__init__()
        self.w13_weight = torch.nn.Parameter(w13, requires_grad=False)
        self.w2_weight = torch.nn.Parameter(w2, requires_grad=False)


class _Cfg:
    """The two attributes of vLLM's config object the wrapper reads."""

    def __init__(self, topk):
        self.model_config = type("M", (), {"hf_text_config": type("H", (), {"num_experts_per_tok": topk})()})()


class _FakeBlock(torch.nn.Module):
    """Stand-in with the attribute layout of vLLM's Qwen3MoeSparseMoeBlock on one rank."""
    weights = None

    def __init__(self, vllm_config, prefix=""):
        super().__init__()
        gate, w13, w2 = _FakeBlock.weights
        self.gate = torch.nn.Linear(gate.shape[1], gate.shape[0], bias=False, dtype=gate.dtype, device=gate.device)
        self.gate.weight = torch.nn.Parameter(gate, requires_grad=False)
        self.experts = _Experts(w13, w2)
        self.ep_group, self.ep_rank, self.ep_size = None, 0, 1
        self.fallback_calls = 0

    def forward(self, hidden_states):
        self.fallback_calls += 1
        return hidden_states


@pytest.mark.gpu
def test_wrapper_class_runs_the_layer_in_place_and_falls_back_above_max_tokens(monkeypatch):
    s = synth.TINY
    gate, w13, w2 = synth.make_weights(s, std=0.05)
    _FakeBlock.weights = (gate.cuda(), w13.cuda(), w2.cuda())
    monkeypatch.setenv("FLASH_MOE_MAX_TOKENS", "64")
    wrapper = vllm_patch.make_wrapper_class(_FakeBlock)(_Cfg(s.topk))
    port = cpu_oracle.PortOracle()
    for batch in (1, 16, 64):
        x = synth.make_tokens(s, batch, seed=40 + batch)
        hidden = x.cuda()
        got = wrapper(hidden)
        torch.cuda.synchronize()
        assert got.data_ptr() == hidden.data_ptr()
        ref = port.full_moe(tl.f32(x), tl.f32(gate), tl.f32(w13), tl.f32(w2), s.topk)
        tl.assert_close_bf16(tl.f32(got.cpu()), ref, f"wrapper, batch {batch}")
    assert wrapper.fallback_calls == 0
    wrapper(synth.make_tokens(s, 65).cuda())  # more tokens than the launcher takes: vLLM's own block
    assert wrapper.fallback_calls == 1
    wrapper.launcher.destroy()
    wrapper.launcher = None


def test_harness_checkpoint_is_a_loadable_qwen3_moe_model(tmp_path):
    # the seeded one-layer checkpoint the vLLM harness writes: a Hugging Face Qwen3-MoE model that loads
    # without missing weights and whose greedy next token is well defined (no tied logits)
    transformers = pytest.importorskip("transformers")
    import vllm_dp_harness as harness
    path = harness.make_model_dir(str(tmp_path / "model"))
    model, info = transformers.AutoModelForCausalLM.from_pretrained(path, dtype=torch.bfloat16, output_loading_info=True)
    assert not info["missing_keys"] and not info["unexpected_keys"], info
    assert model.config.num_experts == harness.EXPERTS and model.config.num_experts_per_tok == harness.TOPK
    ids = torch.from_numpy(np.random.RandomState(0).randint(3, harness.VOCAB, size=(4, 16)))
    with torch.no_grad():
        logits = model(ids).logits[:, -1].float()
    assert torch.isfinite(logits).all()
    best = logits.topk(2, dim=-1).values
    assert ((best[:, 0] - best[:, 1]) > 0).all()


def test_oracle_equals_the_hugging_face_qwen3_moe_block(tmp_path):
    # The layer the launcher replaces, as the model library itself computes it (transformers'
    # Qwen3MoeSparseMoeBlock, fp32, CPU) against the CPU oracle on the harness's checkpoint: pins the
    # meaning of the weight layout (gate projection in rows 0..I-1 of w13) and of the routing weights
    # (softmax renormalised over the selected experts) at the boundary where the operator is dropped in.
    transformers = pytest.importorskip("transformers")
    from safetensors.torch import load_file
    import vllm_dp_harness as harness
    path = harness.make_model_dir(str(tmp_path / "model"))
    model = transformers.AutoModelForCausalLM.from_pretrained(path, dtype=torch.float32)
    block = model.model.layers[0].mlp
    x = torch.randn(40, harness.HIDDEN, generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        y = block(x.unsqueeze(0))
    y = (y[0] if isinstance(y, tuple) else y).reshape(40, harness.HIDDEN)
    t = load_file(os.path.join(path, "model.safetensors"))
    p = "model.layers.0.mlp."
    gate = t[p + "gate.weight"].float()
    w13 = torch.stack([torch.cat([t[p + f"experts.{e}.gate_proj.weight"], t[p + f"experts.{e}.up_proj.weight"]], 0)
                       for e in range(harness.EXPERTS)]).float()
    w2 = torch.stack([t[p + f"experts.{e}.down_proj.weight"] for e in range(harness.EXPERTS)]).float()
    cpu_oracle.build()
    ref = cpu_oracle.PortOracle().full_moe(tl.f32(x), tl.f32(gate), tl.f32(w13), tl.f32(w2), harness.TOPK)
    np.testing.assert_allclose(y.numpy(), ref, atol=1e-4, rtol=1e-4)
