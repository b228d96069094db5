"""vLLM integration: routes vLLM's Qwen3 MoE block through the launcher, with data parallelism and
expert parallelism (one process per GPU).

Twin of the reference's test/multiGPU/python/flash_moe_patch.py:35-114,300-346: a subclass of
`vllm.model_executor.models.qwen3_moe.Qwen3MoeSparseMoeBlock` replaces the original class, in every
process of a vLLM job, through a `sitecustomize.py` on PYTHONPATH that takes effect when the
environment variable FLASH_MOE_ENABLED=1 is set.  Differences from the reference's patch:

  * the wrapper also serves expert-parallel jobs (`ep_size > 1`): the reference falls back to vLLM's
    own block there (flash_moe_patch.py:104), this kernel dispatches rows to the experts' owners
    itself.  The unique id travels over `torch.distributed.broadcast_object_list` in the EP group,
    as in the reference (flash_moe_patch.py:73-87);
  * the launcher is created at the first forward call, when the weights have been loaded.  It needs
    the expert weights in vLLM's canonical layout `[experts/ep, 2*inter, hidden]` (gate projection
    rows first) and `[experts/ep, hidden, inter]`, bf16 or fp32.  vLLM's weight post-processing may
    re-block them for its own kernels (on B200, vLLM 0.22 turns `[32, 256, 256]` into
    `[32, 4, 256, 64]`), so the patch keeps a copy in the canonical layout, taken just before that
    step, while leaving the step itself alone (the reference turns it into a no-op, which would
    break vLLM's own path for batches above the token bound);
  * `FLASH_MOE_MAX_TOKENS` (default 8192) bounds the tokens per call that go through the kernel;
    larger batches use vLLM's block, like the reference's `num_tokens < maxTokens` test;
  * `FLASH_MOE_VERIFY=1` (a checking mode, not for production: it runs both implementations and
    synchronises) makes every call also run vLLM's own block on a copy of the input and appends one
    JSON line per call to the file `$FLASH_MOE_VERIFY_LOG.<pid>`: rows, rows whose relative L2 distance
    to vLLM's result exceeds 2e-2, and the largest and the median of those distances.

With expert parallelism every forward call is collective over the EP group: vLLM's data-parallel
engines already run in lockstep for their own all-to-all (idle ranks run dummy batches).

    from flash_distributed_moe_b200.vllm_patch import enable_flash_moe_patching
    enable_flash_moe_patching()      # before the engine (and its worker processes) is created
"""
from __future__ import annotations

import atexit
import os
import shutil
import sys
import tempfile

_PATCHED = False
_SITECUSTOMIZE_DIR = None
_PKG_PARENT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def make_wrapper_class(base):
    """Subclass of vLLM's `Qwen3MoeSparseMoeBlock` (passed in as `base`) that runs the layer in place
    through the launcher (reference: flash_moe_patch.py:42-112)."""
    import torch
    import torch.distributed as dist

    from .flashMoeLauncher import MoeKernelLauncher

    class FlashMoeWrapper(base):
        def __init__(self, vllm_config, prefix: str = ""):
            super().__init__(vllm_config, prefix)
            self.maxTokens = int(os.environ.get("FLASH_MOE_MAX_TOKENS", "8192"))
            self.launcher = None
            self._flash_moe_topk = int(vllm_config.model_config.hf_text_config.num_experts_per_tok)
            self._flash_moe_verify = os.environ.get("FLASH_MOE_VERIFY", "0") == "1"

        def _create_launcher(self) -> None:
            gate_w = self.gate.weight
            w13 = getattr(self.experts, "_flash_moe_w13", None)
            w2 = getattr(self.experts, "_flash_moe_w2", None)
            if w13 is None or w2 is None:
                w13, w2 = self.experts.w13_weight, self.experts.w2_weight
            experts, hidden = gate_w.shape
            inter = w2.shape[2]
            if (tuple(w13.shape) != (experts // self.ep_size, 2 * inter, hidden) or not w13.is_contiguous()
                    or not w2.is_contiguous()):
                raise RuntimeError("FlashMoeWrapper: expert weights are not in vLLM's canonical layout "
                                   f"(w13 {tuple(w13.shape)}, w2 {tuple(w2.shape)})")
            launcher = MoeKernelLauncher()
            if self.ep_size == 1:
                uid = launcher.getDistributedUniqueId(empty=True)
                launcher.create(gate_w, w13, w2, self.maxTokens, uid, 0, 1, topk=self._flash_moe_topk)
            else:
                box = [launcher.getDistributedUniqueId() if self.ep_rank == 0 else None]
                dist.broadcast_object_list(box, src=dist.get_process_group_ranks(self.ep_group)[0],
                                           group=self.ep_group)
                launcher.create(gate_w, w13, w2, self.maxTokens, box[0], self.ep_rank, self.ep_size,
                                topk=self._flash_moe_topk)
            self.launcher = launcher

        def __del__(self):
            try:
                if self.launcher is not None:
                    self.launcher.destroy()
            except Exception:
                pass

        def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
            if hidden_states.dim() != 2 or hidden_states.shape[0] > self.maxTokens:
                return super().forward(hidden_states)
            if self.launcher is None:
                self._create_launcher()
            tokens = hidden_states if hidden_states.is_contiguous() else hidden_states.contiguous()
            theirs = super().forward(tokens.clone()) if self._flash_moe_verify else None
            self.launcher.launch(tokens, tokens)  # in place: output memory = input memory
            if theirs is not None:
                record_row_distances(tokens, theirs.reshape(tokens.shape))
            return tokens

    return FlashMoeWrapper


VERIFY_ROW_TOLERANCE = 2e-2


def row_distances(ours, theirs):
    """Relative L2 distance of every row of `ours` to the same row of `theirs` (fp32, 1-D tensor)."""
    a, b = ours.float(), theirs.float()
    return (a - b).norm(dim=1) / b.norm(dim=1).clamp_min(1e-12)


def record_row_distances(ours, theirs) -> None:
    """Appends one JSON line about this call to `$FLASH_MOE_VERIFY_LOG.<pid>` (checking mode)."""
    import json
    path = os.environ.get("FLASH_MOE_VERIFY_LOG", "")
    if not path or ours.shape[0] == 0:
        return
    d = row_distances(ours, theirs)
    line = {"rows": int(d.numel()), "rows_beyond": int((d > VERIFY_ROW_TOLERANCE).sum().item()),
            "max": float(d.max().item()), "median": float(d.median().item())}
    with open(f"{path}.{os.getpid()}", "a") as f:
        f.write(json.dumps(line) + "\n")


def apply_flash_moe_patch() -> bool:
    """Replaces vLLM's block class in this process (idempotent).  Returns whether the patch is active."""
    global _PATCHED
    if _PATCHED:
        return True
    try:
        import vllm.model_executor.models.qwen3_moe as qwen3_moe
    except ImportError as e:
        print(f"[PID {os.getpid()}] FlashMoE patch not applied: {e}")
        return False
    if not getattr(qwen3_moe.Qwen3MoeSparseMoeBlock, "_flash_moe_wrapper", False):
        wrapper = make_wrapper_class(qwen3_moe.Qwen3MoeSparseMoeBlock)
        wrapper._flash_moe_wrapper = True
        qwen3_moe.Qwen3MoeSparseMoeBlock = wrapper
    try:
        # keep the expert weights in their canonical layout before vLLM re-blocks them
        from vllm.model_executor.layers.fused_moe import UnquantizedFusedMoEMethod as method
        if not getattr(method.process_weights_after_loading, "_flash_moe_wrapped", False):
            original = method.process_weights_after_loading

            def process_weights_after_loading(self, layer):
                if hasattr(layer, "w13_weight") and hasattr(layer, "w2_weight"):
                    layer._flash_moe_w13 = layer.w13_weight.data.clone().contiguous()
                    layer._flash_moe_w2 = layer.w2_weight.data.clone().contiguous()
                return original(self, layer)

            process_weights_after_loading._flash_moe_wrapped = True
            method.process_weights_after_loading = process_weights_after_loading
    except Exception as e:
        print(f"[PID {os.getpid()}] FlashMoE patch: expert weights are not copied before post-processing: {e}")
    _PATCHED = True
    return True


# Executed at interpreter start-up in every process whose PYTHONPATH holds the directory this text is
# written to (reference: flash_moe_patch.py:156-286).
_SITECUSTOMIZE_CODE = '''
import os, sys
if os.environ.get("FLASH_MOE_ENABLED", "0") == "1":
    _parent = os.environ.get("FLASH_MOE_PACKAGE_PARENT", "")
    if _parent and _parent not in sys.path:
        sys.path.insert(0, _parent)

    class _PatchingLoader:
        """Runs the module's own loader, then applies the patch to the freshly executed module."""

        def __init__(self, real):
            self._real = real

        def create_module(self, spec):
            return self._real.create_module(spec)

        def exec_module(self, module):
            self._real.exec_module(module)
            try:
                from flash_distributed_moe_b200.vllm_patch import apply_flash_moe_patch
                apply_flash_moe_patch()
            except Exception as e:  # never break the host process
                print(f"[PID {os.getpid()}] FlashMoE patch failed: {e}")

    class _FlashMoeImportHook:
        """Wraps the loader of vLLM's qwen3_moe module so that the patch is applied as soon as the
        module has been executed."""
        _name = "vllm.model_executor.models.qwen3_moe"

        def find_spec(self, fullname, path=None, target=None):
            if fullname != self._name:
                return None
            for finder in sys.meta_path:
                if finder is self or not hasattr(finder, "find_spec"):
                    continue
                spec = finder.find_spec(fullname, path, target)
                if spec is not None and spec.loader is not None:
                    spec.loader = _PatchingLoader(spec.loader)
                    return spec
            return None

    if not any(type(h).__name__ == "_FlashMoeImportHook" for h in sys.meta_path):
        sys.meta_path.insert(0, _FlashMoeImportHook())
'''


def _cleanup() -> None:
    global _SITECUSTOMIZE_DIR
    if _SITECUSTOMIZE_DIR and os.path.exists(_SITECUSTOMIZE_DIR):
        shutil.rmtree(_SITECUSTOMIZE_DIR, ignore_errors=True)
    _SITECUSTOMIZE_DIR = None


def enable_flash_moe_patching() -> None:
    """Enables the patch for this process and for every process started from it (vLLM's workers are
    spawned and do not inherit monkey patches): sets FLASH_MOE_ENABLED=1 and puts a directory with a
    `sitecustomize.py` in front of PYTHONPATH (reference: flash_moe_patch.py:300-346)."""
    global _SITECUSTOMIZE_DIR
    os.environ["FLASH_MOE_ENABLED"] = "1"
    os.environ["FLASH_MOE_PACKAGE_PARENT"] = _PKG_PARENT
    if _SITECUSTOMIZE_DIR is None:
        _SITECUSTOMIZE_DIR = tempfile.mkdtemp(prefix="flash_moe_patch_")
        with open(os.path.join(_SITECUSTOMIZE_DIR, "sitecustomize.py"), "w") as f:
            f.write(_SITECUSTOMIZE_CODE)
        atexit.register(_cleanup)
    path = os.environ.get("PYTHONPATH", "")
    if _SITECUSTOMIZE_DIR not in path.split(os.pathsep):
        os.environ["PYTHONPATH"] = _SITECUSTOMIZE_DIR + (os.pathsep + path if path else "")
    apply_flash_moe_patch()


def disable_flash_moe_patching() -> None:
    """Processes started from now on are not patched (reference: flash_moe_patch.py:349-358)."""
    os.environ["FLASH_MOE_ENABLED"] = "0"
