"""Python face of the launcher: same class, methods and checks as the reference's
`flashMoeLauncher` torch extension (python/pyMoeLauncherTorch.cpp:33-133), bound to libflashMoe.so
through its C ABI instead of pybind11.

Differences that come with the B200 build: tensors are bf16 (the native path) or fp32 (converted at
the boundary), and the layer shape is taken from the tensor shapes instead of being compiled in.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib

_DTYPES = {torch.bfloat16: 0, torch.float32: 1}


def _check_tensor(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None) -> None:
    # reference: CHECK_TENSOR, python/pyMoeLauncherTorch.cpp:24-31
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"{name} tensor is undefined")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if t.dtype not in _DTYPES:
        raise RuntimeError(f"{name} must be bfloat16 or float32")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _stream_ptr() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class MoeKernelLauncher:
    """create / launch / destroy / valid / getDistributedUniqueId, as in the reference extension."""

    def __init__(self) -> None:
        self._h = C.c_void_p(None)
        self._dtype: Optional[torch.dtype] = None
        self._hidden = 0
        self._keep = None  # weights are borrowed by the library: keep them alive

    @staticmethod
    def getDistributedUniqueId(empty: bool = False) -> bytes:
        """128 bytes identifying a multi-rank job; zeros when empty=True
        (reference: pyMoeLauncherTorch.cpp:37-42)."""
        buf = (C.c_uint8 * 128)()
        _lib.check(_lib.lib().FlashMoeGetUniqueId(1 if empty else 0, buf), "GetDistributedUniqueId")
        return bytes(buf)

    @property
    def valid(self) -> bool:
        return bool(self._h.value)

    def create(self, gate_weights: torch.Tensor, ffn1_expert_weights: torch.Tensor,
               ffn2_expert_weights: torch.Tensor, max_tokens: int, uid: bytes, rank: int,
               world_size: int, topk: int = 8) -> None:
        """reference: pyMoeLauncherTorch.cpp:71-107 (same shape checks)."""
        if self.valid:
            raise RuntimeError("Launcher already created")
        _check_tensor(gate_weights, "gate_weights")
        _check_tensor(ffn1_expert_weights, "ffn1_expert_weights", gate_weights.dtype)
        _check_tensor(ffn2_expert_weights, "ffn2_expert_weights", gate_weights.dtype)
        if world_size <= 0:
            raise RuntimeError("worldSize must be positive")
        experts, hidden = gate_weights.shape
        inter = ffn2_expert_weights.shape[2]
        if tuple(ffn1_expert_weights.shape) != (experts // world_size, 2 * inter, hidden):
            raise RuntimeError("ffn1_expert_weights must be [experts/world, 2*inter, hidden]")
        if tuple(ffn2_expert_weights.shape) != (experts // world_size, hidden, inter):
            raise RuntimeError("ffn2_expert_weights must be [experts/world, hidden, inter]")
        if len(uid) != 128:
            raise RuntimeError("uid must be 128 bytes")
        cfg = _lib.FlashMoeConfig(hidden, inter, experts, topk, _DTYPES[gate_weights.dtype], (C.c_int32 * 3)())
        uid_buf = (C.c_uint8 * 128).from_buffer_copy(uid)
        h = C.c_void_p(None)
        code = _lib.lib().FlashMoeCreate(C.byref(h), gate_weights.data_ptr(), ffn1_expert_weights.data_ptr(),
                                         ffn2_expert_weights.data_ptr(), int(max_tokens), _stream_ptr(),
                                         uid_buf, int(rank), int(world_size), C.byref(cfg))
        _lib.check(code, "CreateLauncher")
        self._h = h
        self._dtype = gate_weights.dtype
        self._hidden = hidden
        self._keep = (gate_weights, ffn1_expert_weights, ffn2_expert_weights)

    def launch(self, tokens: torch.Tensor, output: torch.Tensor) -> None:
        """Asynchronous on the current torch stream; output may be the same tensor as tokens
        (reference: pyMoeLauncherTorch.cpp:44-61)."""
        if not self.valid:
            raise RuntimeError("Launcher was destroyed")
        _check_tensor(tokens, "tokens", self._dtype)
        _check_tensor(output, "output", self._dtype)
        if tokens.dim() != 2 or tokens.shape[1] != self._hidden or tuple(output.shape) != tuple(tokens.shape):
            raise RuntimeError("tokens and output must both be [tokens, hidden]")
        code = _lib.lib().FlashMoeLaunch(self._h, tokens.data_ptr(), output.data_ptr(), int(tokens.shape[0]),
                                         _stream_ptr())
        _lib.check(code, "Launch")

    def launch_host(self, tokens: torch.Tensor, output: torch.Tensor) -> None:
        """Host-buffer entry point: `tokens`/`output` are CPU tensors (pinned for an asynchronous call).
        `tokens` must be complete when the call is made; `output` is complete once the current stream
        has reached this point.  The library copies in, runs and copies out on internal streams, so
        calls made back to back overlap the copies of one with the kernel of the other."""
        if not self.valid:
            raise RuntimeError("Launcher was destroyed")
        if tokens.is_cuda or output.is_cuda or tokens.dtype != self._dtype or output.dtype != self._dtype:
            raise RuntimeError("launch_host takes CPU tensors of the launcher's dtype")
        if not (tokens.is_contiguous() and output.is_contiguous()) or tuple(tokens.shape) != tuple(output.shape):
            raise RuntimeError("tokens and output must be contiguous and of equal shape")
        code = _lib.lib().FlashMoeLaunchHost(self._h, tokens.data_ptr(), output.data_ptr(), int(tokens.shape[0]),
                                             _stream_ptr())
        _lib.check(code, "LaunchHost")

    def last_status(self):
        """(code, info) of the first device-side error, (0, 0) if none."""
        code, info = C.c_uint32(0), C.c_uint32(0)
        _lib.lib().FlashMoeGetLastStatus(self._h, C.byref(code), C.byref(info))
        return int(code.value), int(info.value)

    def destroy(self) -> None:
        """reference: pyMoeLauncherTorch.cpp:63-69."""
        if self.valid:
            h, self._h = self._h, C.c_void_p(None)
            self._keep = None
            _lib.check(_lib.lib().FlashMoeDestroy(h, _stream_ptr()), "DestroyLauncher")

    # -- parity-test access to the stage buffers of the last launch (FlashMoeDebugRead)
    def debug_read(self, which: int, nbytes: int, offset: int = 0) -> bytes:
        buf = (C.c_uint8 * nbytes)()
        _lib.check(_lib.lib().FlashMoeDebugRead(self._h, which, buf, offset, nbytes), "DebugRead")
        return bytes(buf)
