"""ctypes front end for the CPU checkers under oracle/.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
cpu_baseline / reference legs of bench.py.  The shipped package never imports it.

Two libraries, both built by oracle/Makefile:
  * `_build/libmoe_oracle.so`  - moe_oracle.c, the C restatement ("port");
  * `_ref/libref_moe.so`       - the reference project's own CPU headers compiled
                                 from their original location ("reference").  It is
                                 built only where the reference sources exist and
                                 then travels as a prebuilt file.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT = os.path.join(_HERE, "_build", "libmoe_oracle.so")
_REF = os.path.join(_HERE, "_ref", "libref_moe.so")

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


def build(ref_root: str = "/root/reference") -> None:
    """Compile the port, and the reference library when its sources are present."""
    # quiet on stdout: callers such as the benchmark print exactly one JSON line there
    subprocess.run(["make", "-s", "-C", _HERE, f"REF={ref_root}", "oracle", "ref"], check=True,
                   stdout=subprocess.DEVNULL)


def _ptr(a: Optional[np.ndarray], ty=C.c_float):
    if a is None:
        return C.cast(None, C.POINTER(ty))
    return a.ctypes.data_as(C.POINTER(ty))


class PortOracle:
    """moe_oracle.c through ctypes."""

    kind = "port"

    def __init__(self) -> None:
        if not os.path.exists(_PORT):
            build()
        self.lib = C.CDLL(_PORT)
        L = self.lib
        L.oracle_gemm_nt.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.oracle_topk_rows.argtypes = [_f32p, C.c_int, C.c_int, _f32p, _i32p, C.c_int]
        L.oracle_softmax_rows.argtypes = [_f32p, C.c_int, C.c_int]
        L.oracle_gate.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, _i32p,
                                  C.POINTER(C.c_float)]
        L.oracle_ffn1.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int, _f32p]
        L.oracle_full_moe.argtypes = [_f32p, _f32p, _f32p, _f32p] + [C.c_int] * 5 + [
            _f32p, C.POINTER(C.c_float), C.POINTER(C.c_int), C.POINTER(C.c_float),
            C.POINTER(C.c_float), C.c_int]
        _u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
        L.oracle_full_moe_bw.argtypes = [_f32p, _f32p, _u16p, _u16p] + [C.c_int] * 5 + [
            _f32p, C.POINTER(C.c_float), C.POINTER(C.c_int), C.c_int]
        L.oracle_rand_uniform_fill.argtypes = [_f32p, C.c_size_t, C.c_float, C.c_float, C.c_int]
        L.oracle_max_threads.restype = C.c_int

    def max_threads(self) -> int:
        return int(self.lib.oracle_max_threads())

    def gemm_nt(self, A: np.ndarray, B: np.ndarray) -> np.ndarray:
        M, K = A.shape
        N = B.shape[0]
        out = np.empty((M, N), np.float32)
        self.lib.oracle_gemm_nt(A, B, out, M, N, K)
        return out

    def topk_rows(self, x: np.ndarray, k: int):
        rows, cols = x.shape
        v = np.empty((rows, k), np.float32)
        i = np.empty((rows, k), np.int32)
        self.lib.oracle_topk_rows(x, rows, cols, v, i, k)
        return v, i

    def softmax_rows(self, x: np.ndarray) -> np.ndarray:
        y = np.ascontiguousarray(x, np.float32).copy()
        self.lib.oracle_softmax_rows(y, y.shape[0], y.shape[1])
        return y

    def gate(self, tokens: np.ndarray, gate_w: np.ndarray, topk: int, want_logits: bool = False):
        T, H = tokens.shape
        E = gate_w.shape[0]
        w = np.empty((T, topk), np.float32)
        idx = np.empty((T, topk), np.int32)
        logits = np.empty((T, E), np.float32) if want_logits else None
        self.lib.oracle_gate(tokens, gate_w, T, E, H, topk, w, idx, _ptr(logits))
        return (w, idx, logits) if want_logits else (w, idx)

    def ffn1(self, tokens: np.ndarray, w13_e: np.ndarray) -> np.ndarray:
        rows, H = tokens.shape
        I = w13_e.shape[0] // 2
        out = np.empty((rows, I), np.float32)
        self.lib.oracle_ffn1(tokens, w13_e, rows, H, I, out)
        return out

    def full_moe(self, tokens, gate_w, w13, w2, topk: int, threads: int = 1, stages: bool = False):
        """Returns out [T,H]; with stages=True also (topk_w, topk_idx, act[T,K,I], y[T,K,H])."""
        T, H = tokens.shape
        E = gate_w.shape[0]
        I = w2.shape[2]
        out = np.zeros((T, H), np.float32)
        if not stages:
            self.lib.oracle_full_moe(tokens, gate_w, w13, w2, T, E, H, topk, I, out,
                                     _ptr(None), _ptr(None, C.c_int), _ptr(None), _ptr(None), threads)
            return out
        tw = np.zeros((T, topk), np.float32)
        ti = np.zeros((T, topk), np.int32)
        act = np.zeros((T, topk, I), np.float32)
        y = np.zeros((T, topk, H), np.float32)
        self.lib.oracle_full_moe(tokens, gate_w, w13, w2, T, E, H, topk, I, out,
                                 _ptr(tw), _ptr(ti, C.c_int), _ptr(act), _ptr(y), threads)
        return out, tw, ti, act, y

    def full_moe_bf16_weights(self, tokens, gate_w, w13_bits, w2_bits, topk: int, threads: int = 1):
        """The layer with the expert weights given as bf16 bit patterns (uint16 arrays [E,2I,H] and
        [E,H,I], e.g. a memory map shared between processes).  Returns (out, topk_w, topk_idx); equal
        bit for bit to full_moe on the widened weights."""
        T, H = tokens.shape
        E = gate_w.shape[0]
        I = w2_bits.shape[2]
        out = np.zeros((T, H), np.float32)
        tw = np.zeros((T, topk), np.float32)
        ti = np.zeros((T, topk), np.int32)
        self.lib.oracle_full_moe_bw(tokens, gate_w, w13_bits, w2_bits, T, E, H, topk, I, out, _ptr(tw),
                                    _ptr(ti, C.c_int), threads)
        return out, tw, ti

    def rand_uniform(self, n: int, lo: float, hi: float, reseed: bool) -> np.ndarray:
        out = np.empty(n, np.float32)
        self.lib.oracle_rand_uniform_fill(out, n, lo, hi, int(reseed))
        return out


class RefOracle:
    """The reference project's own CPU MoE (oracle/_ref/libref_moe.so)."""

    kind = "reference"

    def __init__(self) -> None:
        if not os.path.exists(_REF):
            raise FileNotFoundError(_REF)
        self.lib = C.CDLL(_REF)
        L = self.lib
        L.ref_gemm_nt.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.ref_gate.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, _i32p]
        L.ref_ffn1.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int, _f32p]
        L.ref_full_moe.argtypes = [_f32p, _f32p, _f32p, _f32p] + [C.c_int] * 5 + [_f32p]
        L.ref_full_moe_mt.argtypes = [_f32p, _f32p, _f32p, _f32p] + [C.c_int] * 5 + [_f32p, C.c_int]
        L.ref_max_threads.restype = C.c_int

    @staticmethod
    def available() -> bool:
        return os.path.exists(_REF)

    def max_threads(self) -> int:
        return int(self.lib.ref_max_threads())

    def gemm_nt(self, A, B):
        M, K = A.shape
        N = B.shape[0]
        out = np.empty((M, N), np.float32)
        self.lib.ref_gemm_nt(A, B, out, M, N, K)
        return out

    def gate(self, tokens, gate_w, topk: int):
        T, H = tokens.shape
        E = gate_w.shape[0]
        w = np.empty((T, topk), np.float32)
        idx = np.empty((T, topk), np.int32)
        self.lib.ref_gate(tokens, gate_w, T, E, H, topk, w, idx)
        return w, idx

    def ffn1(self, tokens, w13_e):
        rows, H = tokens.shape
        I = w13_e.shape[0] // 2
        out = np.empty((rows, I), np.float32)
        self.lib.ref_ffn1(tokens, w13_e, rows, H, I, out)
        return out

    def full_moe(self, tokens, gate_w, w13, w2, topk: int, threads: int = 1):
        T, H = tokens.shape
        E = gate_w.shape[0]
        I = w2.shape[2]
        out = np.zeros((T, H), np.float32)
        if threads <= 1:
            self.lib.ref_full_moe(tokens, gate_w, w13, w2, T, E, H, topk, I, out)
        else:
            self.lib.ref_full_moe_mt(tokens, gate_w, w13, w2, T, E, H, topk, I, out, threads)
        return out


def best_oracle():
    """The reference build when present, else the port."""
    return RefOracle() if RefOracle.available() else PortOracle()
