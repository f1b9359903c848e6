"""ctypes front end of the CPU oracle (oracle/rwkv_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline legs.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Dict, List, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liborc.so")
_lib: Optional[ctypes.CDLL] = None


def build(force: bool = False) -> str:
    """Compile rwkv_oracle.c -> liborc.so (gcc, OpenMP, AVX2 baseline so the file runs on any x86-64-v3 host)."""
    src = os.path.join(_HERE, "rwkv_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-o", _LIB_PATH,
                               src, "-lm"])
    return _LIB_PATH


class _Cfg(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in
                ("version", "n_layer", "n_embd", "n_ffn", "n_head", "vocab", "rescale_every", "state_fp16", "gate_from_xx")]


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        L.orc_state_floats.restype = ctypes.c_size_t
        L.orc_state_floats.argtypes = [ctypes.POINTER(_Cfg)]
        L.orc_state_reset.argtypes = [ctypes.POINTER(_Cfg), ctypes.c_void_p]
        L.orc_forward.restype = ctypes.c_int
        L.orc_forward.argtypes = [ctypes.POINTER(_Cfg), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                  ctypes.c_int, ctypes.c_void_p]
        L.orc_num_threads.restype = ctypes.c_int
        L.orc_set_threads.argtypes = [ctypes.c_int]
        L.orc_quant_int8.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        L.orc_quant_int4.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        L.orc_dequant_int8.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        L.orc_dequant_int4.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        L.orc_wkv4_step.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 9
        L.orc_wkv5_step.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 7
        L.orc_layernorm.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        L.orc_f32_to_f16.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
        L.orc_f16_to_f32.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
        _lib = L
    return _lib


def _version_code(version: str) -> int:
    return {"4": 4, "5": 50, "5.1": 51, "5.2": 52}[str(version)]


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


# ------------------------------------------------------------------ quantisers

def quant_int8(W: np.ndarray):
    """W [K,N] fp32 -> (q int8 [N,K], scales fp16 [N])."""
    W = np.ascontiguousarray(W, np.float32)
    K, N = W.shape
    q = np.empty((N, K), np.int8)
    s = np.empty(N, np.uint16)
    lib().orc_quant_int8(_ptr(W), K, N, _ptr(q), _ptr(s))
    return q, s.view(np.float16)


def quant_int4(W: np.ndarray):
    """W [K,N] fp32 -> (packed uint8 [N,K/2], scales fp16 [N,K/32])."""
    W = np.ascontiguousarray(W, np.float32)
    K, N = W.shape
    assert K % 32 == 0
    p = np.empty((N, K // 2), np.uint8)
    s = np.empty((N, K // 32), np.uint16)
    lib().orc_quant_int4(_ptr(W), K, N, _ptr(p), _ptr(s))
    return p, s.view(np.float16)


def dequant_int8(q: np.ndarray, s: np.ndarray) -> np.ndarray:
    N, K = q.shape
    W = np.empty((K, N), np.float32)
    q = np.ascontiguousarray(q)
    s = np.ascontiguousarray(s.view(np.uint16))
    lib().orc_dequant_int8(_ptr(q), _ptr(s), K, N, _ptr(W))
    return W


def dequant_int4(p: np.ndarray, s: np.ndarray) -> np.ndarray:
    N, K2 = p.shape
    K = K2 * 2
    W = np.empty((K, N), np.float32)
    p = np.ascontiguousarray(p)
    s = np.ascontiguousarray(s.view(np.uint16))
    lib().orc_dequant_int4(_ptr(p), _ptr(s), K, N, _ptr(W))
    return W


def fake_quant(W: np.ndarray, fmt: str) -> np.ndarray:
    """Quantise + dequantise a [K,N] matrix: what a quantised strategy actually multiplies by."""
    if fmt == "int8":
        return dequant_int8(*quant_int8(W))
    if fmt == "int4":
        return dequant_int4(*quant_int4(W))
    return np.asarray(W, np.float32)


# ------------------------------------------------------------------ single formulas (per-kernel tests)

def _f32(a):
    return np.ascontiguousarray(a, np.float32)


def layernorm(x, g, b) -> np.ndarray:
    """LayerNorm of every row of x [rows, n] (eps 1e-5)."""
    x = _f32(np.atleast_2d(x))
    g, b = _f32(g), _f32(b)
    y = np.empty_like(x)
    for i in range(x.shape[0]):
        lib().orc_layernorm(_ptr(x[i]), _ptr(g), _ptr(b), x.shape[1], _ptr(y[i]))
    return y


def wkv4_step(k, v, r, decay, first, aa, bb, pp):
    """One RWKV-4 WKV step; returns (sigmoid(r) * wkv, aa', bb', pp')."""
    k, v, r, decay, first = map(_f32, (k, v, r, decay, first))
    aa, bb, pp = _f32(aa).copy(), _f32(bb).copy(), _f32(pp).copy()
    out = np.empty_like(k)
    lib().orc_wkv4_step(len(k), _ptr(k), _ptr(v), _ptr(r), _ptr(decay), _ptr(first), _ptr(aa), _ptr(bb), _ptr(pp), _ptr(out))
    return out, aa, bb, pp


def wkv5_step(r, k, v, decay, first, s, per_head: bool):
    """One RWKV-5 state step over s [H, S, S]; returns (readout before GroupNorm [H * S], s')."""
    r, k, v, decay, first = map(_f32, (r, k, v, decay, first))
    s = _f32(s).copy()
    H, S = s.shape[0], s.shape[1]
    out = np.empty(H * S, np.float32)
    lib().orc_wkv5_step(H, S, int(per_head), _ptr(r), _ptr(k), _ptr(v), _ptr(decay), _ptr(first), _ptr(s), _ptr(out))
    return out, s


# ------------------------------------------------------------------ model

MATRIX_SUFFIXES = ("key.weight", "value.weight", "receptance.weight", "gate.weight", "output.weight", "head.weight")


class OracleModel:
    """fp32 forward over a dict of reference-named tensors (any float dtype; converted to fp32).

    rescale_every=6 reproduces the fp16 strategy's x /= 2 every 6 layers
    (kernels/default/model_forward.cpp:173-175) for files whose weights were pre-divided.
    state_fp16=True stores the token-shift states rounded to fp16, as the "cuda fp16" strategy does
    (its state tensors have the activation dtype, model.cpp:149-151).
    gate_from_xx=True reproduces kernels/default/att.cpp:101 (RWKV-5.1/5.2 gate fed by xx); the default
    follows the CUDA path (kernels/cuda/att.cu:289, gate fed by the mixed gx).
    weight_format "int8" / "int4" replaces every projection matrix and the head by its
    quantise->dequantise image, which is what the quantised strategies multiply by.
    """

    def __init__(self, shape, tensors: Dict[str, np.ndarray], param_order: List[str], rescale_every: int = 0,
                 weight_format: str = "fp16", state_fp16: bool = False, gate_from_xx: bool = False):
        self.shape = shape
        self.cfg = _Cfg(_version_code(shape.version), shape.n_layer, shape.n_embd, shape.n_ffn, shape.n_head,
                        shape.vocab, rescale_every, int(state_fp16), int(gate_from_xx))
        self._keep = []
        for name in param_order:
            a = np.ascontiguousarray(tensors[name], dtype=np.float32)
            if a.ndim == 2 and name.endswith(MATRIX_SUFFIXES) and weight_format in ("int8", "int4"):
                a = fake_quant(a, weight_format)
            self._keep.append(np.ascontiguousarray(a.reshape(-1) if a.ndim != 2 else a))
        self._params = (ctypes.c_void_p * len(self._keep))(*[_ptr(a) for a in self._keep])
        self.emb = np.ascontiguousarray(tensors["emb.weight"], dtype=np.float32)
        self.state = np.empty(lib().orc_state_floats(ctypes.byref(self.cfg)), np.float32)
        self.reset()

    def reset(self) -> None:
        lib().orc_state_reset(ctypes.byref(self.cfg), _ptr(self.state))

    def run(self, token_id: int) -> np.ndarray:
        logits = np.empty(self.shape.vocab, np.float32)
        rc = lib().orc_forward(ctypes.byref(self.cfg), self._params, _ptr(self.emb), _ptr(self.state),
                               int(token_id), _ptr(logits))
        if rc != 0:
            raise ValueError(f"token id {token_id} out of range")
        return logits

    def advance(self, token_id: int) -> None:
        """One token without the head: only the state moves (what a prompt token before the last one needs)."""
        rc = lib().orc_forward(ctypes.byref(self.cfg), self._params, _ptr(self.emb), _ptr(self.state),
                               int(token_id), None)
        if rc != 0:
            raise ValueError(f"token id {token_id} out of range")

    def run_seq(self, ids) -> np.ndarray:
        """Seq mode = token loop (kernels/default/model_forward_seq.cpp:34-46); returns the last logits."""
        ids = list(ids)
        for t in ids[:-1]:
            self.advance(int(t))
        return self.run(int(ids[-1]))

    # state accessors in the reference's layout (model.cpp:145-177)
    def state_v4(self) -> np.ndarray:
        return self.state.reshape(self.shape.n_layer, 5, self.shape.n_embd)
