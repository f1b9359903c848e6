"""Host-side mirror of the reference's model API over the fr_b200 C ABI.

`Model(path, strategy)` follows rwkv::Model (model.h:14-54, model.cpp:23-208) and the reference's
Python binding (python/fr_python.cpp:49-60): strategy strings "cuda fp16" / "cuda int8" /
"cuda int4" (model.cpp:25-60), `run(id | ids)` returning fp32 logits on the host, `reset_states()`,
`states()`, `save_state_file()` / `load_state_file()`.  All GPU work goes through
csrc/libfr_b200.so (include/fr_b200.h); there is no CPU fallback — without the library or a B200
every call raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Iterable, List, Optional, Sequence, Union

import numpy as np

from . import shard  # noqa: F401  (re-exported: stream partitioning across ranks)
from . import synth  # noqa: F401  (re-exported: synthetic `.fr` generator)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FR_B200_LIB") or os.path.join(_HERE, "csrc", "libfr_b200.so")

W_FP16, W_INT8, W_INT4 = 0, 1, 2
T_F16, T_F32 = 0, 1
_VERSIONS = {"4": 4, "5": 50, "5.0": 50, "5.1": 51, "5.2": 52}
_FORMATS = {"fp16": W_FP16, "int8": W_INT8, "int4": W_INT4}


class FrB200Error(RuntimeError):
    """A C-ABI call returned a negative status (the reference throws FRException, check.h:11-48)."""

    def __init__(self, status: int, what: str, detail: str):
        super().__init__(f"{what}: {detail}" if detail else what)
        self.status = status


class Config(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in
                ("version", "n_layer", "n_embd", "n_ffn", "n_head", "vocab", "weight_format", "act_fp16",
                 "max_batch", "device", "host_visible_state")]


class Info(ctypes.Structure):
    _fields_ = [("n_ctas", ctypes.c_int), ("n_threads", ctypes.c_int), ("smem_bytes", ctypes.c_int),
                ("n_stages", ctypes.c_int), ("stage_bytes", ctypes.c_int), ("n_phases", ctypes.c_int),
                ("weight_stream_bytes", ctypes.c_longlong), ("launches", ctypes.c_longlong)]


_lib: Optional[ctypes.CDLL] = None

# name -> (restype, argtypes); every symbol include/fr_b200.h declares
_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
SIGNATURES = {
    "fr_b200_create": (_i, [ctypes.POINTER(Config), ctypes.POINTER(_vp)]),
    "fr_b200_set_tensor": (_i, [_vp, ctypes.c_char_p, _vp, _i, ctypes.POINTER(ctypes.c_int64), _i]),
    "fr_b200_finalize": (_i, [_vp]),
    "fr_b200_destroy": (None, [_vp]),
    "fr_b200_save_packed": (_i, [_vp, ctypes.c_char_p]),
    "fr_b200_load_packed": (_i, [ctypes.c_char_p, _i, _i, _i, ctypes.POINTER(_vp)]),
    "fr_b200_get_config": (_i, [_vp, ctypes.POINTER(Config)]),
    "fr_b200_decode": (_i, [_vp, _vp, _i, _vp, _vp, _vp]),
    "fr_b200_decode_greedy": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "fr_b200_logits_device": (_i, [_vp, ctypes.POINTER(_vp)]),
    "fr_b200_logits_add": (_i, [_vp, _i, _vp, _vp, _vp, _vp]),
    "fr_b200_sample": (_i, [_vp, _i, ctypes.c_float, _i, ctypes.c_float, _vp, _vp, _vp]),
    "fr_b200_vocab_padded": (_i, [_vp]),
    "fr_b200_run_seq": (_i, [_vp, _i, _vp, _i, _vp, _vp]),
    "fr_b200_state_reset": (_i, [_vp, _i]),
    "fr_b200_state_count": (_i, [_vp]),
    "fr_b200_state_tensor": (_i, [_vp, _i, _i, _i, ctypes.POINTER(_vp), ctypes.POINTER(_i),
                                  ctypes.POINTER(ctypes.c_int64)]),
    "fr_b200_state_export": (_i, [_vp, _i, _vp, _sz]),
    "fr_b200_state_import": (_i, [_vp, _i, _vp, _sz]),
    "fr_b200_state_bytes": (_sz, [_vp]),
    "fr_b200_quantize_int8": (_i, [_vp, _i, _i, _vp, _vp, _i]),
    "fr_b200_quantize_int4": (_i, [_vp, _i, _i, _vp, _vp, _i]),
    "fr_b200_dequantize_int8": (_i, [_vp, _vp, _i, _i, _vp, _i]),
    "fr_b200_dequantize_int4": (_i, [_vp, _vp, _i, _i, _vp, _i]),
    "fr_b200_unpack_matrix": (_i, [_vp, ctypes.c_char_p, _vp, _i, _i]),
    "fr_b200_matvec": (_i, [_vp, _i, _i, _i, _vp, _i, _vp, _i]),
    "fr_b200_gemm_f16": (_i, [_vp, _vp, _i, _i, _i, _i, _vp, _vp, ctypes.c_float, _vp, _i]),
    "fr_b200_matvec_noalloc": (_i, [_vp, _i, _i, _i, _vp, _i, _vp, _i, _vp]),
    "fr_b200_noalloc_last_error": (ctypes.c_char_p, []),
    "fr_b200_get_info": (_i, [_vp, ctypes.POINTER(Info)]),
    "fr_b200_decode_profile": (_i, [_vp, _vp, _i, _vp, _i]),
    "fr_b200_wait_selftest": (_i, [_i, ctypes.c_uint]),
    "fr_b200_ln_mix": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "fr_b200_wkv4_step": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "fr_b200_wkv5_step": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp]),
    "fr_b200_wkv5_chunk_scan": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _vp, _vp]),
    "fr_b200_groupnorm": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "fr_b200_elementwise": (_i, [_i, _vp, _i, _vp, _i, _vp, _i, ctypes.c_float, _vp, _i, _sz, _vp]),
    "fr_b200_matmul": (_i, [_vp, _i, _i, _i, _vp, _i, _i, _vp, _i, _i, _vp]),
    "fr_b200_op_last_error": (ctypes.c_char_p, []),
    "fr_b200_strerror": (ctypes.c_char_p, [_i]),
    "fr_b200_last_error": (ctypes.c_char_p, []),
}


def lib() -> ctypes.CDLL:
    """Load csrc/libfr_b200.so.  Raises if it was not built: there is no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FrB200Error(-100, "libfr_b200.so is missing", "run `python -m faster_rwkv_b200.build` "
                              "(or __graft_entry__.build()) first")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            if not hasattr(L, name):
                continue
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int, what: str) -> None:
    if status < 0:
        L = lib()
        raise FrB200Error(status, f"{what}: {L.fr_b200_strerror(status).decode()}",
                          L.fr_b200_last_error().decode())


def _np_ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def parse_strategy(strategy: str):
    """"<device> <dtype>" -> (weight_format, act_fp16), model.cpp:25-60.  Only the cuda device exists here."""
    parts = strategy.split(" ")
    if len(parts) != 2 or parts[0] != "cuda":
        raise FrB200Error(-2, "unsupported strategy", f"{strategy!r}: this backend implements 'cuda fp16|int8|int4'")
    if parts[1] not in _FORMATS:
        raise FrB200Error(-2, "unsupported strategy", f"{strategy!r}: dtype must be fp16, int8 or int4")
    fmt = _FORMATS[parts[1]]
    return fmt, 1 if fmt == W_FP16 else 0


class Model:
    """rwkv::Model on the B200 backend.  `max_batch` > 1 adds the batched decode the reference lacks."""

    def __init__(self, path_or_tensors, strategy: str, max_batch: int = 1, device: int = 0, shape=None):
        fmt, act_fp16 = parse_strategy(strategy)
        if isinstance(path_or_tensors, (str, os.PathLike)):
            shape, tensors = synth.read_fr(os.fspath(path_or_tensors))
        else:
            tensors = path_or_tensors
            if shape is None:
                raise ValueError("shape is required when tensors are given directly")
        self.shape = shape
        self.strategy = strategy
        self.max_batch = max_batch
        self.vocab = shape.vocab
        self._h = _vp()
        cfg = Config(_VERSIONS[str(shape.version)], shape.n_layer, shape.n_embd, shape.n_ffn, shape.n_head,
                     shape.vocab, fmt, act_fp16, max_batch, device, 0)
        L = lib()
        check(L.fr_b200_create(ctypes.byref(cfg), ctypes.byref(self._h)), "fr_b200_create")
        try:
            for name, arr in tensors.items():
                self.set_tensor(name, arr)
            check(L.fr_b200_finalize(self._h), "fr_b200_finalize")
        except Exception:
            self.close()
            raise

    # -- packed model files ------------------------------------------------------------------
    def save_packed(self, path: str) -> None:
        """Write the finalized model's device blobs to `path` (fr_b200_save_packed)."""
        check(lib().fr_b200_save_packed(self._h, os.fspath(path).encode()), "fr_b200_save_packed")

    @classmethod
    def load_packed(cls, path: str, shape, strategy: str, max_batch: int = 1, device: int = 0) -> "Model":
        """A model from a packed file written by save_packed; shape and strategy must be the writer's."""
        self = cls.__new__(cls)
        self.shape, self.strategy, self.max_batch, self.vocab = shape, strategy, max_batch, shape.vocab
        self._h = _vp()
        check(lib().fr_b200_load_packed(os.fspath(path).encode(), max_batch, device, 0, ctypes.byref(self._h)), "fr_b200_load_packed")
        return self

    # -- upload ------------------------------------------------------------------------------
    def set_tensor(self, name: str, arr) -> None:
        """arr: numpy array (host) or anything with data_ptr()/dtype/shape (a torch CUDA tensor)."""
        if hasattr(arr, "data_ptr"):
            import torch
            t = arr.contiguous()
            dt = {torch.float16: T_F16, torch.float32: T_F32}[t.dtype]
            ptr, shp = t.data_ptr(), list(t.shape)
        else:
            a = np.ascontiguousarray(arr)
            if a.dtype not in (np.float16, np.float32):
                a = a.astype(np.float32)
            dt = T_F16 if a.dtype == np.float16 else T_F32
            ptr, shp = _np_ptr(a), list(a.shape)
        sh = (ctypes.c_int64 * len(shp))(*shp)
        check(lib().fr_b200_set_tensor(self._h, name.encode(), ptr, dt, sh, len(shp)), f"fr_b200_set_tensor({name})")

    # -- forward -----------------------------------------------------------------------------
    def run(self, ids: Union[int, Sequence[int]], slot: int = 0) -> np.ndarray:
        """Model::Run (model.cpp:188-208): one id, or a list processed in order; logits of the last token.
        slot: the stream whose state the prompt advances (prompts on slots > 0 need the seq / GEMM path)."""
        if isinstance(ids, (int, np.integer)):
            ids = [int(ids)]
        ids = np.ascontiguousarray(ids, np.int32)
        out = np.empty(self.vocab, np.float32)
        check(lib().fr_b200_run_seq(self._h, slot, _np_ptr(ids), len(ids), _np_ptr(out), None), "fr_b200_run_seq")
        return out

    def decode(self, ids: Sequence[int], want_logits: bool = True, want_argmax: bool = False):
        """One token for each of len(ids) independent streams (stream b = state slot b)."""
        ids = np.ascontiguousarray(ids, np.int32)
        B = len(ids)
        logits = np.empty((B, self.vocab), np.float32) if want_logits else None
        amax = np.empty(B, np.int32) if want_argmax else None
        check(lib().fr_b200_decode(self._h, _np_ptr(ids), B, _np_ptr(logits) if want_logits else None,
                                   _np_ptr(amax) if want_argmax else None, None), "fr_b200_decode")
        if want_logits and want_argmax:
            return logits, amax
        return logits if want_logits else amax

    def decode_greedy(self, first_ids: Sequence[int], n_tokens: int) -> np.ndarray:
        """n_tokens greedy steps per stream without a host round trip; returns the sampled ids [n_tokens, B]."""
        ids = np.ascontiguousarray(first_ids, np.int32)
        out = np.empty((n_tokens, len(ids)), np.int32)
        check(lib().fr_b200_decode_greedy(self._h, _np_ptr(ids), len(ids), n_tokens, _np_ptr(out), None),
              "fr_b200_decode_greedy")
        return out

    def sample(self, batch: int, temperature: float, top_k: int, top_p: float, uniform) -> np.ndarray:
        """Sampler::Sample (sampler.cpp:38-101) on the device over the logits of the last decode; uniform = the
        draws in [0, 1], one per stream."""
        u = np.ascontiguousarray(uniform, np.float32)
        out = np.empty(batch, np.int32)
        check(lib().fr_b200_sample(self._h, batch, temperature, top_k, top_p, _np_ptr(u), _np_ptr(out), None),
              "fr_b200_sample")
        return out

    def logits_add(self, streams, tokens, deltas) -> None:
        """logits[streams[i]][tokens[i]] += deltas[i] on the device (penalties / biases before `sample`, chat.cpp:57-75)."""
        s, t = np.ascontiguousarray(streams, np.int32), np.ascontiguousarray(tokens, np.int32)
        d = np.ascontiguousarray(deltas, np.float32)
        check(lib().fr_b200_logits_add(self._h, len(s), _np_ptr(s), _np_ptr(t), _np_ptr(d), None), "fr_b200_logits_add")

    def decode_profile(self, ids: Sequence[int]) -> np.ndarray:
        """One decode step; returns the [n_ctas, n_phases, 8] trace described at fr_b200_decode_profile in include/fr_b200.h."""
        ids = np.ascontiguousarray(ids, np.int32)
        inf = self.info()
        n, g = inf["n_phases"], inf["n_ctas"]
        st = np.zeros((g, n, 8), np.uint64)
        check(lib().fr_b200_decode_profile(self._h, _np_ptr(ids), len(ids), _np_ptr(st), g * n * 8),
              "fr_b200_decode_profile")
        return st

    # -- state -------------------------------------------------------------------------------
    def reset_states(self, slot: int = -1) -> None:
        check(lib().fr_b200_state_reset(self._h, slot), "fr_b200_state_reset")

    def states(self, slot: int = 0) -> List[List[np.ndarray]]:
        """Per layer the 5 (RWKV-4) or 3 (RWKV-5) state tensors, shapes and dtypes of model.cpp:145-177."""
        L = lib()
        nbytes = L.fr_b200_state_bytes(self._h)
        raw = np.empty(nbytes, np.uint8)
        check(L.fr_b200_state_export(self._h, slot, _np_ptr(raw), nbytes), "fr_b200_state_export")
        return self._split_state(raw)

    def _split_state(self, raw: np.ndarray) -> List[List[np.ndarray]]:
        C, H = self.shape.n_embd, self.shape.n_head
        act = np.float16 if self.strategy.endswith("fp16") else np.float32
        ab = np.dtype(act).itemsize
        v5 = str(self.shape.version).startswith("5")
        per = (2 * C * ab + H * 4096 * 4) if v5 else (2 * C * ab + 3 * C * 4)
        out = []
        for l in range(self.shape.n_layer):
            b = raw[l * per:(l + 1) * per]
            if v5:
                out.append([b[:C * ab].view(act).copy(),
                            b[C * ab:C * ab + H * 4096 * 4].view(np.float32).reshape(H, 64, 64).copy(),
                            b[C * ab + H * 4096 * 4:].view(act).copy()])
            else:
                o = C * ab
                out.append([b[:o].view(act).copy(), b[o:o + 4 * C].view(np.float32).copy(),
                            b[o + 4 * C:o + 8 * C].view(np.float32).copy(),
                            b[o + 8 * C:o + 12 * C].view(np.float32).copy(), b[o + 12 * C:].view(act).copy()])
        return out

    def export_state(self, slot: int = 0) -> np.ndarray:
        nbytes = lib().fr_b200_state_bytes(self._h)
        raw = np.empty(nbytes, np.uint8)
        check(lib().fr_b200_state_export(self._h, slot, _np_ptr(raw), nbytes), "fr_b200_state_export")
        return raw

    def import_state(self, raw: np.ndarray, slot: int = 0) -> None:
        raw = np.ascontiguousarray(raw, np.uint8)
        check(lib().fr_b200_state_import(self._h, slot, _np_ptr(raw), raw.nbytes), "fr_b200_state_import")

    def save_state_file(self, path: str, slot: int = 0) -> None:
        """Model::SaveStateFile (model.cpp:89-132): msgpack [[{dtype,data,shape}...] per layer]."""
        import msgpack
        out = []
        for layer in self.states(slot):
            out.append([{"dtype": "torch.float16" if t.dtype == np.float16 else "torch.float32",
                         "data": t.tobytes(), "shape": list(t.shape)} for t in layer])
        with open(path, "wb") as f:
            msgpack.pack(out, f)

    def load_state_file(self, path: str, slot: int = 0) -> None:
        """Model::LoadStateFile (model.cpp:134-143): shapes must match the model's states."""
        import msgpack
        with open(path, "rb") as f:
            layers = msgpack.unpack(f, raw=False)
        cur = self.states(slot)
        if len(layers) != len(cur):
            raise FrB200Error(-1, "load_state_file", "layer count mismatch")
        chunks = []
        for ls, cs in zip(layers, cur):
            if len(ls) != len(cs):
                raise FrB200Error(-1, "load_state_file", "state count mismatch")
            for t, c in zip(ls, cs):
                if list(t["shape"]) != list(c.shape):
                    raise FrB200Error(-1, "load_state_file", "state shape mismatch")
                dt = np.float16 if t["dtype"] == "torch.float16" else np.float32
                chunks.append(np.frombuffer(t["data"], dt).astype(c.dtype).tobytes())
        self.import_state(np.frombuffer(b"".join(chunks), np.uint8), slot)

    # -- misc --------------------------------------------------------------------------------
    def unpack_matrix(self, name: str, K: int, N: int) -> np.ndarray:
        W = np.empty((K, N), np.float32)
        check(lib().fr_b200_unpack_matrix(self._h, name.encode(), _np_ptr(W), K, N), "fr_b200_unpack_matrix")
        return W

    def info(self) -> Dict[str, int]:
        inf = Info()
        check(lib().fr_b200_get_info(self._h, ctypes.byref(inf)), "fr_b200_get_info")
        return {n: getattr(inf, n) for n, _ in Info._fields_}

    @property
    def handle(self):
        return self._h

    def close(self) -> None:
        if self._h:
            lib().fr_b200_destroy(self._h)
            self._h = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- free functions over the quantiser / kernel entry points -------------------------------------------

def quantize_int8(W: np.ndarray, device: int = 0):
    W = np.ascontiguousarray(W, np.float32)
    K, N = W.shape
    q = np.empty((N, K), np.int8)
    s = np.empty(N, np.uint16)
    check(lib().fr_b200_quantize_int8(_np_ptr(W), K, N, _np_ptr(q), _np_ptr(s), device), "fr_b200_quantize_int8")
    return q, s.view(np.float16)


def quantize_int4(W: np.ndarray, device: int = 0):
    W = np.ascontiguousarray(W, np.float32)
    K, N = W.shape
    p = np.empty((N, K // 2), np.uint8)
    s = np.empty((N, K // 32), np.uint16)
    check(lib().fr_b200_quantize_int4(_np_ptr(W), K, N, _np_ptr(p), _np_ptr(s), device), "fr_b200_quantize_int4")
    return p, s.view(np.float16)


def dequantize_int8(q: np.ndarray, s: np.ndarray, device: int = 0) -> np.ndarray:
    N, K = q.shape
    W = np.empty((K, N), np.float32)
    q = np.ascontiguousarray(q)
    s = np.ascontiguousarray(s).view(np.uint16)
    check(lib().fr_b200_dequantize_int8(_np_ptr(q), _np_ptr(s), K, N, _np_ptr(W), device), "fr_b200_dequantize_int8")
    return W


def dequantize_int4(p: np.ndarray, s: np.ndarray, device: int = 0) -> np.ndarray:
    N, K2 = p.shape
    W = np.empty((K2 * 2, N), np.float32)
    p = np.ascontiguousarray(p)
    s = np.ascontiguousarray(s).view(np.uint16)
    check(lib().fr_b200_dequantize_int4(_np_ptr(p), _np_ptr(s), K2 * 2, N, _np_ptr(W), device),
          "fr_b200_dequantize_int4")
    return W


def gemm_f16(A: np.ndarray, W: np.ndarray, epilogue: int = 0, aux0=None, aux1=None, scale: float = 1.0,
             device: int = 0) -> np.ndarray:
    """epilogue(A[M,K] @ W[K,N]) through the seq-mode tensor-core GEMM (operands rounded to fp16)."""
    A = np.ascontiguousarray(A, np.float32)
    W = np.ascontiguousarray(W, np.float32)
    M, K = A.shape
    N = W.shape[1]
    out = np.empty((M, N), np.float32)
    a0 = None if aux0 is None else np.ascontiguousarray(aux0, np.float32)
    a1 = None if aux1 is None else np.ascontiguousarray(aux1, np.float32)
    check(lib().fr_b200_gemm_f16(_np_ptr(A), _np_ptr(W), M, N, K, epilogue, None if a0 is None else _np_ptr(a0),
                                 None if a1 is None else _np_ptr(a1), scale, _np_ptr(out), device), "fr_b200_gemm_f16")
    return out


def matvec(W: np.ndarray, x: np.ndarray, weight_format: int, device: int = 0) -> np.ndarray:
    """y[B,N] = x[B,K] @ W[K,N] through the streaming dequant-matvec kernel."""
    W = np.ascontiguousarray(W, np.float32)
    x = np.ascontiguousarray(np.atleast_2d(x), np.float32)
    K, N = W.shape
    B = x.shape[0]
    y = np.empty((B, N), np.float32)
    check(lib().fr_b200_matvec(_np_ptr(W), K, N, weight_format, _np_ptr(x), B, _np_ptr(y), device), "fr_b200_matvec")
    return y
