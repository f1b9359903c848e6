"""Seeded synthetic RWKV weights in the reference's `.fr` container.

The `.fr` file is the msgpack map written by the reference's
tools/convert_weight.py:9-55 and read by kernels/default/init_model.cpp:19-133:
  {"embd_weights": [tensor per vocab row], "weights": {name: tensor},
   "version": "4"|"5"|"5.1"|"5.2", "n_layer", "n_embd", "n_att", "n_ffn", ["n_head"]}
with tensor = {"dtype": "torch.float16"|"torch.float32", "data": bytes, "shape": [...]}.

What the run-time consumes (fixed by the reference kernels, not by the file):
  * matrices are stored [in, out] (y = x @ W), kernels/cuda/matmul.cpp:105-122;
  * RWKV-4 `time_decay` already holds -exp(raw) (kernels/cuda/att.cu:53 adds it to pp),
    RWKV-5.x `time_decay` holds exp(-exp(raw)) (att.cu:79), `time_first` is used raw;
  * fp16 files carry att.output / ffn.value divided by 2**(layer // 6), matching the
    x /= 2 every 6 layers of kernels/default/model_forward.cpp:173-175;
  * dtypes under "cuda fp16": fp16 everywhere except time_decay, time_first and
    (RWKV-5) ln_x.weight / ln_x.bias, which are fp32.

Distributions: matrices ~ N(0, 1/sqrt(fan_in)), time_mix ~ U(0,1), raw decay ~ U(-6,1),
time_first ~ U(-1,1), LayerNorm gamma=1 / beta=0 (or randomised with ln_random=True so
that tests exercise the affine part), embedding rows ~ N(0,1).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List

import numpy as np

try:
    import msgpack
except ImportError:  # pragma: no cover - msgpack is part of the image
    msgpack = None


@dataclasses.dataclass
class Shape:
    """Model dimensions. version is "4", "5", "5.1" or "5.2"."""
    version: str
    n_layer: int
    n_embd: int
    n_ffn: int
    vocab: int
    n_head: int = 0  # RWKV-5 only; head size is n_embd // n_head

    @property
    def n_att(self) -> int:
        return self.n_embd


# The five benchmark shapes plus tiny shapes for tests.
SHAPES: Dict[str, Shape] = {
    "c0": Shape("4", 12, 768, 3072, 65536),
    "c1": Shape("4", 24, 2048, 8192, 65536),
    "c3": Shape("5.2", 32, 2560, 8960, 65536, n_head=40),
    "c4": Shape("4", 40, 5120, 20480, 50277),
    "tiny4": Shape("4", 2, 128, 512, 96),
    "tiny4b": Shape("4", 7, 192, 448, 211),
    "tiny52": Shape("5.2", 2, 128, 448, 96, n_head=2),
    "tiny51": Shape("5.1", 2, 128, 448, 96, n_head=2),
    "tiny50": Shape("5", 2, 128, 448, 96, n_head=2),
    "mid4": Shape("4", 7, 256, 1024, 512),
    "mid52": Shape("5.2", 3, 256, 1024, 512, n_head=4),
    "wide4": Shape("4", 2, 256, 8192, 512),   # channel-mix width of c1: 8 streams of it exceed the persistent kernel
}


def param_names(shape: Shape) -> List[str]:
    """Parameter names in the order kernels/default/init_model.cpp:75-126 pushes them."""
    v5 = shape.version.startswith("5")
    gate = shape.version in ("5.1", "5.2")
    names: List[str] = []
    for i in range(shape.n_layer):
        b, a, f = f"blocks.{i}.", f"blocks.{i}.att.", f"blocks.{i}.ffn."
        names += [b + "ln1.weight", b + "ln1.bias"]
        if v5:
            names += [a + "ln_x.weight", a + "ln_x.bias"]
        names += [a + "time_mix_k", a + "time_mix_v", a + "time_mix_r"]
        if gate:
            names += [a + "time_mix_g"]
        names += [a + "time_decay", a + "time_first", a + "key.weight", a + "value.weight",
                  a + "receptance.weight"]
        if gate:
            names += [a + "gate.weight"]
        names += [a + "output.weight", b + "ln2.weight", b + "ln2.bias", f + "time_mix_k",
                  f + "time_mix_r", f + "key.weight", f + "value.weight", f + "receptance.weight"]
    names += ["ln_out.weight", "ln_out.bias", "head.weight"]
    return names


def generate(shape: Shape, seed: int = 0, ln_random: bool = False) -> Dict[str, np.ndarray]:
    """fp32 master weights, keyed by the reference's tensor names, plus 'emb.weight' [V, C]."""
    rng = np.random.default_rng(seed)
    C, F, V, L = shape.n_embd, shape.n_ffn, shape.vocab, shape.n_layer
    v5 = shape.version.startswith("5")
    H = shape.n_head
    S = C // H if v5 else 0
    w: Dict[str, np.ndarray] = {}

    def mat(fan_in: int, fan_out: int) -> np.ndarray:
        return (rng.standard_normal((fan_in, fan_out), dtype=np.float32) / np.float32(np.sqrt(fan_in)))

    def ln(prefix: str, n: int) -> None:
        if ln_random:
            w[prefix + ".weight"] = rng.uniform(0.5, 1.5, n).astype(np.float32)
            w[prefix + ".bias"] = (0.1 * rng.standard_normal(n)).astype(np.float32)
        else:
            w[prefix + ".weight"] = np.ones(n, np.float32)
            w[prefix + ".bias"] = np.zeros(n, np.float32)

    w["emb.weight"] = rng.standard_normal((V, C), dtype=np.float32)
    for i in range(L):
        b, a, f = f"blocks.{i}.", f"blocks.{i}.att.", f"blocks.{i}.ffn."
        ln(b + "ln1", C)
        if v5:
            ln(a + "ln_x", C)
        for m in ("k", "v", "r") + (("g",) if shape.version in ("5.1", "5.2") else ()):
            w[a + "time_mix_" + m] = rng.uniform(0, 1, C).astype(np.float32)
        raw = rng.uniform(-6, 1, C).astype(np.float32)
        first = rng.uniform(-1, 1, C).astype(np.float32)
        if not v5:
            w[a + "time_decay"] = -np.exp(raw)
            w[a + "time_first"] = first
        elif shape.version == "5":
            # one scalar decay / bonus per head (kernels/cuda/att.cu:242 indexes i / (S*S))
            w[a + "time_decay"] = np.exp(-np.exp(raw[:H])).reshape(H, 1, 1)
            w[a + "time_first"] = first[:H].reshape(H, 1, 1)
        else:
            w[a + "time_decay"] = np.exp(-np.exp(raw)).reshape(H, S, 1)
            w[a + "time_first"] = first.reshape(H, S, 1)
        w[a + "key.weight"] = mat(C, C)
        w[a + "value.weight"] = mat(C, C)
        w[a + "receptance.weight"] = mat(C, C)
        if shape.version in ("5.1", "5.2"):
            w[a + "gate.weight"] = mat(C, C)
        w[a + "output.weight"] = mat(C, C)
        ln(b + "ln2", C)
        w[f + "time_mix_k"] = rng.uniform(0, 1, C).astype(np.float32)
        w[f + "time_mix_r"] = rng.uniform(0, 1, C).astype(np.float32)
        w[f + "key.weight"] = mat(C, F)
        w[f + "value.weight"] = mat(F, C)
        w[f + "receptance.weight"] = mat(C, C)
    ln("ln_out", C)
    w["head.weight"] = mat(C, V)
    return w


_FP32_ONLY = ("time_decay", "time_first", "ln_x.weight", "ln_x.bias")


def to_file_dtypes(shape: Shape, master: Dict[str, np.ndarray], dtype: str) -> Dict[str, np.ndarray]:
    """Master fp32 weights -> the arrays a `.fr` file of `dtype` ("fp16" | "fp32") holds.

    fp16 files get att.output / ffn.value divided by 2**(layer // 6) before rounding
    (kernels/default/model_forward.cpp:173-175 divides the residual at those layers).
    """
    assert dtype in ("fp16", "fp32")
    out: Dict[str, np.ndarray] = {}
    for k, v in master.items():
        if dtype == "fp32":
            out[k] = v.astype(np.float32)
            continue
        if k.endswith(_FP32_ONLY):
            out[k] = v.astype(np.float32)
            continue
        if k.endswith(("att.output.weight", "ffn.value.weight")):
            layer = int(k.split(".")[1])
            v = v / np.float32(2 ** (layer // 6))
        out[k] = v.astype(np.float16)
    return out


def fp16_exact_pair(shape: Shape, master: Dict[str, np.ndarray]):
    """(fp16 file tensors, fp32 file tensors) that describe the SAME model exactly: the fp32 set is the fp16
    set widened, with the 2**(layer//6) pre-division of att.output / ffn.value undone (exact: a power of two).
    An fp32 strategy without the x/2 rescale on the second set and the fp16 strategy on the first then
    multiply by identical weight values."""
    f16 = to_file_dtypes(shape, master, "fp16")
    f32 = {}
    for k, v in f16.items():
        w = v.astype(np.float32)
        if k.endswith(("att.output.weight", "ffn.value.weight")):
            w = w * np.float32(2 ** (int(k.split(".")[1]) // 6))
        f32[k] = w
    return f16, f32


def write_fr(path: str, shape: Shape, tensors: Dict[str, np.ndarray]) -> None:
    """Write the msgpack container of tools/convert_weight.py:9-55."""
    def pack(x: np.ndarray) -> dict:
        dt = {"float16": "torch.float16", "float32": "torch.float32", "int8": "torch.int8"}[x.dtype.name]
        return {"dtype": dt, "data": np.ascontiguousarray(x).tobytes(), "shape": list(x.shape)}

    d = {"embd_weights": [pack(r) for r in tensors["emb.weight"]],
         "weights": {k: pack(v) for k, v in tensors.items() if k != "emb.weight"},
         "version": shape.version, "n_layer": shape.n_layer, "n_embd": shape.n_embd,
         "n_att": shape.n_att, "n_ffn": shape.n_ffn}
    if shape.version.startswith("5"):
        d["n_head"] = shape.n_head
    with open(path, "wb") as f:
        msgpack.pack(d, f)


def read_fr(path: str):
    """Read a `.fr` file -> (Shape, {name: ndarray}) with 'emb.weight' stacked to [V, C]."""
    with open(path, "rb") as f:
        d = msgpack.unpack(f, raw=False, strict_map_key=False)

    def unpack(t: dict) -> np.ndarray:
        dt = {"torch.float16": np.float16, "torch.float32": np.float32, "torch.int8": np.int8}[t["dtype"]]
        return np.frombuffer(t["data"], dtype=dt).reshape(t["shape"]).copy()

    tensors = {k: unpack(v) for k, v in d["weights"].items()}
    tensors["emb.weight"] = np.stack([unpack(t) for t in d["embd_weights"]])
    version = str(d.get("version", "4"))
    shape = Shape(version, int(d["n_layer"]), int(d["n_embd"]),
                  int(d.get("n_ffn", tensors["blocks.0.ffn.key.weight"].shape[1])),
                  tensors["emb.weight"].shape[0], int(d.get("n_head", 0)))
    return shape, tensors


def token_ids(shape: Shape, n: int, seed: int = 0) -> np.ndarray:
    """n token ids ~ U[0, vocab) from `seed`."""
    return np.random.default_rng(seed + 12345).integers(0, shape.vocab, n).astype(np.int32)


def device_tensors(shape: Shape, seed: int, device, file_dtype: str = "fp32"):
    """Yield (name, CUDA tensor) for a model of `shape` with the distributions of generate(), drawn on the GPU (the
    1.5B- to 14B-shaped models take minutes to draw with numpy).  The stream of values differs from generate()'s.
    file_dtype "fp16" applies what a "cuda fp16" `.fr` file holds: fp16 everywhere except time_decay, time_first and
    ln_x, att.output / ffn.value pre-divided by 2**(layer // 6) (kernels/default/model_forward.cpp:173-175)."""
    import math
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    C, F, V, L, H = shape.n_embd, shape.n_ffn, shape.vocab, shape.n_layer, shape.n_head
    v5 = shape.version.startswith("5")
    gate = shape.version in ("5.1", "5.2")

    def mat(k, n):
        return torch.randn(k, n, generator=g, device=device, dtype=torch.float32) / math.sqrt(k)

    def uni(n, lo, hi):
        return torch.rand(n, generator=g, device=device, dtype=torch.float32) * (hi - lo) + lo

    def raw():
        yield "emb.weight", torch.randn(V, C, generator=g, device=device, dtype=torch.float32)
        for i in range(L):
            b, a, f = f"blocks.{i}.", f"blocks.{i}.att.", f"blocks.{i}.ffn."
            for ln in (b + "ln1", b + "ln2"):
                yield ln + ".weight", torch.ones(C, device=device)
                yield ln + ".bias", torch.zeros(C, device=device)
            if v5:
                yield a + "ln_x.weight", torch.ones(C, device=device)
                yield a + "ln_x.bias", torch.zeros(C, device=device)
            for m in ("k", "v", "r") + (("g",) if gate else ()):
                yield a + "time_mix_" + m, uni(C, 0, 1)
            if not v5:
                yield a + "time_decay", -torch.exp(uni(C, -6, 1))
                yield a + "time_first", uni(C, -1, 1)
            elif shape.version == "5":
                yield a + "time_decay", torch.exp(-torch.exp(uni(H, -6, 1))).reshape(H, 1, 1)
                yield a + "time_first", uni(H, -1, 1).reshape(H, 1, 1)
            else:
                yield a + "time_decay", torch.exp(-torch.exp(uni(C, -6, 1))).reshape(H, C // H, 1)
                yield a + "time_first", uni(C, -1, 1).reshape(H, C // H, 1)
            yield a + "key.weight", mat(C, C)
            yield a + "value.weight", mat(C, C)
            yield a + "receptance.weight", mat(C, C)
            if gate:
                yield a + "gate.weight", mat(C, C)
            yield a + "output.weight", mat(C, C)
            yield f + "time_mix_k", uni(C, 0, 1)
            yield f + "time_mix_r", uni(C, 0, 1)
            yield f + "key.weight", mat(C, F)
            yield f + "value.weight", mat(F, C)
            yield f + "receptance.weight", mat(C, C)
        yield "ln_out.weight", torch.ones(C, device=device)
        yield "ln_out.bias", torch.zeros(C, device=device)
        yield "head.weight", mat(C, V)

    for name, t in raw():
        if file_dtype == "fp16" and not name.endswith(_FP32_ONLY):
            if name.endswith(("att.output.weight", "ffn.value.weight")):
                t = t / float(2 ** (int(name.split(".")[1]) // 6))
            t = t.half()
        yield name, t
