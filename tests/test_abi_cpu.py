"""CPU checks of the boundary: the shared library loads, exports every symbol include/fr_b200.h declares,
and fails loudly (no fallback) when there is no GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    src = open(os.path.join(ROOT, "include", "fr_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(fr_b200_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol(pkg):
    L = pkg.lib()
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/fr_b200.h but not exported"
    # and the ctypes table binds exactly the declared set
    assert sorted(pkg.SIGNATURES) == names


def test_strerror_and_argument_errors(pkg):
    L = pkg.lib()
    assert L.fr_b200_strerror(0) == b"ok"
    assert b"argument" in L.fr_b200_strerror(-1)
    assert L.fr_b200_create(None, None) == -1
    h = ctypes.c_void_p()
    bad = pkg.Config(7, 1, 64, 64, 0, 10, 0, 1, 1, 0)
    assert L.fr_b200_create(ctypes.byref(bad), ctypes.byref(h)) == -2      # unknown version
    bad = pkg.Config(4, 1, 100, 64, 0, 10, 0, 1, 1, 0)
    assert L.fr_b200_create(ctypes.byref(bad), ctypes.byref(h)) == -2      # n_embd not a multiple of 64
    bad = pkg.Config(4, 1, 64, 64, 0, 10, 0, 1, 5000, 0)
    assert L.fr_b200_create(ctypes.byref(bad), ctypes.byref(h)) == -2      # more than 4096 stream slots
    assert b"max_batch" in L.fr_b200_last_error()


def test_strategy_parsing(pkg):
    assert pkg.parse_strategy("cuda fp16") == (pkg.W_FP16, 1)
    assert pkg.parse_strategy("cuda int8") == (pkg.W_INT8, 0)
    assert pkg.parse_strategy("cuda int4") == (pkg.W_INT4, 0)
    for s in ("cpu fp32", "cuda fp32", "cuda", "ncnn auto"):
        with pytest.raises(pkg.FrB200Error):
            pkg.parse_strategy(s)


def test_no_silent_fallback_without_gpu(pkg, synth):
    """Without a CUDA device the model constructor must raise: the product has no CPU path."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    shape = synth.SHAPES["tiny4"]
    with pytest.raises(pkg.FrB200Error):
        pkg.Model(synth.to_file_dtypes(shape, synth.generate(shape, 0), "fp16"), "cuda fp16", shape=shape)


def test_package_does_not_import_oracle():
    pkg_dir = os.path.join(ROOT, "faster-rwkv_b200")
    for dirpath, _, files in os.walk(pkg_dir):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "oracle" not in text.replace("rwkv_oracle.c", "").replace("oracle/rwkv_oracle", "") or \
                    f in ("pack.cu",), f"{f} mentions the oracle"


def test_fr_file_roundtrip(synth, tmp_path):
    shape = synth.SHAPES["tiny52"]
    master = synth.generate(shape, seed=4)
    for dt in ("fp16", "fp32"):
        t = synth.to_file_dtypes(shape, master, dt)
        p = str(tmp_path / f"m_{dt}.fr")
        synth.write_fr(p, shape, t)
        shape2, t2 = synth.read_fr(p)
        assert shape2 == shape
        assert set(t2) == set(t)
        for k in t:
            assert t2[k].dtype == t[k].dtype and np.array_equal(t2[k], t[k]), k
    assert t["blocks.0.att.time_decay"].dtype == np.float32 and t["blocks.0.att.time_decay"].shape == (2, 64, 1)
    assert synth.to_file_dtypes(shape, master, "fp16")["blocks.0.att.ln_x.weight"].dtype == np.float32
    names = synth.param_names(shape)
    assert len(names) == shape.n_layer * 22 + 3 and names[-1] == "head.weight"
