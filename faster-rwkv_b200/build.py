"""Compile the sm_100a kernels and the C-ABI into csrc/libfr_b200.so (in-tree, nvcc, no cmake).

nvcc cross-compiles without a GPU.  Object files are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(CSRC, "libfr_b200.so")
SOURCES = ["pack.cu", "decode.cu", "prefill.cu", "sample.cu", "api.cu", "noalloc.cu", "ops.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _newest_header() -> float:
    t = 0.0
    for d in (CSRC, INCLUDE):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh")):
                t = max(t, os.path.getmtime(os.path.join(d, f)))
    return t


def build_lib(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(os.path.join(CSRC, "build"), exist_ok=True)
    hdr = _newest_header()
    objs, rebuilt = [], False
    procs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        if not os.path.exists(s):
            continue
        o = os.path.join(CSRC, "build", src.replace(".cu", ".o"))
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr):
            cmd = ["nvcc", *ARCH, *FLAGS, "-I", INCLUDE, "-c", s, "-o", o]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
            rebuilt = True
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        with open(os.path.join(CSRC, "build", src.replace(".cu", ".ptxas.txt")), "w") as f:
            f.write(out)
    if rebuilt or not os.path.exists(LIB):
        subprocess.check_call(["nvcc", *ARCH, "-shared", "-o", LIB, *objs])
    return LIB


if __name__ == "__main__":
    print(build_lib(force="--force" in sys.argv, verbose=True))
