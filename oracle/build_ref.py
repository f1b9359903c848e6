"""Build the reference's own CPU path from its sources where they lie (never copied into this tree).

Outputs go to oracle/_ref/ only (the whole folder is git-ignored; the built files still travel to a GPU box):
  fr_ref_run   rwkv::Model driver: reference model.cpp, tensor.cpp, utils.cpp, kernels/cpu/*,
               kernels/default/*, kernels/shape/*, kernels/export-ncnn/kernels.cpp  +  oracle/ref/cpu_prims.cpp
               (the fp32 CPU primitives the reference lacks)  +  faster-rwkv_b200/backend/fr_run.cpp
msgpack-c (a FetchContent dependency of the reference) is replaced by faster-rwkv_b200/backend/compat/msgpack.hpp.
The reference's CMake build is not run.  TEST INFRASTRUCTURE ONLY.
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BACKEND = os.path.join(os.path.dirname(HERE), "faster-rwkv_b200", "backend")   # msgpack stand-in + the shared driver
# the reference tree: FR_REFERENCE_DIR, else a checkout named "reference" beside this repository
REF = os.environ.get("FR_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
OUT = os.path.join(HERE, "_ref")


def build(force: bool = False) -> str:
    if not os.path.isdir(REF):
        raise RuntimeError(f"reference tree not found at {REF}")
    os.makedirs(OUT, exist_ok=True)
    exe = os.path.join(OUT, "fr_ref_run")
    srcs = [os.path.join(REF, f) for f in ("model.cpp", "tensor.cpp", "utils.cpp", "sampler.cpp")]
    for d in ("kernels/cpu", "kernels/default", "kernels/shape"):
        srcs += sorted(glob.glob(os.path.join(REF, d, "*.cpp")))
    srcs.append(os.path.join(REF, "kernels/export-ncnn/kernels.cpp"))
    srcs += [os.path.join(HERE, "ref", "cpu_prims.cpp"), os.path.join(BACKEND, "fr_run.cpp")]
    newest = max(os.path.getmtime(s) for s in srcs + [os.path.join(BACKEND, "compat", "msgpack.hpp")])
    if not force and os.path.exists(exe) and os.path.getmtime(exe) >= newest:
        return exe
    objs, procs = [], []
    for s in srcs:
        o = os.path.join(OUT, os.path.relpath(s, "/").replace("/", "_").replace(".cpp", ".o"))
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < newest:
            cmd = ["g++", "-std=c++17", "-O2", "-march=x86-64-v3", "-w", "-include", "immintrin.h", "-I", os.path.join(BACKEND, "compat"), "-I", REF,
                   "-c", s, "-o", o]
            procs.append((s, subprocess.Popen(cmd)))
    for s, p in procs:
        if p.wait() != 0:
            raise RuntimeError(f"g++ failed on {s}")
    subprocess.check_call(["g++", "-o", exe, *objs])
    return exe


def build_cuda(force: bool = False) -> str:
    """fr_ref_cuda_run: the reference's own kernels/cuda/* + cuBLAS path, compiled for sm_100a, same driver.
    This is the reference GPU baseline ("cuda fp16") that the backend is compared with on the B200."""
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    os.makedirs(OUT, exist_ok=True)
    exe = os.path.join(OUT, "fr_ref_cuda_run")
    srcs = [os.path.join(REF, f) for f in ("model.cpp", "tensor.cpp", "utils.cpp", "sampler.cpp")]
    for d in ("kernels/cpu", "kernels/default", "kernels/shape"):
        srcs += sorted(glob.glob(os.path.join(REF, d, "*.cpp")))
    srcs.append(os.path.join(REF, "kernels/export-ncnn/kernels.cpp"))
    srcs += sorted(glob.glob(os.path.join(REF, "kernels/cuda", "*.cpp")))
    srcs += sorted(glob.glob(os.path.join(REF, "kernels/cuda", "*.cu")))
    srcs += sorted(glob.glob(os.path.join(REF, "kernels/cuda", "activations", "*.cu")))
    srcs.append(os.path.join(BACKEND, "fr_run.cpp"))
    newest = max(os.path.getmtime(s) for s in srcs + [os.path.join(BACKEND, "compat", "msgpack.hpp")])
    if not force and os.path.exists(exe) and os.path.getmtime(exe) >= newest:
        return exe
    objs, procs = [], []
    for s in srcs:
        o = os.path.join(OUT, "cu_" + os.path.relpath(s, "/").replace("/", "_").replace(".cpp", ".o").replace(".cu", ".o"))
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < newest:
            if s.endswith(".cu"):
                cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O2", "-w", "-DFR_ENABLE_CUDA",
                       "-I", os.path.join(BACKEND, "compat"), "-I", REF, "-c", s, "-o", o]
            else:
                cmd = ["g++", "-std=c++17", "-O2", "-march=x86-64-v3", "-w", "-include", "immintrin.h", "-DFR_ENABLE_CUDA",
                       "-I", os.path.join(BACKEND, "compat"), "-I", REF, "-I", os.path.join(cuda, "include"), "-c", s, "-o", o]
            procs.append((s, subprocess.Popen(cmd)))
    for s, p in procs:
        if p.wait() != 0:
            raise RuntimeError(f"compile failed on {s}")
    subprocess.check_call(["g++", "-o", exe, *objs, "-L", os.path.join(cuda, "lib64"), "-lcudart", "-lcublas",
                           "-Wl,-rpath," + os.path.join(cuda, "lib64")])
    return exe


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
    try:
        print(build_cuda(force="--force" in sys.argv))
    except Exception as ex:  # the CUDA baseline is optional: report and go on
        print("reference CUDA build failed:", ex)
