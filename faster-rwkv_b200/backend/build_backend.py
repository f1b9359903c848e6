"""Link the reference's unchanged model.cpp / tensor.cpp / kernels/{cpu,default,shape} with the registry glue
(registry_backend.cpp) and libfr_b200.so into a driver binary: the drop-in demonstration.

  backend/build/fr_b200_run <model.fr> "cuda fp16|int8|int4" <out.bin> [--seq] ids...

The reference sources are compiled where they lie (FR_REFERENCE_DIR, else a checkout named "reference" beside this repository) with
-DFR_ENABLE_CUDA; kernels/cuda/* is left out (this backend replaces it).  registry_backend.o is linked last so
that its registrations for Device::kCUDA win over def::init_model / def::ModelForward (kernels/registry.h:17-19).
msgpack-c is not available offline; backend/compat/msgpack.hpp stands in for it in this container.
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("FR_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
OUT = os.path.join(HERE, "build")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def build(force: bool = False) -> str:
    if not os.path.isdir(REF):
        raise RuntimeError(f"reference tree not found at {REF}")
    os.makedirs(OUT, exist_ok=True)
    exe = os.path.join(OUT, "fr_b200_run")
    srcs = [os.path.join(REF, f) for f in ("model.cpp", "tensor.cpp", "utils.cpp", "sampler.cpp")]
    for d in ("kernels/cpu", "kernels/default", "kernels/shape"):
        srcs += sorted(glob.glob(os.path.join(REF, d, "*.cpp")))
    srcs.append(os.path.join(REF, "kernels/export-ncnn/kernels.cpp"))
    srcs.append(os.path.join(HERE, "fr_run.cpp"))
    srcs.append(os.path.join(HERE, "registry_backend.cpp"))      # last: its registrations must win
    lib = os.path.join(os.path.dirname(HERE), "csrc", "libfr_b200.so")
    deps = srcs + [os.path.join(ROOT, "include", "fr_b200.h"), os.path.join(HERE, "compat", "msgpack.hpp")]
    newest = max(os.path.getmtime(s) for s in deps)
    if not force and os.path.exists(exe) and os.path.getmtime(exe) >= max(newest, os.path.getmtime(lib)):
        return exe
    objs, procs = [], []
    for s in srcs:
        o = os.path.join(OUT, os.path.relpath(s, "/").replace("/", "_").replace(".cpp", ".o"))
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < newest:
            cmd = ["g++", "-std=c++17", "-O2", "-march=x86-64-v3", "-w", "-include", "immintrin.h", "-DFR_ENABLE_CUDA",
                   "-I", os.path.join(HERE, "compat"), "-I", REF, "-I", os.path.join(CUDA, "include"),
                   "-c", s, "-o", o]
            procs.append((s, subprocess.Popen(cmd)))
    for s, p in procs:
        if p.wait() != 0:
            raise RuntimeError(f"g++ failed on {s}")
    subprocess.check_call(["g++", "-o", exe, *objs, lib, "-L", os.path.join(CUDA, "lib64"), "-lcudart",
                           "-Wl,-rpath,$ORIGIN/../../csrc", "-Wl,-rpath," + os.path.join(CUDA, "lib64")])
    return exe


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
