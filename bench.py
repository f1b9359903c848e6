#!/usr/bin/env python3
"""Decode benchmark of the B200 RWKV backend.

  python bench.py [--gpus N] [--steps K] [--warmup W]             # batched decode, the workload below
  python bench.py --workload c1 --weights fp16 --batch 1 ...      # one model, B streams per GPU (profiling runs)
  python bench.py --impl reference ...                            # the CPU fp32 path timed on the host cores
  python bench.py --phase-budget                                  # per-phase time budget of the batch-1 kernel

Default workload ("c2"): an RWKV-4 1.5B-shaped model (24 layers, n_embd 2048, FFN 8192, vocab 65536), int4 weights
(group-32 scales), 256 independent streams in total, each with a random 32-token prompt and then greedy decode.
The streams are cut into contiguous slices, one per GPU (faster-rwkv_b200/shard.py); every GPU holds a full weight
replica and its own recurrent states, and no collective sits on the data path.  A step = one new token for every
stream.  `value` is tokens/s of the whole job with the token ids staying on the device (greedy feedback on the GPU,
steps replayed as a CUDA graph); `e2e` goes through the public Model.decode call with host ids in and host arg-max
ids out every step.  The total is fixed, so scaling is "strong"; the line also carries the "weak" figure (256 streams
on every GPU).  NCCL only gathers the sampled ids for the cross-GPU check after the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

WORKLOADS = {  # name -> (shape key, description)
    "c2": ("c1", "RWKV-4 1.5B-shaped (L24 C2048 F8192 V65536), batched decode"),
    "c1": ("c1", "RWKV-4 1.5B-shaped (L24 C2048 F8192 V65536), decode"),
    "c0": ("c0", "RWKV-4 0.1B-shaped (L12 C768 F3072 V65536), decode"),
    "c3": ("c3", "RWKV-5.2 3B-shaped (L32 C2560 F8960 H40 V65536), decode"),
    "c4": ("c4", "RWKV-4 14B-shaped (L40 C5120 F20480 V50277), decode"),
    "tiny": ("tiny4b", "tiny RWKV-4 (L7 C192 F448 V211)"),
}
FILE_OF = {"fp16": "fp16", "int8": "fp32", "int4": "fp32"}   # strategy -> dtype of the `.fr` tensors it is given
DTYPE_OF = {"fp16": "f16", "int8": "i8->f16 x f16 (f32 acc)", "int4": "i4->f16 x f16 (f32 acc)"}
C2_STREAMS, C2_PROMPT = 256, 32


def projection_params(shape) -> int:
    C, F, V, L = shape.n_embd, shape.n_ffn, shape.vocab, shape.n_layer
    att = 5 if str(shape.version) in ("4", "5") else 6
    return L * (att * C * C + 2 * C * F) + C * V


def algorithmic_bytes(shape, fmt: str) -> int:
    """Bytes of projection weights (+ quantisation scales) one step must read: every matvec weight once."""
    C, F, V, L = shape.n_embd, shape.n_ffn, shape.vocab, shape.n_layer
    att = 5 if str(shape.version) in ("4", "5") else 6
    P = projection_params(shape)
    rows = L * (att * C + F + C) + V          # output rows (one int8 scale each)
    if fmt == "fp16":
        return 2 * P
    if fmt == "int8":
        return P + 2 * rows
    return P // 2 + 2 * (P // 32)


def measured_peaks():
    """(HBM GB/s, bf16 TFLOP/s burst, sustained, source) from the driver-written MEASURED_PEAKS.json, else the fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    except Exception:
        return 6650.0, 1590.0, 1400.0, "fallback"


def hbm_roofline(shape, fmt, ms_per_step, kernel):
    peak, _, _, kind = measured_peaks()
    algo = algorithmic_bytes(shape, fmt)
    ach = algo / (ms_per_step * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
            "peak_source": kind, "kernel": kernel, "algorithmic_bytes_per_launch": algo}


def batched_roofline(shape, fmt, streams, ms_per_step):
    """A step of `streams` streams reads every weight once and does 2 * P * streams flops: the tighter of the two
    bounds names the roofline (the sustained tensor figure: the step sits inside a seconds-long loop)."""
    hbm, _, tens, kind = measured_peaks()
    algo_b, algo_f = algorithmic_bytes(shape, fmt), 2.0 * projection_params(shape) * streams
    t_b, t_f = algo_b / (hbm * 1e9), algo_f / (tens * 1e12)
    s = ms_per_step * 1e-3
    kernel = "batched decode step: few-row tcgen05 GEMMs + row kernels (steps replayed as a CUDA graph)"
    if t_f >= t_b:
        ach = algo_f / s / 1e12
        return {"bound": "tensor", "achieved": ach, "peak": tens, "unit": "TFLOP/s", "frac": ach / tens, "traffic": None,
                "peak_source": kind + " (sustained)", "kernel": kernel, "algorithmic_flops_per_step": algo_f,
                "hbm_bound_ms": t_b * 1e3, "tensor_bound_ms": t_f * 1e3}
    ach = algo_b / s / 1e9
    return {"bound": "hbm", "achieved": ach, "peak": hbm, "unit": "GB/s", "frac": ach / hbm, "traffic": None,
            "peak_source": kind, "kernel": kernel, "algorithmic_bytes_per_step": algo_b,
            "hbm_bound_ms": t_b * 1e3, "tensor_bound_ms": t_f * 1e3}


# ------------------------------------------------------------------ synthetic weights on the GPU

def build_model(pkg, shape, fmt: str, max_batch: int, device_index: int, seed: int = 0, keep_host=None):
    """Model with seeded weights generated on the GPU (synth.device_tensors); keep_host, when given, receives the
    tensors as numpy arrays in the file dtype (what the CPU oracle is built from)."""
    import torch
    dev = torch.device("cuda", device_index)

    # Model() walks tensors.items() once; a generator-backed feed keeps peak memory low
    class Feed:
        def items(self_inner):
            for name, t in pkg.synth.device_tensors(shape, seed, dev, FILE_OF[fmt]):
                if keep_host is not None:
                    keep_host[name] = t.cpu().numpy()
                yield name, t
    m = pkg.Model(Feed(), f"cuda {fmt}", max_batch=max_batch, device=device_index, shape=shape)
    torch.cuda.synchronize(dev)
    return m


def drop(model):
    import torch
    model.close()
    torch.cuda.empty_cache()


# ------------------------------------------------------------------ seq mode (prompt processing)

def prefill_leg(pkg, device_index: int, wl: str = "c3", T: int = 4096, reps: int = 3):
    """One 4096-token prompt through the seq path of an RWKV-5.2 3B-shaped model (L32 C2560 F8960 H40), fp16 weights:
    Model.run(ids) with host ids in and host logits out.  FLOPs = 2 * (projection params) * T + the head once."""
    import torch
    try:
        shape = pkg.synth.SHAPES[wl]
        m = build_model(pkg, shape, "fp16", 1, device_index, seed=0)
        ids = [int(t) for t in pkg.synth.token_ids(shape, T, seed=1)]
        C, F, V, L = shape.n_embd, shape.n_ffn, shape.vocab, shape.n_layer
        P = L * (6 * C * C + 2 * C * F)
        flops = 2.0 * P * T + 2.0 * C * V
        m.run(ids)                                   # warm-up (allocates the activation buffers)
        best = None
        for _ in range(reps):
            m.reset_states()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            m.run(ids)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        _, burst, sustained, kind = measured_peaks()
        tf = flops / (best * 1e-3) / 1e12
        out = {"workload": "c3: RWKV-5.2 3B-shaped (L32 C2560 F8960 H40 V65536), one 4096-token prompt, fp16 weights",
               "ms": best, "tok_s": T / (best * 1e-3), "tflops": tf, "algorithmic_flops": flops,
               "roofline": {"bound": "tensor", "achieved": tf, "peak": burst, "unit": "TFLOP/s", "frac": tf / burst,
                            "traffic": None, "peak_source": kind + " (burst: the prompt is one 30-50 ms call)",
                            "frac_of_sustained_peak": tf / sustained,
                            "kernel": "gemm_f16_kernel (tcgen05) + state scan + row kernels"}}
        drop(m)
        del m
        # 16 streams: one prompt each, slot by slot (a 4096-token prompt already fills the tensor cores), then 64
        # greedy steps of all 16 together through the GEMM path
        try:
            B = 16
            m = build_model(pkg, shape, "fp16", B, device_index, seed=0)
            prompts = [[int(t) for t in pkg.synth.token_ids(shape, T, seed=10 + b)] for b in range(B)]
            m.run(prompts[0], slot=0)
            m.reset_states()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            firsts = [int(np.argmax(m.run(prompts[b], slot=b))) for b in range(B)]
            e1.record()
            torch.cuda.synchronize()
            ms16 = e0.elapsed_time(e1)
            m.decode_greedy(firsts, 4)
            torch.cuda.synchronize()
            e0.record()
            m.decode_greedy(firsts, 64)
            e1.record()
            torch.cuda.synchronize()
            msd = e0.elapsed_time(e1)
            out["batch16"] = {"prefill_ms": ms16, "prefill_tok_s": B * T / (ms16 * 1e-3),
                              "prefill_tflops": B * flops / (ms16 * 1e-3) / 1e12,
                              "decode_64_steps_ms_per_step": msd / 64, "decode_tok_s": B * 64 / (msd * 1e-3)}
            drop(m)
            del m
        except Exception as ex:
            out["batch16"] = {"error": str(ex)[:200]}
        return out
    except Exception as ex:
        return {"error": str(ex)[:200]}


# ------------------------------------------------------------------ clocks

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
                for n, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ CPU baseline (oracle)

def cpu_baseline(shape, fmt, host_tensors, n_tokens: int, seed: int = 0, threads: int = 0):
    """The fp32 CPU path (oracle port of the reference's op compositions), batch 1, on `threads` host threads
    (0 = every core of the box)."""
    orc = entry.load_oracle()
    orc.build()
    pkg = entry.load_package()
    orc.lib().orc_set_threads(threads if threads > 0 else (os.cpu_count() or 1))
    if host_tensors is None:
        host_tensors = pkg.synth.to_file_dtypes(shape, pkg.synth.generate(shape, seed), "fp32")
        fmt = "fp32"
    m = orc.OracleModel(shape, host_tensors, pkg.synth.param_names(shape), rescale_every=6 if fmt == "fp16" else 0,
                        state_fp16=fmt == "fp16")
    ids = pkg.synth.token_ids(shape, n_tokens + 1, seed)
    m.run(int(ids[0]))  # warm-up: page in the weights
    t0 = time.perf_counter()
    for t in ids[1:]:
        m.run(int(t))
    dt = time.perf_counter() - t0
    return {"value": n_tokens / dt, "unit": "tok/s", "cores": orc.lib().orc_num_threads(), "kind": "port",
            "sample": f"{n_tokens} tokens of one stream, fp32 arithmetic, same model shape ({dt:.1f} s)"}


# ------------------------------------------------------------------ reference GPU path, same driver binary

def reference_gpu_leg(pkg, n_tokens: int = 128):
    """The reference's own kernels/cuda + cuBLAS ("cuda fp16", rebuilt for sm_100a: oracle/_ref/fr_ref_cuda_run) and
    this backend behind the same unchanged rwkv::Model (faster-rwkv_b200/backend/build/fr_b200_run), on the same
    `.fr` files, wall clock: Model::Run(int) + host argmax on the 0.1B- and 1.5B-shaped models (what the reference's
    bench_model.cpp times), and one 4096-token prompt through Model::Run(vector) on the RWKV-5.2 3B shape cut to 4
    layers (file size; the per-layer work is that of the full model)."""
    import dataclasses
    import tempfile
    import torch
    ref_exe = os.path.join(ROOT, "oracle", "_ref", "fr_ref_cuda_run")
    our_exe = os.path.join(ROOT, "faster-rwkv_b200", "backend", "build", "fr_b200_run")
    if not (os.path.exists(ref_exe) and os.path.exists(our_exe)):
        return {"unavailable": "reference-linked binaries not built (need the reference tree at build time)"}
    synth = pkg.synth
    out = {"timing": "wall clock inside the driver binary (std::chrono around the Run calls)"}
    dev = torch.device("cuda", 0)

    def run(exe, args):
        return subprocess.run([exe] + args, capture_output=True, text=True, timeout=900)

    with tempfile.TemporaryDirectory() as tmp:
        for wl in ("c0", "c1"):
            shape = synth.SHAPES[wl]
            fr = os.path.join(tmp, f"{wl}-fp16.fr")
            synth.write_fr(fr, shape, {n: t.cpu().numpy() for n, t in synth.device_tensors(shape, 0, dev, "fp16")})
            leg = {"workload": f"{wl}: {WORKLOADS[wl][1]}, cuda fp16, batch 1, Model::Run(int) + host argmax", "tokens": n_tokens}
            for key, exe in (("reference_cuda", ref_exe), ("b200_backend", our_exe)):
                try:
                    r = run(exe, [fr, "cuda fp16", os.path.join(tmp, "o.bin"), "--bench", str(n_tokens), "1"])
                    ms = [float(l.split()[1]) for l in r.stdout.splitlines() if l.startswith("ms_per_token")]
                    leg[key] = {"ms_per_token": ms[0], "tok_s": 1e3 / ms[0]} if ms else {"unavailable": (r.stderr or r.stdout)[-200:]}
                except Exception as ex:
                    leg[key] = {"unavailable": str(ex)[:200]}
            if "tok_s" in leg.get("reference_cuda", {}) and "tok_s" in leg.get("b200_backend", {}):
                leg["speedup"] = leg["b200_backend"]["tok_s"] / leg["reference_cuda"]["tok_s"]
            out[wl] = leg
            os.remove(fr)
        # prompt: RWKV-5.2 3B-shaped, 4 layers, T = 4096 through Run(vector)
        shape = dataclasses.replace(synth.SHAPES["c3"], n_layer=4)
        fr = os.path.join(tmp, "c3-L4-fp16.fr")
        synth.write_fr(fr, shape, {n: t.cpu().numpy() for n, t in synth.device_tensors(shape, 0, dev, "fp16")})
        ids = [str(int(t)) for t in synth.token_ids(shape, 4096, seed=1)]
        leg = {"workload": "c3 shape with 4 of 32 layers, one 4096-token prompt, cuda fp16, Model::Run(vector)"}
        for key, exe in (("reference_cuda", ref_exe), ("b200_backend", our_exe)):
            try:
                r = run(exe, [fr, "cuda fp16", os.path.join(tmp, "o.bin"), "--seq", "--time-seq", "3"] + ids)
                ms = [float(l.split()[1]) for l in r.stdout.splitlines() if l.startswith("ms_per_prompt")]
                leg[key] = {"ms_per_prompt": ms[0], "tok_s": 4096e3 / ms[0]} if ms else {"unavailable": (r.stderr or r.stdout)[-200:]}
            except Exception as ex:
                leg[key] = {"unavailable": str(ex)[:200]}
        if "tok_s" in leg.get("reference_cuda", {}) and "tok_s" in leg.get("b200_backend", {}):
            leg["speedup"] = leg["b200_backend"]["tok_s"] / leg["reference_cuda"]["tok_s"]
        out["c3_prompt_L4"] = leg
    return out


# ------------------------------------------------------------------ per-phase budget of the batch-1 kernel

def phase_budget(pkg, device_index: int, wl: str = "c1", reps: int = 5):
    """Medians over layers, CTAs and repetitions of the persistent kernel's own trace (fr_b200_decode_profile), per phase
    kind: ns from phase start to inputs staged (hand-over wait + prologue), staged to row blocks done (tile loop +
    reduce + epilogue), of which waiting for weight tiles, and how far the completion front of the whole grid moves
    per phase (the phase's share of the token)."""
    shape = pkg.synth.SHAPES[wl]
    out = {}
    for fmt, B in (("fp16", 1), ("int8", 1), ("int4", 1), ("fp16", 4), ("int4", 4)):
        m = build_model(pkg, shape, fmt, B, device_index, seed=0)
        ids = [1] * B
        for _ in range(8):
            m.decode(ids)
        info = m.info()
        names = {0: "att_kvr", 1: "att_out", 2: "ffn_kr", 3: "ffn_v"}
        acc = {k: {"prologue_ns": [], "items_ns": [], "tile_wait_cycles": [], "front_ns": [], "wait_inputs_cycles": [],
                   "convert_cycles": [], "stage_cycles": []} for k in list(names.values()) + ["head"]}
        tok = []
        for _ in range(reps):
            st = m.decode_profile(ids).astype(np.int64)          # [cta][phase][8]
            P = st.shape[1]
            done = np.where(st[:, :, 2] > 0, st[:, :, 2], 0).max(axis=0)       # completion front per phase
            start0 = st[:, 0, 0][st[:, 0, 0] > 0].min()
            tok.append(done[-1] - start0)
            for pi in range(P):
                kind = "head" if pi == P - 1 else names[pi % 4]
                act = st[:, pi, 0] > 0
                if not act.any():
                    continue
                a = acc[kind]
                a["prologue_ns"].append(np.median(st[act, pi, 1] - st[act, pi, 0]))
                a["items_ns"].append(np.median(st[act, pi, 2] - st[act, pi, 1]))
                a["tile_wait_cycles"].append(np.median(st[act, pi, 3]))
                a["wait_inputs_cycles"].append(np.median(st[act, pi, 5]))
                a["convert_cycles"].append(np.median(st[act, pi, 6]))
                a["stage_cycles"].append(np.median(st[act, pi, 7]))
                if pi > 0:
                    a["front_ns"].append(done[pi] - done[pi - 1])
        out[f"{fmt}_b{B}"] = {"token_ns": float(np.median(tok)), "n_phases": info["n_phases"], "n_stages": info["n_stages"],
                              "phases": {k: {q: float(np.median(v)) if v else None for q, v in a.items()} for k, a in acc.items()}}
        drop(m)
    return out


# ------------------------------------------------------------------ helpers of the timed legs

def timed_greedy(torch, barrier, m, first_ids, steps, warm):
    """`warm` untimed greedy steps, then exactly `steps` timed ones (CUDA events on the stream the calls use)."""
    m.decode_greedy(first_ids, warm)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = m.info()["launches"]
    e0.record()
    ids = m.decode_greedy(first_ids, steps)
    e1.record()
    barrier()
    return e0.elapsed_time(e1), ids, m.info()["launches"] - l0


def run_prompts(m, shape, synth, stream_ids, n_prompt):
    """A random n_prompt-token prompt for each global stream id (seeded by that id) into slots 0.. ; returns the first
    greedy token of every stream."""
    firsts = []
    for slot, sid in enumerate(stream_ids):
        prompt = [int(t) for t in synth.token_ids(shape, n_prompt, seed=1000 + sid)]
        firsts.append(int(np.argmax(m.run(prompt, slot=slot))))
    return np.asarray(firsts, np.int32)


# ------------------------------------------------------------------ main

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--weights", default=None, choices=["fp16", "int8", "int4"])
    ap.add_argument("--batch", type=int, default=None, help="streams per GPU (single-model workloads); c2: total streams")
    ap.add_argument("--cpu-tokens", type=int, default=24)
    ap.add_argument("--no-variants", action="store_true")
    ap.add_argument("--no-weak", action="store_true")
    ap.add_argument("--prefill-only", action="store_true",
                    help="run only the seq-mode leg (c3, one 4096-token prompt) and print its JSON; for profiling")
    ap.add_argument("--phase-budget", action="store_true", help="print the per-phase budget of the batch-1 kernel (c1)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-ref-gpu", action="store_true")
    ap.add_argument("--steps-only", action="store_true",
                    help="build the model of --workload/--weights/--batch, run --warmup + --steps greedy decode steps and "
                         "print their mean time; nothing else runs (for profiler captures)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    pkg = entry.load_package()
    synth = pkg.synth
    shape = synth.SHAPES[WORKLOADS[args.workload][0]]
    c2 = args.workload == "c2"
    fmt = args.weights or ("int4" if c2 else "fp16")
    total = (args.batch or C2_STREAMS) if c2 else None
    B1 = args.batch or 1
    if c2:
        config = {"workload": f"c2: {WORKLOADS['c2'][1]}, {fmt} weights, {total} streams in total partitioned over the GPUs, "
                              f"{C2_PROMPT}-token prompts then greedy decode",
                  "weights": fmt, "total_streams": total, "prompt_tokens": C2_PROMPT,
                  "parallelism": f"streams partitioned x{world} (full weight replica per GPU, no data-path collective)",
                  "l2": "weights streamed per step exceed L2 (no flush needed)"}
    else:
        config = {"workload": f"{args.workload}: {WORKLOADS[args.workload][1]}, {fmt} weights, {B1} stream(s) per GPU, greedy decode",
                  "weights": fmt, "streams_per_gpu": B1, "parallelism": f"replica x{world}",
                  "l2": "weights streamed per step exceed L2 (no flush needed)"}

    if args.impl == "reference":
        # the reference has no CPU forward of its own (its att/ffn kernels are registered for CUDA and the exporters
        # only); the timed CPU arm is the fp32 oracle port of its op compositions, one stream, on every host core.
        # Under torchrun the launcher exports OMP_NUM_THREADS=1: the thread count is set explicitly.
        if rank != 0:
            return
        n = max(1, min(args.steps, args.cpu_tokens))
        cb = cpu_baseline(shape, "fp32", None, n, threads=os.cpu_count() or 1)
        line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": cb["value"], "unit": "tok/s",
                "n_gpus": args.gpus, "steps": n, "warmup": 1, "ms_per_step": 1e3 / cb["value"],
                "higher_is_better": True, "scaling": "strong" if c2 else "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if args.prefill_only:
        if rank == 0:
            print(json.dumps({"metric": "prefill_tokens_per_s", "n_gpus": 1, "data": "synthetic", **prefill_leg(pkg, local_rank)}))
        return
    if args.steps_only:
        if rank == 0:
            import torch
            torch.cuda.set_device(local_rank)
            n = args.batch or 1
            m = build_model(pkg, shape, fmt, n, local_rank)
            ids = synth.token_ids(shape, n, seed=0)
            ms, _, launches = timed_greedy(torch, torch.cuda.synchronize, m, ids, args.steps, args.warmup)
            print(json.dumps({"metric": "decode_step_ms", "workload": args.workload, "weights": fmt, "streams": n,
                              "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
                              "gpu_launches": int(launches)}))
            drop(m)
        return
    if args.phase_budget:
        if rank == 0:
            print(json.dumps({"metric": "phase_budget", "workload": "c1, batch 1 and 4, persistent kernel",
                              **phase_budget(pkg, local_rank)}))
        return

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    K, W = args.steps, max(args.warmup, 3)
    shard = pkg.shard
    host = {} if (rank == 0 and not args.no_cpu) else None
    extra, check_ok = {}, True

    if c2:
        lo, hi = shard.partition_streams(total, world, rank)
        B = hi - lo
        model = build_model(pkg, shape, fmt, max(B, 1), local_rank, seed=0, keep_host=host)
        t0 = time.perf_counter()
        first = run_prompts(model, shape, synth, range(lo, hi), C2_PROMPT)
        torch.cuda.synchronize()
        prompt_s = max_over_ranks(time.perf_counter() - t0)
        with ClockSampler(local_rank) as cs:
            ms, ids, launches = timed_greedy(torch, barrier, model, first, K, W)
        clocks = cs.summary()
        ms_max = max_over_ranks(ms)
        value = total * K / (ms_max * 1e-3)
        roofline = batched_roofline(shape, fmt, B, ms_max / K)
        extra["streams_per_gpu"] = B
        extra["prompt_phase"] = {"ms": prompt_s * 1e3, "tok_s": total * C2_PROMPT / prompt_s,
                                 "note": "32-token prompts, one stream slot after the other through the GEMM path; not part of `value`"}
        # end to end: host ids in, host arg-max ids out, every step, through the public API
        cur = np.array(first, np.int32)
        for _ in range(W):
            cur = model.decode(cur, want_logits=False, want_argmax=True)
        barrier()
        t0 = time.perf_counter()
        ke = min(K, 64)
        for _ in range(ke):
            cur = model.decode(cur, want_logits=False, want_argmax=True)
        torch.cuda.synchronize()
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        e2e = {"value": total * ke / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B + 4,
               "steps": ke, "call": "Model.decode(ids, want_argmax=True): host ids in, host greedy ids out"}
        # cross-GPU check: rank 0 repeats every other rank's slice (same streams, same batch size, so the same kernels
        # and tiles) and must reproduce its sampled ids exactly
        check = None
        if world > 1:
            n_chk = min(K, 16)
            allv = shard.gather_ids(ids[:n_chk].astype(np.int64), total, world, rank, dist)
            if rank == 0:
                for r in range(1, world):
                    a, b = shard.partition_streams(total, world, r)
                    model.reset_states()
                    f_r = run_prompts(model, shape, synth, range(a, b), C2_PROMPT)
                    model.decode_greedy(f_r, W)
                    again = model.decode_greedy(f_r, n_chk)
                    check_ok = check_ok and np.array_equal(again[:, : b - a], allv[:, a:b])
                check = "sampled ids of every rank's streams reproduced on rank 0" if check_ok else "MISMATCH"
        drop(model)
        del model
        # weak scaling: the full 256 streams on every GPU
        if world > 1 and not args.no_weak:
            mw = build_model(pkg, shape, fmt, total, local_rank, seed=0)
            fw = synth.token_ids(shape, total, seed=rank)
            wms, _, _ = timed_greedy(torch, barrier, mw, fw, min(K, 64), W)
            wms = max_over_ranks(wms)
            extra["weak"] = {"streams_per_gpu": total, "tok_s": world * total * min(K, 64) / (wms * 1e-3),
                             "ms_per_step": wms / min(K, 64),
                             "roofline": batched_roofline(shape, fmt, total, wms / min(K, 64))}
            drop(mw)
            del mw
        scaling = "strong"
    else:
        B = B1
        model = build_model(pkg, shape, fmt, B, local_rank, seed=0, keep_host=host)
        first = synth.token_ids(shape, B, seed=rank)
        model.reset_states()
        with ClockSampler(local_rank) as cs:
            ms, ids, launches = timed_greedy(torch, barrier, model, first, K, W)
        clocks = cs.summary()
        ms_max = max_over_ranks(ms)
        value = world * B * K / (ms_max * 1e-3)
        roofline = hbm_roofline(shape, fmt, ms_max / K, "decode_kernel (persistent, one launch per token)") if B <= 8 else \
            batched_roofline(shape, fmt, B, ms_max / K)
        # end to end: host ids in, host logits out, every step, through the public API
        model.reset_states()
        cur = np.array(first, np.int32)
        for _ in range(W):
            cur = model.decode(cur).argmax(1).astype(np.int32)
        barrier()
        t0 = time.perf_counter()
        ke = min(K, 128)
        for _ in range(ke):
            cur = model.decode(cur).argmax(1).astype(np.int32)
        torch.cuda.synchronize()
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        e2e = {"value": world * B * ke / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 4 * B,
               "d2h_bytes_per_step": 4 * B * shape.vocab + 4 * (B + 1), "steps": ke}
        check = None
        if world > 1:
            n_chk = min(K, 16)
            allv = shard.gather_ids(ids[:n_chk].astype(np.int64), world * B, world, rank, dist)
            if rank == 0:
                for r in range(1, world):
                    model.reset_states()
                    first_r = synth.token_ids(shape, B, seed=r)
                    model.decode_greedy(first_r, W)
                    again = model.decode_greedy(first_r, n_chk)
                    check_ok = check_ok and np.array_equal(again, allv[:, r * B:(r + 1) * B])
                check = "sampled ids of every rank reproduced on rank 0" if check_ok else "MISMATCH"
        extra["kernel_geometry"] = {k: model.info()[k] for k in ("n_ctas", "n_threads", "smem_bytes", "n_stages", "n_phases")}
        drop(model)
        del model
        scaling = "weak"

    variants = {}
    if rank == 0 and world == 1 and not args.no_variants:
        c1 = synth.SHAPES["c1"]
        for vf, vb in (("fp16", 1), ("int8", 1), ("int4", 1), ("int4", 4), ("fp16", 4)):
            try:
                mv = build_model(pkg, c1, vf, vb, local_rank, seed=0)
                steps_v = 256
                vms, _, _ = timed_greedy(torch, barrier, mv, synth.token_ids(c1, vb, seed=0), steps_v, W)
                variants[f"c1_{vf}_b{vb}"] = {"tok_s": vb * steps_v / (vms * 1e-3), "ms_per_step": vms / steps_v,
                                             "roofline": hbm_roofline(c1, vf, vms / steps_v, "decode_kernel (persistent, one launch per token)")}
                drop(mv)
                del mv
            except Exception as ex:  # a variant must not lose the headline
                variants[f"c1_{vf}_b{vb}"] = {"error": str(ex)[:200]}
        for vf, vb in (("int4", 32), ("fp16", 256)):
            try:
                mv = build_model(pkg, c1, vf, vb, local_rank, seed=0)
                vms, _, _ = timed_greedy(torch, barrier, mv, synth.token_ids(c1, vb, seed=0), 64, W)
                variants[f"c1_{vf}_b{vb}"] = {"tok_s": vb * 64 / (vms * 1e-3), "ms_per_step": vms / 64,
                                             "roofline": batched_roofline(c1, vf, vb, vms / 64)}
                drop(mv)
                del mv
            except Exception as ex:
                variants[f"c1_{vf}_b{vb}"] = {"error": str(ex)[:200]}
        variants["prefill_c3_T4096"] = prefill_leg(pkg, local_rank)
        try:
            # configuration 4: RWKV-4 14B-shaped, int8, batch-1 latency (p50 over single greedy steps)
            c4 = synth.SHAPES["c4"]
            mv = build_model(pkg, c4, "int8", 1, local_rank, seed=0)
            mv.decode_greedy([1], 8)
            lat = []
            cur = [1]
            for _ in range(48):
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                cur = [int(mv.decode_greedy(cur, 1)[0, 0])]
                e1.record()
                torch.cuda.synchronize()
                lat.append(e0.elapsed_time(e1))
            p50 = float(np.median(lat))
            variants["c4_int8_b1"] = {"p50_ms_per_token": p50, "tok_s": 1e3 / p50,
                                      "roofline": hbm_roofline(c4, "int8", p50, "decode_kernel (persistent, one launch per token)")}
            drop(mv)
            del mv
        except Exception as ex:
            variants["c4_int8_b1"] = {"error": str(ex)[:200]}

    cb = None
    if host is not None and rank == 0:
        cb = cpu_baseline(shape, FILE_OF[fmt], host, args.cpu_tokens, threads=os.cpu_count() or 1)
    ref_gpu = None
    if rank == 0 and world == 1 and not args.no_ref_gpu and not args.no_variants:
        ref_gpu = reference_gpu_leg(pkg)

    if rank == 0:
        line = {"metric": "decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K,
                "warmup": W, "ms_per_step": ms_max / K, "higher_is_better": True, "scaling": scaling,
                "vs_baseline": None, "dtype": DTYPE_OF[fmt], "data": "synthetic", "config": config, "e2e": e2e,
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "cpu_baseline": cb,
                "variants": variants, **extra}
        if ref_gpu:
            line["reference_gpu"] = ref_gpu
        if check:
            line["cross_gpu_check"] = check
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if not check_ok:
        sys.exit(3)


if __name__ == "__main__":
    main()
