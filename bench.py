#!/usr/bin/env python3
"""Decode benchmark of the B200 RWKV backend.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--weights fp16|int8|int4] [--batch B]
  python bench.py --impl reference ...        # CPU fp32 path timed on the host cores

A step = one decoded token for each of B independent streams of an RWKV-4 1.5B-shaped model
(24 layers, n_embd 2048, FFN 8192, vocab 65536) with seeded random weights.  `value` is tokens/s
with the token ids staying on the device (greedy feedback on the GPU); `e2e` goes through the
public Model.decode call with host ids in and host logits out every step.  With --gpus N each rank
runs its own replica on its own streams (no collective on the data path); NCCL only gathers the
sampled ids for the cross-GPU check after the timed region.
"""
from __future__ import annotations

import argparse
import json
import math
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
    "c1": ("c1", "RWKV-4 1.5B-shaped (L24 C2048 F8192 V65536), decode"),
    "c0": ("c0", "RWKV-4 0.1B-shaped (L12 C768 F3072 V65536), decode"),
    "c3": ("c3", "RWKV-5.2 3B-shaped (L32 C2560 F8960 H40 V65536), decode"),
    "c4": ("c4", "RWKV-4 14B-shaped (L40 C5120 F20480 V50277), decode"),
    "tiny": ("tiny4b", "tiny RWKV-4 (L7 C192 F448 V211)"),
}
FILE_DTYPE = {"fp16": "fp16", "int8": "fp32", "int4": "fp32"}


def algorithmic_bytes(shape, fmt: str) -> int:
    """Bytes of projection weights (+ quantisation scales) one token must read: every matvec weight once."""
    C, F, V, L = shape.n_embd, shape.n_ffn, shape.vocab, shape.n_layer
    att = 5 if str(shape.version) in ("4", "5") else 6
    P = L * (att * C * C + 2 * C * F) + C * V
    rows = L * (att * C + F + C) + V          # output rows (one int8 scale each)
    if fmt == "fp16":
        return 2 * P
    if fmt == "int8":
        return P + 2 * rows
    return P // 2 + 2 * (P // 32)


# DRAM bytes per decode_kernel launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu capture summarised
# in profiles/decode_kernel_c1_fp16_launch_list.md; other workloads have no capture yet.
MEASURED_TRAFFIC = {("c1", "fp16", 1): 2_891_602_330}


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ------------------------------------------------------------------ synthetic weights on the GPU

def gpu_master_weights(shape, seed: int, device):
    """Yield (name, fp32 CUDA tensor) with the distributions of faster-rwkv_b200/synth.py, generated on the device."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    C, F, V, L = shape.n_embd, shape.n_ffn, shape.vocab, shape.n_layer

    def mat(k, n):
        return torch.randn(k, n, generator=g, device=device, dtype=torch.float32) / math.sqrt(k)

    def uni(n, lo, hi):
        return torch.rand(n, generator=g, device=device, dtype=torch.float32) * (hi - lo) + lo

    yield "emb.weight", torch.randn(V, C, generator=g, device=device, dtype=torch.float32)
    for i in range(L):
        b, a, f = f"blocks.{i}.", f"blocks.{i}.att.", f"blocks.{i}.ffn."
        for ln in (b + "ln1", b + "ln2"):
            yield ln + ".weight", torch.ones(C, device=device)
            yield ln + ".bias", torch.zeros(C, device=device)
        v5 = str(shape.version).startswith("5")
        gate = str(shape.version) in ("5.1", "5.2")
        if v5:
            yield a + "ln_x.weight", torch.ones(C, device=device)
            yield a + "ln_x.bias", torch.zeros(C, device=device)
        for m in ("k", "v", "r") + (("g",) if gate else ()):
            yield a + "time_mix_" + m, uni(C, 0, 1)
        if not v5:
            yield a + "time_decay", -torch.exp(uni(C, -6, 1))
            yield a + "time_first", uni(C, -1, 1)
        elif str(shape.version) == "5":
            yield a + "time_decay", torch.exp(-torch.exp(uni(shape.n_head, -6, 1))).reshape(shape.n_head, 1, 1)
            yield a + "time_first", uni(shape.n_head, -1, 1).reshape(shape.n_head, 1, 1)
        else:
            yield a + "time_decay", torch.exp(-torch.exp(uni(C, -6, 1))).reshape(shape.n_head, C // shape.n_head, 1)
            yield a + "time_first", uni(C, -1, 1).reshape(shape.n_head, C // shape.n_head, 1)
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


def build_model(pkg, shape, fmt: str, max_batch: int, device_index: int, seed: int = 0, keep_host=None):
    """Model with seeded weights generated on the GPU; fp16 files get the 2**(layer//6) pre-division."""
    import torch
    dev = torch.device("cuda", device_index)

    # Model() walks tensors.items() once; a generator-backed feed keeps peak memory low
    class Feed:
        def items(self_inner):
            for name, t in gpu_master_weights(shape, seed, dev):
                if keep_host is not None:
                    keep_host[name] = t.cpu().numpy()
                if fmt == "fp16" and not name.endswith(("time_decay", "time_first", "ln_x.weight", "ln_x.bias")):
                    if name.endswith(("att.output.weight", "ffn.value.weight")):
                        t = t / float(2 ** (int(name.split(".")[1]) // 6))
                    t = t.half()
                yield name, t
    m = pkg.Model(Feed(), f"cuda {fmt}", max_batch=max_batch, device=device_index, shape=shape)
    torch.cuda.synchronize(dev)
    return m


# ------------------------------------------------------------------ seq mode (prompt processing)

def measured_peak_tflops():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    except Exception:
        return 1590.0, 1400.0, "fallback"


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
        burst, sustained, kind = measured_peak_tflops()
        tf = flops / (best * 1e-3) / 1e12
        out = {"workload": "c3: RWKV-5.2 3B-shaped (L32 C2560 F8960 H40 V65536), one 4096-token prompt, fp16 weights",
               "ms": best, "tok_s": T / (best * 1e-3), "tflops": tf, "tensor_frac_of_burst_peak": tf / burst,
               "tensor_frac_of_sustained_peak": tf / sustained, "peak_source": kind,
               "algorithmic_flops": flops}
        m.close()
        del m
        torch.cuda.empty_cache()
        # 16 streams: one prompt each (slot by slot: a 4096-token prompt already fills the tensor cores), then 64
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
            m.close()
            del m
            torch.cuda.empty_cache()
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

def cpu_baseline(shape, host_master, n_tokens: int, seed: int = 0):
    """The fp32 CPU path (oracle port of the reference's op compositions) on all host threads."""
    orc = entry.load_oracle()
    orc.build()
    pkg = entry.load_package()
    if host_master is None:
        host_master = pkg.synth.generate(shape, seed)
    m = orc.OracleModel(shape, host_master, pkg.synth.param_names(shape))
    ids = pkg.synth.token_ids(shape, n_tokens + 1, seed)
    m.run(int(ids[0]))  # warm-up: page in the weights
    t0 = time.perf_counter()
    for t in ids[1:]:
        m.run(int(t))
    dt = time.perf_counter() - t0
    return {"value": n_tokens / dt, "unit": "tok/s", "cores": orc.lib().orc_num_threads(), "kind": "port",
            "sample": f"{n_tokens} tokens, batch 1, fp32 weights, same model shape ({dt:.1f} s)"}


# ------------------------------------------------------------------ reference GPU path, same driver binary

def reference_gpu_leg(pkg, n_tokens: int = 256):
    """The reference's own kernels/cuda + cuBLAS ("cuda fp16", rebuilt for sm_100a: oracle/_ref/fr_ref_cuda_run) and
    this backend behind the same unchanged rwkv::Model (faster-rwkv_b200/backend/build/fr_b200_run), both timed
    through Model::Run(int) + host argmax on the 0.1B-shaped model the reference's bench_model.cpp uses."""
    import tempfile
    ref_exe = os.path.join(ROOT, "oracle", "_ref", "fr_ref_cuda_run")
    our_exe = os.path.join(ROOT, "faster-rwkv_b200", "backend", "build", "fr_b200_run")
    if not (os.path.exists(ref_exe) and os.path.exists(our_exe)):
        return {"unavailable": "reference-linked binaries not built (need the reference tree at build time)"}
    synth = pkg.synth
    shape = synth.SHAPES["c0"]
    out = {"workload": "c0: RWKV-4 0.1B-shaped, cuda fp16, batch 1, Model::Run(int) + host argmax, wall clock",
           "tokens": n_tokens}
    with tempfile.TemporaryDirectory() as tmp:
        fr = os.path.join(tmp, "c0-fp16.fr")
        synth.write_fr(fr, shape, synth.to_file_dtypes(shape, synth.generate(shape, seed=0), "fp16"))
        for key, exe in (("reference_cuda", ref_exe), ("b200_backend", our_exe)):
            try:
                r = subprocess.run([exe, fr, "cuda fp16", os.path.join(tmp, "o.bin"), "--bench", str(n_tokens), "1"],
                                   capture_output=True, text=True, timeout=600)
                ms = [float(l.split()[1]) for l in r.stdout.splitlines() if l.startswith("ms_per_token")]
                out[key] = {"ms_per_token": ms[0], "tok_s": 1e3 / ms[0]} if ms else {"error": (r.stderr or r.stdout)[-200:]}
            except Exception as ex:
                out[key] = {"error": str(ex)[:200]}
    if "tok_s" in out.get("reference_cuda", {}) and "tok_s" in out.get("b200_backend", {}):
        out["speedup"] = out["b200_backend"]["tok_s"] / out["reference_cuda"]["tok_s"]
    return out


# ------------------------------------------------------------------ main

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c1", choices=sorted(WORKLOADS))
    ap.add_argument("--weights", default="fp16", choices=["fp16", "int8", "int4"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--cpu-tokens", type=int, default=24)
    ap.add_argument("--no-variants", action="store_true")
    ap.add_argument("--prefill-only", action="store_true",
                    help="run only the seq-mode leg (c3, one 4096-token prompt) and print its JSON; for profiling")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-ref-gpu", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    pkg = entry.load_package()
    shape = pkg.synth.SHAPES[WORKLOADS[args.workload][0]]
    config = {"workload": f"{args.workload}: {WORKLOADS[args.workload][1]}, {args.weights} weights, "
                          f"{args.batch} stream(s) per GPU, greedy decode",
              "weights": args.weights, "streams_per_gpu": args.batch, "parallelism": f"replica x{world}",
              "l2": "weights streamed per step exceed L2 (no flush needed)"}

    if args.impl == "reference":
        # the reference has no CPU forward of its own (its att/ffn kernels are registered for CUDA and
        # the exporters only); the timed CPU arm is the fp32 oracle port of its op compositions
        if rank != 0:
            return
        n = max(1, min(args.steps, args.cpu_tokens))
        cb = cpu_baseline(shape, None, n)
        line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": cb["value"], "unit": "tok/s",
                "n_gpus": args.gpus, "steps": n, "warmup": 1, "ms_per_step": 1e3 / cb["value"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if args.prefill_only:
        if rank == 0:
            print(json.dumps({"metric": "prefill_tokens_per_s", "n_gpus": 1, "data": "synthetic", **prefill_leg(pkg, local_rank)}))
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

    K, W, B = args.steps, max(args.warmup, 3), args.batch
    host_master = {} if (rank == 0 and world == 1 and not args.no_cpu) else None
    model = build_model(pkg, shape, args.weights, B, local_rank, seed=0, keep_host=host_master)
    first = pkg.synth.token_ids(shape, B, seed=rank)

    def timed_greedy(m, first_ids, steps, warm):
        m.reset_states()
        m.decode_greedy(first_ids, warm)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = m.info()["launches"]
        e0.record()
        ids = m.decode_greedy(first_ids, steps)
        e1.record()
        barrier()
        return e0.elapsed_time(e1), ids, m.info()["launches"] - l0

    with ClockSampler(local_rank) as cs:
        ms, ids, launches = timed_greedy(model, first, K, W)
    clocks = cs.summary()
    t = torch.tensor([ms], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    value = world * B * K / (ms_max * 1e-3)

    # end to end: host ids in, host logits out, every step, through the public API
    model.reset_states()
    cur = np.array(first, np.int32)
    for _ in range(W):
        cur = model.decode(cur).argmax(1).astype(np.int32)
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        logits = model.decode(cur)
        cur = logits.argmax(1).astype(np.int32)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e = {"value": world * B * K / float(t.item()), "unit": "tok/s", "h2d_bytes_per_step": 4 * B,
           "d2h_bytes_per_step": 4 * B * shape.vocab + 4 * (B + 1)}

    # cross-GPU check: every replica started from its own ids; rank r's run must equal a rerun on rank 0
    check = None
    if world > 1:
        mine = torch.tensor(ids[: min(K, 16)].astype(np.int64), device="cuda")
        allv = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allv, mine)
        if rank == 0:
            ok = True
            for r in range(1, world):
                model.reset_states()
                first_r = pkg.synth.token_ids(shape, B, seed=r)
                model.decode_greedy(first_r, W)          # the timed run followed W warm-up tokens from the same start
                again = model.decode_greedy(first_r, min(K, 16))
                ok = ok and np.array_equal(again, allv[r].cpu().numpy())
            check = "sampled ids of every rank reproduced on rank 0" if ok else "MISMATCH"

    info = model.info()
    algo = algorithmic_bytes(shape, args.weights)
    peak, peak_kind = measured_peak_gbs()
    achieved = algo * K / (ms_max * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": MEASURED_TRAFFIC.get((args.workload, args.weights, B)), "peak_source": peak_kind,
                "kernel": "decode_kernel (persistent, one launch per token)" if B <= 8 else
                          "gemm_wt_kernel + row kernels (one row per stream; two steps replayed as a CUDA graph)",
                "algorithmic_bytes_per_launch": algo}

    variants = {}
    if rank == 0 and world == 1 and not args.no_variants:
        del model
        torch.cuda.empty_cache()
        for fmt, vb in (("fp16", 1), ("int8", 1), ("int4", 1), ("int4", 4), ("fp16", 4)):
            if fmt == args.weights and vb == B:
                variants[f"{fmt}_b{vb}"] = {"tok_s": value, "hbm_frac": achieved / peak}
                continue
            try:
                mv = build_model(pkg, shape, fmt, vb, local_rank, seed=0)
                vms, _, _ = timed_greedy(mv, pkg.synth.token_ids(shape, vb, seed=0), min(K, 256), W)
                steps_v = min(K, 256)
                gbs = algorithmic_bytes(shape, fmt) * steps_v / (vms * 1e-3) / 1e9
                variants[f"{fmt}_b{vb}"] = {"tok_s": vb * steps_v / (vms * 1e-3), "ms_per_step": vms / steps_v,
                                            "hbm_gbs": gbs, "hbm_frac": gbs / peak}
                mv.close()
                del mv
                torch.cuda.empty_cache()
            except Exception as ex:  # a variant must not lose the headline
                variants[f"{fmt}_b{vb}"] = {"error": str(ex)[:200]}

        variants["prefill_c3_T4096"] = prefill_leg(pkg, local_rank)
        # many streams at once: one row per stream through the tensor-core GEMM path (c2-shaped: int4 weights, 256 streams)
        for fmt, vb in (("int4", 256), ("fp16", 256)):
            try:
                mv = build_model(pkg, shape, fmt, vb, local_rank, seed=0)
                vms, _, _ = timed_greedy(mv, pkg.synth.token_ids(shape, vb, seed=0), 32, W)
                P = algorithmic_bytes(shape, "fp16") // 2          # projection parameters
                tf = 2.0 * P * vb * 32 / (vms * 1e-3) / 1e12
                variants[f"{fmt}_b{vb}_gemm"] = {"tok_s": vb * 32 / (vms * 1e-3), "ms_per_step": vms / 32, "tflops": tf,
                                                 "note": "weights held as fp16 W^T (dequantised) for the GEMM path"}
                mv.close()
                del mv
                torch.cuda.empty_cache()
            except Exception as ex:
                variants[f"{fmt}_b{vb}_gemm"] = {"error": str(ex)[:200]}

    cb = None
    if host_master is not None:
        cb = cpu_baseline(shape, host_master, args.cpu_tokens)
    ref_gpu = None
    if rank == 0 and world == 1 and not args.no_ref_gpu and args.workload == "c1":
        ref_gpu = reference_gpu_leg(pkg)

    if rank == 0:
        line = {"metric": "decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K,
                "warmup": W, "ms_per_step": ms_max / K, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": {"fp16": "f16", "int8": "i8->f16 x f16 (f32 acc)",
                                               "int4": "i4->f16 x f16 (f32 acc)"}[args.weights],
                "data": "synthetic", "config": config, "e2e": e2e, "gpu_launches": int(launches),
                "clocks": clocks, "roofline": roofline, "cpu_baseline": cb, "variants": variants,
                "kernel_geometry": {k: info[k] for k in ("n_ctas", "n_threads", "smem_bytes", "n_stages", "n_phases")}}
        if ref_gpu:
            line["reference_gpu"] = ref_gpu
        if check:
            line["cross_gpu_check"] = check
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
