"""GPU parity at the widths, depths and vocabularies of the benchmark configurations, not only on tiny models.

Shape decides which code runs: the register-resident LayerNorm prologue up to n_embd 2048 and the two-pass one above
it, ring depth and slot geometry per width, the padded head rows of an odd vocabulary (50277), how often the
residual stream is halved, how the 8-bit phase tags wrap over 49 / 97 / 161 phases, which stream counts fall to the
GEMM path.  Every case compares the CUDA path with the CPU oracle (the fp32 restatement of
kernels/default/{att,ffn,model_forward}.cpp) on the same seeded weights, at the north star's tolerance: logits and
recurrent state within 1e-2 max-abs and 1e-3 relative L2.

  c0  RWKV-4 0.1B-shaped (L12 C768 F3072 V65536), fp16: 64 prompt ids through Model::Run(vector), then 128 greedy
      tokens at batch 1, logits of every step and the final state; the same file and ids through the reference's own
      kernels/cuda + cuBLAS path ("cuda fp16", rebuilt for sm_100a) where that binary exists
  c1  RWKV-4 1.5B-shaped (L24 C2048 F8192 V65536), fp16 / int8 / int4: 32 tokens at batch 1, 4 streams in one
      launch of the persistent kernel, 16 streams through the GEMM path
  c3  RWKV-5.2 3B-shaped at full width (C2560 H40 F8960 V65536) with 4 of its 32 layers: one 4096-token prompt
      against the oracle's token loop, then 64 decode steps
  c4  RWKV-4 14B-shaped at full width (C5120 F20480 V50277) with 7 of its 40 layers (one halving of the residual
      stream happens), int8: 32 tokens at batch 1
The measured distances go to parity_shapes.json in the run's output directory beside the assertions.
"""
import dataclasses
import json
import os
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_CUDA = os.path.join(ROOT, "oracle", "_ref", "fr_ref_cuda_run")
ABS_TOL, REL_TOL = 1e-2, 1e-3
FILE_OF = {"fp16": "fp16", "int8": "fp32", "int4": "fp32"}
REPORT = {}


def _dist(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max()), float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _close(got, want, what):
    err, rel = _dist(got, want)
    assert err < ABS_TOL and rel < REL_TOL, f"{what}: max-abs {err:.3e}, rel-L2 {rel:.3e}"
    return err, rel


def _note(key, **kw):
    REPORT.setdefault(key, {}).update(kw)
    out = os.path.join(ROOT, "gpurun_out")
    os.makedirs(out, exist_ok=True)
    with open(os.path.join(out, "parity_shapes.json"), "w") as f:
        json.dump(REPORT, f, indent=1, sort_keys=True)


def _build(pkg, orc, shape, fmt, max_batch=1, seed=0):
    """(model on the GPU, oracle on the host) over the same tensors, drawn on the GPU."""
    import torch
    host = {}

    class Feed:
        def items(self):
            for name, t in pkg.synth.device_tensors(shape, seed, torch.device("cuda", 0), FILE_OF[fmt]):
                host[name] = t.cpu().numpy()
                yield name, t
    m = pkg.Model(Feed(), f"cuda {fmt}", shape=shape, max_batch=max_batch)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    ref = orc.OracleModel(shape, host, pkg.synth.param_names(shape), rescale_every=6 if fmt == "fp16" else 0,
                          weight_format=fmt, state_fp16=fmt == "fp16")
    return m, ref, host


def _state_check(m, ref, shape, what, slot=0):
    """Recurrent state of one stream against the oracle's; returns the worst distances (max-abs relative to the
    largest entry for the two running sums aa and bb)."""
    st = m.states(slot)
    C, worst = shape.n_embd, (0.0, 0.0)
    if str(shape.version) == "4":
        want = ref.state_v4()
        for l in range(shape.n_layer):
            for j in range(5):
                if j == 3:
                    # pp starts at -1e30 and follows max(pp + w, k): compare where it has left the initial value
                    live = want[l, j] > -1e29
                    d = _close(st[l][j][live], want[l, j][live], f"{what} pp[{l}]")
                elif j in (1, 2):
                    # aa and bb are running sums of exp-weighted values: they grow with the number of tokens, so the
                    # max-abs bound scales with their largest entry (the relative L2 bound does not)
                    e, r = _dist(st[l][j], want[l, j])
                    big = max(1.0, float(np.abs(want[l, j]).max()))
                    assert r < REL_TOL and e < ABS_TOL * big, f"{what} state[{l}][{j}]: max-abs {e:.3e} (largest entry {big:.1f}), rel-L2 {r:.3e}"
                    d = (e / big, r)
                else:
                    d = _close(st[l][j].astype(np.float32), want[l, j], f"{what} state[{l}][{j}]")
                worst = (max(worst[0], d[0]), max(worst[1], d[1]))
    return worst


# --------------------------------------------------------------------------------------------- c0

def test_c0_prompt_then_greedy_per_step(pkg, orc, synth, tmp_path):
    """BASELINE configuration 0 as written: 64 seeded prompt ids, 128 greedy tokens at batch 1, per-step logits.
    Both sides are fed the oracle's greedy choice, so one near-tie cannot send the two runs down different paths."""
    shape = synth.SHAPES["c0"]
    m, ref, host = _build(pkg, orc, shape, "fp16")
    prompt = [int(t) for t in synth.token_ids(shape, 64, seed=100)]
    got, want = m.run(prompt), ref.run_seq(prompt)
    worst = list(_close(got, want, "c0 prompt"))
    ours, exact, fed = [got], [want], list(prompt)
    for step in range(128):
        tok = int(np.argmax(want))
        fed.append(tok)
        got, want = m.run(tok), ref.run(tok)
        d = _close(got, want, f"c0 greedy step {step}")
        worst = [max(worst[0], d[0]), max(worst[1], d[1])]
        ours.append(got)
        exact.append(want)
    sd = _state_check(m, ref, shape, "c0")
    _note("c0_fp16", logits_max_abs=worst[0], logits_rel_l2=worst[1], state_max_abs=sd[0], state_rel_l2=sd[1],
          steps="64-token prompt + 128 greedy tokens")
    m.close()
    if not os.path.exists(REF_CUDA):
        _note("c0_fp16", reference_cuda="binary not built (needs the reference tree at build time)")
        return
    # the reference's own CUDA path on the same file and the same ids, token by token (it has no RWKV-4 seq mode,
    # kernels/default/model_forward_seq.cpp:111-112)
    fr = str(tmp_path / "c0-fp16.fr")
    synth.write_fr(fr, shape, host)
    out = str(tmp_path / "ref.bin")
    r = subprocess.run([REF_CUDA, fr, "cuda fp16", out] + [str(t) for t in fed[:-1]], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-400:]
    theirs = np.fromfile(out, np.float32).reshape(len(fed) - 1, shape.vocab)[63:]      # rows of the compared steps
    ours, exact = np.stack(ours[:-1]), np.stack(exact[:-1])
    d_ours = max(_dist(a, b)[1] for a, b in zip(ours, exact))
    d_theirs = max(_dist(a, b)[1] for a, b in zip(theirs, exact))
    pair = [_dist(a, b) for a, b in zip(ours, theirs)]
    p_abs, p_rel = max(p[0] for p in pair), max(p[1] for p in pair)
    _note("c0_fp16", rel_l2_ours_vs_fp32=d_ours, rel_l2_reference_cuda_vs_fp32=d_theirs, rel_l2_ours_vs_reference_cuda=p_rel,
          max_abs_ours_vs_reference_cuda=p_abs, pair_within_1e2_1e3=bool(p_abs < ABS_TOL and p_rel < REL_TOL))
    assert d_ours < REL_TOL and d_ours <= d_theirs
    # the two CUDA paths are apart by what the reference loses when it rounds every activation to fp16
    assert p_rel < d_theirs + d_ours + 1e-4
    assert p_abs < 3e-2


# --------------------------------------------------------------------------------------------- c1

@pytest.mark.parametrize("fmt", ["fp16", "int8", "int4"])
def test_c1_batch1_four_streams_and_sixteen_streams(pkg, orc, synth, fmt):
    shape = synth.SHAPES["c1"]
    m, ref, _ = _build(pkg, orc, shape, fmt, max_batch=16)
    # 32 tokens at batch 1 through the persistent kernel (one stream)
    ids = synth.token_ids(shape, 32, seed=7)
    worst = [0.0, 0.0]
    for i, t in enumerate(ids):
        d = _close(m.run(int(t)), ref.run(int(t)), f"c1 {fmt} step {i}")
        worst = [max(worst[0], d[0]), max(worst[1], d[1])]
    sd = _state_check(m, ref, shape, f"c1 {fmt}")
    _note(f"c1_{fmt}", b1_logits_max_abs=worst[0], b1_logits_rel_l2=worst[1], b1_state_max_abs=sd[0], b1_state_rel_l2=sd[1])
    # 4 streams in one launch of the persistent kernel, 5 steps; streams 0 and 3 checked
    m.reset_states()
    ids4 = synth.token_ids(shape, 20, seed=8).reshape(5, 4)
    got = [m.decode(ids4[t]) for t in range(5)]
    w4 = [0.0, 0.0]
    for b in (0, 3):
        ref.reset()
        for t in range(5):
            d = _close(got[t][b], ref.run(int(ids4[t, b])), f"c1 {fmt} 4 streams: stream {b} step {t}")
            w4 = [max(w4[0], d[0]), max(w4[1], d[1])]
    # 16 streams through the GEMM path (one row per stream), 4 steps; streams 0, 7 and 15 checked
    m.reset_states()
    ids16 = synth.token_ids(shape, 64, seed=9).reshape(4, 16)
    got = [m.decode(ids16[t]) for t in range(4)]
    w16 = [0.0, 0.0]
    for b in (0, 7, 15):
        ref.reset()
        for t in range(4):
            d = _close(got[t][b], ref.run(int(ids16[t, b])), f"c1 {fmt} 16 streams: stream {b} step {t}")
            w16 = [max(w16[0], d[0]), max(w16[1], d[1])]
    _note(f"c1_{fmt}", b4_logits_max_abs=w4[0], b4_logits_rel_l2=w4[1], b16_logits_max_abs=w16[0], b16_logits_rel_l2=w16[1])
    m.close()


# --------------------------------------------------------------------------------------------- c3

def test_c3_width_prompt_4096_then_decode(pkg, orc, synth):
    """Full width of the RWKV-5.2 3B shape, 4 of its 32 layers (the oracle walks the prompt token by token)."""
    shape = dataclasses.replace(synth.SHAPES["c3"], n_layer=4)
    m, ref, _ = _build(pkg, orc, shape, "fp16")
    prompt = [int(t) for t in synth.token_ids(shape, 4096, seed=21)]
    got, want = m.run(prompt), ref.run_seq(prompt)
    d = _close(got, want, "c3 prompt logits")
    # recurrent state after 4096 tokens.  The per-head state sums k v^T over the prompt and reaches tens in magnitude:
    # its bound is 1e-2 of its largest entry; the absolute distance is recorded beside it.
    st = m.states()
    C, H = shape.n_embd, shape.n_head
    per = 2 * C + H * 4096
    s_abs = s_rel = s_scaled = 0.0
    for l in range(shape.n_layer):
        blk = ref.state[l * per:(l + 1) * per]
        _close(st[l][0].astype(np.float32), blk[:C], f"c3 sx[{l}]")
        _close(st[l][2].astype(np.float32), blk[C + H * 4096:], f"c3 ffn_sx[{l}]")
        s_want = blk[C:C + H * 4096]
        e, r = _dist(st[l][1].reshape(-1), s_want)
        assert r < REL_TOL and e < ABS_TOL * max(1.0, float(np.abs(s_want).max())), f"c3 s[{l}]: max-abs {e:.3e}, rel-L2 {r:.3e}"
        s_abs, s_rel, s_scaled = max(s_abs, e), max(s_rel, r), max(s_scaled, e / max(1.0, float(np.abs(s_want).max())))
    _note("c3_fp16_L4", prompt_tokens=4096, logits_max_abs=d[0], logits_rel_l2=d[1], state_max_abs=s_abs, state_rel_l2=s_rel,
          state_max_abs_over_largest_entry=s_scaled, state_within_absolute_1e2=bool(s_abs < ABS_TOL))
    worst = [0.0, 0.0]
    for step in range(64):
        tok = int(np.argmax(want))
        got, want = m.run(tok), ref.run(tok)
        dd = _close(got, want, f"c3 decode step {step}")
        worst = [max(worst[0], dd[0]), max(worst[1], dd[1])]
    _note("c3_fp16_L4", decode_logits_max_abs=worst[0], decode_logits_rel_l2=worst[1])
    m.close()


# --------------------------------------------------------------------------------------------- c4

def test_c4_width_int8_odd_vocab(pkg, orc, synth):
    """Full width of the RWKV-4 14B shape (two-pass LayerNorm prologue, 20480-wide channel mix, vocabulary 50277 ->
    padded head rows), 7 of its 40 layers, int8 weights."""
    shape = dataclasses.replace(synth.SHAPES["c4"], n_layer=7)
    m, ref, _ = _build(pkg, orc, shape, "int8")
    ids = synth.token_ids(shape, 32, seed=5)
    worst = [0.0, 0.0]
    for i, t in enumerate(ids):
        got = m.run(int(t))
        assert got.shape == (50277,)
        d = _close(got, ref.run(int(t)), f"c4 int8 step {i}")
        worst = [max(worst[0], d[0]), max(worst[1], d[1])]
    sd = _state_check(m, ref, shape, "c4 int8")
    _note("c4_int8_L7", logits_max_abs=worst[0], logits_rel_l2=worst[1], state_max_abs=sd[0], state_rel_l2=sd[1])
    # the same model under fp16 activations halves the residual stream after layer 6: run that variant too
    m.close()
    del m, ref
    m, ref, _ = _build(pkg, orc, shape, "fp16")
    worst = [0.0, 0.0]
    for i, t in enumerate(ids[:12]):
        d = _close(m.run(int(t)), ref.run(int(t)), f"c4 fp16 step {i}")
        worst = [max(worst[0], d[0]), max(worst[1], d[1])]
    _note("c4_fp16_L7", logits_max_abs=worst[0], logits_rel_l2=worst[1])
    m.close()
