"""GPU parity of decode for more than 8 streams at once (the batched decode the reference lacks): one row per stream
through the tensor-core GEMM path, every weight format and model version, against the CPU oracle run stream by
stream.  fp16 models created for such batches keep W^T copies, quantised models a row-major copy of their packed
codes (expanded inside the GEMM); their prompts use the same path."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ABS_TOL, REL_TOL = 1e-2, 1e-3
STR = {"fp16": ("cuda fp16", "fp16"), "int8": ("cuda int8", "fp32"), "int4": ("cuda int4", "fp32")}


def _pair(pkg, orc, synth, name, fmt, B):
    shape = synth.SHAPES[name]
    strat, fdt = STR[fmt]
    tensors = synth.to_file_dtypes(shape, synth.generate(shape, seed=11, ln_random=True), fdt)
    ref = orc.OracleModel(shape, tensors, synth.param_names(shape), rescale_every=6 if fmt == "fp16" else 0,
                          weight_format=fmt, state_fp16=fmt == "fp16")
    m = pkg.Model(tensors, strat, shape=shape, max_batch=B)
    return shape, m, ref


def _close(got, want, what):
    err = float(np.abs(got - want).max())
    rel = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
    assert err < ABS_TOL and rel < REL_TOL, f"{what}: max-abs {err:.3e}, rel-L2 {rel:.3e}"


@pytest.mark.parametrize("name,fmt,B", [("tiny4", "fp16", 12), ("tiny4b", "int8", 20), ("tiny4", "int4", 16),
                                        ("tiny52", "fp16", 12), ("tiny50", "int8", 9), ("tiny51", "int4", 10),
                                        ("mid4", "fp16", 40), ("mid52", "int4", 150), ("mid4", "int8", 100),
                                        ("mid4", "int4", 300), ("mid52", "fp16", 70)])
def test_many_streams_match_oracle(pkg, orc, synth, name, fmt, B):
    """Stream b of a B-stream decode == the oracle fed stream b's tokens.  The stream counts walk the few-row GEMM's
    tile widths: 32 (up to 32 streams), 64, 128, 256, and two 256-stream tiles (300 streams)."""
    shape, m, ref = _pair(pkg, orc, synth, name, fmt, B)
    steps = 4
    ids = synth.token_ids(shape, steps * B, seed=9).reshape(steps, B)
    got = [m.decode(ids[t]) for t in range(steps)]
    for b in list(range(min(B, 6))) + ([B // 2 + 1] if B > 64 else []) + [B - 1]:
        ref.reset()
        for t in range(steps):
            _close(got[t][b], ref.run(int(ids[t, b])), f"{name} {fmt} stream {b} step {t}")
    m.close()


@pytest.mark.parametrize("fmt", ["fp16", "int4"])
def test_eight_streams_of_a_wide_model_take_the_gemm_path(pkg, orc, synth, fmt):
    """A model whose channel-mix width does not leave room for 8 streams in the persistent kernel's shared memory
    (8 x 8192 inputs) is still created with max_batch = 8: batches of 5..8 are decoded by the GEMM path, 1..4 by the
    persistent kernel, on the same state."""
    shape, m, ref = _pair(pkg, orc, synth, "wide4", fmt, 8)
    ids = synth.token_ids(shape, 3 * 8, seed=21).reshape(3, 8)
    got = [m.decode(ids[0]), m.decode(ids[1]), m.decode(ids[2][:3])]   # 8, 8, then 3 streams
    for b in (0, 2, 7):
        ref.reset()
        for t in range(3):
            if t == 2 and b >= 3:
                break
            _close(got[t][b], ref.run(int(ids[t, b])), f"wide4 {fmt} stream {b} step {t}")
    m.close()


def test_small_and_large_batches_share_state(pkg, orc, synth):
    """The persistent kernel (<= 8 streams) and the GEMM path (> 8) read and write the same state slots, and streams
    that are decoded together need not have seen the same number of tokens (continuous batching: a stream joins a
    running batch after a reset, a prompt of its own or a few extra steps)."""
    for name in ("tiny4", "tiny52"):
        shape, m, ref = _pair(pkg, orc, synth, name, "fp16", 12)
        ids = synth.token_ids(shape, 48, seed=3).reshape(4, 12)
        fed = [[] for _ in range(12)]

        def step(row, streams):
            got = m.decode(ids[row][:streams])
            for b in range(streams):
                fed[b].append(int(ids[row, b]))
            return got
        step(0, 12)                      # 12 streams: GEMM path
        step(1, 4)                       # streams 0..3 one token further: persistent kernel
        got = step(2, 12)                # all together again, 0..3 a token ahead of 4..11
        m.reset_states(5)                # stream 5 starts over while the others are an odd number of tokens in
        fed[5] = []
        got = step(3, 12)
        for b in (0, 3, 4, 5, 11):
            ref.reset()
            for t in fed[b]:
                want = ref.run(t)
            _close(got[b], want, f"{name} stream {b} after {len(fed[b])} tokens")
        # the same through the persistent kernel: streams 0..5, stream 5 one reset behind
        m.reset_states(2)
        fed[2] = []
        got = step(0, 6)
        for b in (1, 2, 5):
            ref.reset()
            for t in fed[b]:
                want = ref.run(t)
            _close(got[b], want, f"{name} stream {b} (persistent kernel) after {len(fed[b])} tokens")
        m.close()


def test_greedy_many_streams_on_device(pkg, orc, synth):
    """decode_greedy for 16 streams == Run -> argmax -> Run on the host."""
    shape, m, ref = _pair(pkg, orc, synth, "tiny4b", "fp16", 16)
    first = [int(t) for t in synth.token_ids(shape, 16, seed=1)]
    got = m.decode_greedy(first, 5)
    m.reset_states()
    cur = np.array(first, np.int32)
    for t in range(5):
        cur = m.decode(cur).argmax(1).astype(np.int32)
        assert np.array_equal(cur, got[t])
    m.close()


@pytest.mark.parametrize("name,fmt", [("tiny4b", "fp16"), ("tiny4", "int4"), ("tiny52", "int8")])
def test_prompts_of_any_model_use_the_rows_path(pkg, orc, synth, name, fmt, monkeypatch):
    """With the W^T copies present, RWKV-4 and quantised models process prompts as GEMMs too (RWKV-4 WKV scanned per
    channel); result and state must match the oracle's token loop."""
    monkeypatch.setenv("FR_B200_SEQ_MIN", "2")
    shape, m, ref = _pair(pkg, orc, synth, name, fmt, 9)
    ids = [int(t) for t in synth.token_ids(shape, 100, seed=5)]
    launches0 = m.info()["launches"]
    got = m.run(ids)
    assert m.info()["launches"] - launches0 < 100         # not one launch per token
    _close(got, ref.run_seq(ids), f"{name} {fmt} prompt")
    _close(m.run(3), ref.run(3), f"{name} {fmt} next token")
    m.close()


def test_state_export_import_per_slot(pkg, orc, synth):
    """Every stream slot of a 12-stream model exports and imports on its own: a slot's state moved to another slot
    continues exactly as the original does, and the other slots are untouched."""
    shape, m, ref = _pair(pkg, orc, synth, "tiny52", "fp16", 12)
    ids = synth.token_ids(shape, 36, seed=13).reshape(3, 12)
    for t in range(2):
        m.decode(ids[t])
    snap = [m.export_state(b) for b in range(12)]
    m.import_state(snap[3], slot=9)                       # stream 9 becomes a copy of stream 3
    nxt = ids[2].copy()
    nxt[9] = nxt[3]
    got = m.decode(nxt)
    assert np.array_equal(got[9], got[3])
    ref.reset()
    for t in range(2):
        ref.run(int(ids[t, 3]))
    _close(got[9], ref.run(int(nxt[3])), "moved stream")
    for b in (0, 5, 11):                                  # untouched slots: export -> reset -> import restores them
        now = m.export_state(b)
        m.reset_states(b)
        m.import_state(now, slot=b)
        assert np.array_equal(m.export_state(b), now)
    m.close()
