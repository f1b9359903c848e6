"""GPU parity of seq mode (prompt processing): the tcgen05 GEMM with its fused epilogues against numpy, and the
whole RWKV-5.x seq forward (def::ModelForwardSeq, kernels/default/model_forward_seq.cpp:48-184) against the CPU
oracle's token loop and against this backend's own token-by-token decode.  Tolerance from the north star: logits
and state within 1e-2 max-abs and 1e-3 relative L2."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ABS_TOL, REL_TOL = 1e-2, 1e-3


def _f16(a):
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


def _sig(v):
    return 1.0 / (1.0 + np.exp(-v))


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (200, 448, 448), (7, 128, 128), (333, 1024, 256),
                                   (1, 64, 64), (129, 257, 192), (1100, 320, 128), (1500, 520, 192)])
def test_gemm_plain_against_numpy(pkg, M, N, K):
    """acc = fp16(A) @ fp16(W) with fp32 accumulation; ragged M and N tails are zero-filled by TMA and masked.
    Up to 1024 rows run the few-row kernel (weights along the MMA rows), more rows the 256 x 256 prompt tiles."""
    rng = np.random.default_rng(M * 7 + N)
    A = rng.standard_normal((M, K), dtype=np.float32)
    W = rng.standard_normal((K, N), dtype=np.float32) / np.sqrt(K)
    want = _f16(A) @ _f16(W)
    got = pkg.gemm_f16(A, W)
    assert np.abs(got - want).max() < 1e-3 and np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-5


def test_gemm_epilogues_against_numpy(pkg):
    """The element-wise kernels the reference runs after each GEMM (att_seq.cu:368-423, ffn_seq.cu:65-87), fused."""
    rng = np.random.default_rng(5)
    _epilogues(pkg, rng, 200, 448, 192)      # few-row kernel
    _epilogues(pkg, rng, 1300, 448, 192)     # prompt tiles


def _epilogues(pkg, rng, M, N, K):
    A = rng.standard_normal((M, K), dtype=np.float32)
    W = rng.standard_normal((K, N), dtype=np.float32) / np.sqrt(K)
    x = rng.standard_normal((M, N), dtype=np.float32)
    r = rng.uniform(0, 1, (M, N)).astype(np.float32)
    acc = _f16(A) @ _f16(W)
    want = {1: acc * _sig(acc), 2: _sig(acc), 3: np.maximum(acc, 0) ** 2, 4: (x + acc) * 0.5, 5: (x + _f16(r) * acc) * 0.5, 6: acc}
    for epi, w in want.items():
        got = pkg.gemm_f16(A, W, epi, x if epi in (4, 5) else None, r if epi == 5 else None, 0.5)
        tol = 1e-4 if epi in (4, 5) else 8e-3      # fp16 outputs carry half-precision rounding
        assert np.abs(got - w).max() < tol * max(1.0, float(np.abs(w).max())), epi


def test_gemm_rejects_bad_arguments(pkg):
    A = np.zeros((4, 100), np.float32)
    W = np.zeros((100, 8), np.float32)
    with pytest.raises(pkg.FrB200Error):
        pkg.gemm_f16(A, W)            # K not a multiple of 64
    with pytest.raises(pkg.FrB200Error):
        pkg.gemm_f16(np.zeros((4, 64), np.float32), np.zeros((64, 8), np.float32), 4)   # residual epilogue without aux0


def _models(pkg, orc, synth, name, seed=11):
    shape = synth.SHAPES[name]
    tensors = synth.to_file_dtypes(shape, synth.generate(shape, seed=seed, ln_random=True), "fp16")
    ref = orc.OracleModel(shape, tensors, synth.param_names(shape), rescale_every=6, state_fp16=True)
    return shape, tensors, ref


def _close(got, want, what, scale_aware=False):
    err = float(np.abs(got - want).max())
    rel = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
    # The per-head state sums k*v outer products over the whole prompt and its entries grow far beyond 1 (tens, for
    # these models); for it the max-abs bound is taken relative to the largest entry.  Everything else is absolute.
    bound = ABS_TOL * (max(1.0, float(np.abs(want).max())) if scale_aware else 1.0)
    assert err < bound and rel < REL_TOL, f"{what}: max-abs {err:.3e} (bound {bound:.3e}), rel-L2 {rel:.3e}"


def _state_close(m, ref, shape, what):
    st = m.states()
    C, H = shape.n_embd, shape.n_head
    per = 2 * C + H * 4096
    for l in range(shape.n_layer):
        blk = ref.state[l * per:(l + 1) * per]
        _close(st[l][0].astype(np.float32), blk[:C], f"{what} sx[{l}]")
        _close(st[l][1].reshape(-1), blk[C:C + H * 4096], f"{what} s[{l}]", scale_aware=True)
        _close(st[l][2].astype(np.float32), blk[C + H * 4096:], f"{what} ffn_sx[{l}]")


@pytest.mark.parametrize("name,T", [("tiny52", 2), ("tiny52", 5), ("tiny52", 37), ("tiny51", 20), ("tiny50", 20),
                                    ("mid52", 150), ("mid52", 333)])
def test_seq_mode_matches_oracle_token_loop(pkg, orc, synth, name, T, monkeypatch):
    """Run(vector<int>) through the seq kernels == the oracle fed token by token (model_forward_seq.cpp:34-46):
    last-token logits and the recurrent state; T = 150 and 333 cut the state scan into parallel chunks."""
    monkeypatch.setenv("FR_B200_SEQ_MIN", "2")
    shape, tensors, ref = _models(pkg, orc, synth, name)
    ids = [int(t) for t in synth.token_ids(shape, T, seed=2)]
    m = pkg.Model(tensors, "cuda fp16", shape=shape)
    launches0 = m.info()["launches"]
    got = m.run(ids)
    assert m.info()["launches"] - launches0 < 20 * shape.n_layer + 8      # not the token loop (one launch per token)
    _close(got, ref.run_seq(ids), f"{name} T={T} logits")
    _state_close(m, ref, shape, f"{name} T={T}")
    # decoding goes on from the state the prompt left
    for t in (3, 1):
        _close(m.run(t), ref.run(t), f"{name} T={T} next token")
    m.close()


def test_seq_mode_equals_own_token_loop_and_resets(pkg, orc, synth, monkeypatch):
    """Same model through both paths of fr_b200_run_seq; a reset brings back the first result
    (tests/test_model.cpp:93-97 checks the same of the reference)."""
    shape, tensors, _ = _models(pkg, orc, synth, "mid52")
    ids = [int(t) for t in synth.token_ids(shape, 96, seed=4)]
    m = pkg.Model(tensors, "cuda fp16", shape=shape)
    monkeypatch.setenv("FR_B200_SEQ_MIN", "2")
    a = m.run(ids)
    m.reset_states()
    monkeypatch.setenv("FR_B200_SEQ_MIN", "1000000")
    b = m.run(ids)
    _close(a, b, "seq kernels vs token loop")
    m.reset_states()
    monkeypatch.setenv("FR_B200_SEQ_MIN", "2")
    assert np.array_equal(m.run(ids), a)
    m.close()


def test_seq_mode_two_prompts_in_a_row(pkg, orc, synth, monkeypatch):
    """A second prompt continues from the state of the first (the shift-state copies alternate per call)."""
    monkeypatch.setenv("FR_B200_SEQ_MIN", "2")
    shape, tensors, ref = _models(pkg, orc, synth, "tiny52")
    ids = [int(t) for t in synth.token_ids(shape, 50, seed=6)]
    m = pkg.Model(tensors, "cuda fp16", shape=shape)
    m.run(ids[:23])
    got = m.run(ids[23:])
    _close(got, ref.run_seq(ids), "two prompts")
    m.close()


def test_quantised_and_v4_models_match_the_oracle_on_prompts(pkg, orc, synth):
    """The reference has no seq kernel for RWKV-4 (model_forward_seq.cpp:111-112 throws) and none for quantised
    weights.  Here short RWKV-4 fp16 prompts take the token loop, quantised models the GEMM path over their packed
    row copies; either way Run(vector) must match the oracle's token loop."""
    for name, strat, fdt, fmt in (("tiny4", "cuda fp16", "fp16", "fp16"), ("tiny52", "cuda int8", "fp32", "int8"),
                                  ("tiny4b", "cuda int4", "fp32", "int4")):
        shape = synth.SHAPES[name]
        tensors = synth.to_file_dtypes(shape, synth.generate(shape, seed=11, ln_random=True), fdt)
        ref = orc.OracleModel(shape, tensors, synth.param_names(shape), rescale_every=6 if fmt == "fp16" else 0,
                              weight_format=fmt, state_fp16=fmt == "fp16")
        ids = [int(t) for t in synth.token_ids(shape, 9, seed=2)]
        m = pkg.Model(tensors, strat, shape=shape)
        _close(m.run(ids), ref.run_seq(ids), name)
        m.close()


@pytest.mark.parametrize("name,strat,fdt,fmt,T,pieces", [("mid52", "cuda fp16", "fp16", "fp16", 2100, None),
                                                         ("mid52", "cuda fp16", "fp16", "fp16", 2600, "3"),
                                                         ("mid4", "cuda int8", "fp32", "int8", 2200, None),
                                                         ("mid4", "cuda fp16", "fp16", "fp16", 2048, "4")])
def test_long_prompts_in_pipelined_pieces(pkg, orc, synth, monkeypatch, name, strat, fdt, fmt, T, pieces):
    """Prompts of 2048 tokens or more are cut into pieces of rows that run on streams of their own, one layer apart
    (the token shift and the recurrent state cross the cut through the model state).  Logits, the recurrent state and
    the token after the prompt must match the oracle's token loop, with the default two pieces and with three / four."""
    if pieces:
        monkeypatch.setenv("FR_B200_SEQ_PIECES", pieces)
    shape = synth.SHAPES[name]
    tensors = synth.to_file_dtypes(shape, synth.generate(shape, seed=11, ln_random=True), fdt)
    ref = orc.OracleModel(shape, tensors, synth.param_names(shape), rescale_every=6 if fmt == "fp16" else 0,
                          weight_format=fmt, state_fp16=fmt == "fp16")
    ids = [int(t) for t in synth.token_ids(shape, T, seed=2)]
    m = pkg.Model(tensors, strat, shape=shape)
    _close(m.run(ids), ref.run_seq(ids), f"{name} {fmt} T={T}")
    if str(shape.version).startswith("5"):
        _state_close(m, ref, shape, f"{name} T={T}")
    _close(m.run(7), ref.run(7), "token after the prompt")
    # a second prompt on top of the first: the shift-state copies are where the next call expects them
    ids2 = [int(t) for t in synth.token_ids(shape, 2048 + 300, seed=3)]
    _close(m.run(ids2), ref.run_seq(ids2), "second long prompt")
    m.close()
