"""GPU parity of the whole decode path (persistent kernel through the C ABI / host mirror) against the
CPU oracle on seeded synthetic models.  Tolerance from the north star: logits and state within 1e-2
max-abs and 1e-3 relative L2 of the fp32 reference run on the same (dequantised) weights."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ABS_TOL, REL_TOL = 1e-2, 1e-3
STRATS = [("cuda fp16", "fp16", "fp16"), ("cuda int8", "fp32", "int8"), ("cuda int4", "fp32", "int4")]


def _pair(pkg, orc, synth, name, strat, seed=11, max_batch=1, ln_random=True):
    strategy, file_dtype, fmt = strat
    shape = synth.SHAPES[name]
    tensors = synth.to_file_dtypes(shape, synth.generate(shape, seed=seed, ln_random=ln_random), file_dtype)
    m = pkg.Model(tensors, strategy, shape=shape, max_batch=max_batch)
    ref = orc.OracleModel(shape, tensors, synth.param_names(shape), rescale_every=6 if fmt == "fp16" else 0,
                          weight_format=fmt, state_fp16=fmt == "fp16")
    return shape, tensors, m, ref


def _close(got, want, what=""):
    err = float(np.abs(got - want).max())
    rel = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
    assert err < ABS_TOL and rel < REL_TOL, f"{what}: max-abs {err:.3e}, rel-L2 {rel:.3e}"


@pytest.mark.parametrize("strat", STRATS, ids=[s[0] for s in STRATS])
@pytest.mark.parametrize("name", ["tiny4", "tiny4b", "tiny52", "tiny51", "tiny50"])
def test_decode_matches_oracle(pkg, orc, synth, name, strat):
    shape, tensors, m, ref = _pair(pkg, orc, synth, name, strat)
    ids = synth.token_ids(shape, 12, seed=3)
    for i, t in enumerate(ids):
        _close(m.run(int(t)), ref.run(int(t)), f"{name} {strat[0]} step {i}")
    # recurrent state against the oracle's
    st = m.states()
    C = shape.n_embd
    if str(shape.version) == "4":
        want = ref.state_v4()
        for l in range(shape.n_layer):
            for j in range(5):
                _close(st[l][j].astype(np.float32), want[l, j], f"state[{l}][{j}]")
    else:
        H = shape.n_head
        per = 2 * C + H * 4096
        for l in range(shape.n_layer):
            blk = ref.state[l * per:(l + 1) * per]
            _close(st[l][0].astype(np.float32), blk[:C], f"sx[{l}]")
            _close(st[l][1].reshape(-1), blk[C:C + H * 4096], f"s[{l}]")
            _close(st[l][2].astype(np.float32), blk[C + H * 4096:], f"ffn_sx[{l}]")
    m.close()


@pytest.mark.parametrize("strat", STRATS, ids=[s[0] for s in STRATS])
def test_packed_weights_bit_exact(pkg, orc, synth, strat):
    """Every projection matrix read back out of the streaming tiles equals the oracle's dequantised matrix."""
    shape, tensors, m, ref = _pair(pkg, orc, synth, "tiny4b", strat)
    fmt = strat[2]
    for name in synth.param_names(shape):
        if not name.endswith(orc.MATRIX_SUFFIXES):
            continue
        W = np.asarray(tensors[name], np.float32)
        want = W.astype(np.float16).astype(np.float32) if fmt == "fp16" else orc.fake_quant(W, fmt)
        got = m.unpack_matrix(name, *W.shape)
        assert np.array_equal(got, want), name
    m.close()


@pytest.mark.parametrize("strat", STRATS, ids=[s[0] for s in STRATS])
@pytest.mark.parametrize("name,B", [("tiny4", 3), ("tiny4b", 8), ("tiny52", 5)])
def test_batched_streams_match_oracle(pkg, orc, synth, name, B, strat):
    """B independent streams in one launch: stream b must equal the oracle run on stream b's tokens."""
    shape, tensors, m, ref = _pair(pkg, orc, synth, name, strat, max_batch=B)
    ids = synth.token_ids(shape, 5 * B, seed=9).reshape(5, B)
    got = [m.decode(ids[t]) for t in range(5)]
    for b in range(B):
        ref.reset()
        for t in range(5):
            _close(got[t][b], ref.run(int(ids[t, b])), f"stream {b} step {t}")
    # greedy sample = argmax of the logits
    lg, am = m.decode(ids[0], want_argmax=True)
    assert np.array_equal(am, lg.argmax(1))
    m.close()


def test_reset_is_bit_identical_and_deterministic(pkg, orc, synth):
    """tests/test_model.cpp:93-97: after ResetStates the first outputs repeat exactly."""
    for strat in STRATS:
        shape, tensors, m, ref = _pair(pkg, orc, synth, "tiny4b", strat)
        a = [m.run(t) for t in (5, 9, 5)]
        m.reset_states()
        b = [m.run(t) for t in (5, 9, 5)]
        for x, y in zip(a, b):
            assert np.array_equal(x, y)
        m.close()


def test_seq_equals_token_loop(pkg, orc, synth):
    """kernels/default/model_forward_seq.cpp:34-46: Run([a,b,c]) == Run(a); Run(b); Run(c)."""
    for name in ("tiny4", "tiny52"):
        shape, tensors, m, ref = _pair(pkg, orc, synth, name, STRATS[0])
        ids = [int(t) for t in synth.token_ids(shape, 7, seed=4)]
        a = m.run(ids)
        m.reset_states()
        for t in ids:
            b = m.run(t)
        if name == "tiny4":
            assert np.array_equal(a, b)       # RWKV-4 has no seq kernel: Run(vector) is the token loop itself
        else:
            _close(a, b, "seq kernels vs token loop")   # RWKV-5.x prompts go through the GEMM path (fp16 operands)
        m.close()


def test_state_save_load_roundtrip(pkg, orc, synth, tmp_path):
    """tests/test_model.cpp:35-51: save the state, run, load it back, the run repeats."""
    for name in ("tiny4", "tiny52"):
        shape, tensors, m, ref = _pair(pkg, orc, synth, name, STRATS[0])
        m.run([1, 2, 3])
        path = str(tmp_path / f"{name}.state")
        m.save_state_file(path)
        a = m.run(4)
        m.run(5)
        m.load_state_file(path)
        b = m.run(4)
        assert np.array_equal(a, b)
        # initial state: zeros and pp = -1e30 (model.cpp:145-177)
        m.reset_states()
        st = m.states()
        assert all(not t.any() for l in st for i, t in enumerate(l) if not (name == "tiny4" and i == 3))
        if name == "tiny4":
            assert (st[0][3] == np.float32(-1e30)).all() and st[0][0].dtype == np.float16
        else:
            assert st[0][1].shape == (shape.n_head, 64, 64)
        m.close()


def test_token_id_out_of_range_and_missing_tensor(pkg, synth):
    shape = synth.SHAPES["tiny4"]
    tensors = synth.to_file_dtypes(shape, synth.generate(shape, 0), "fp16")
    m = pkg.Model(tensors, "cuda fp16", shape=shape)
    with pytest.raises(pkg.FrB200Error):
        m.run(shape.vocab)
    with pytest.raises(pkg.FrB200Error):
        m.run(-1)
    m.close()
    t2 = dict(tensors)
    del t2["blocks.1.ffn.value.weight"]
    with pytest.raises(pkg.FrB200Error) as e:
        pkg.Model(t2, "cuda fp16", shape=shape)
    assert "missing" in str(e.value)


def test_fr_file_load(pkg, orc, synth, tmp_path):
    """The `.fr` container (tools/convert_weight.py) loads through Model(path, strategy)."""
    shape = synth.SHAPES["tiny4"]
    tensors = synth.to_file_dtypes(shape, synth.generate(shape, 2), "fp16")
    p = str(tmp_path / "tiny4-fp16.fr")
    synth.write_fr(p, shape, tensors)
    m = pkg.Model(p, "cuda fp16")
    ref = orc.OracleModel(shape, tensors, synth.param_names(shape), rescale_every=6, state_fp16=True)
    _close(m.run(0), ref.run(0))
    _close(m.run(0), ref.run(0))
    m.close()


def test_greedy_on_device_equals_host_loop(pkg, orc, synth):
    """decode_greedy (argmax + feedback on the device) == Run -> argmax -> Run on the host."""
    shape, tensors, m, ref = _pair(pkg, orc, synth, "tiny4b", STRATS[0], max_batch=2)
    first = [7, 100]
    got = m.decode_greedy(first, 6)
    m.reset_states()
    cur = np.array(first, np.int32)
    for t in range(6):
        cur = m.decode(cur).argmax(1).astype(np.int32)
        assert np.array_equal(cur, got[t])
    m.close()


@pytest.mark.parametrize("name", ["tiny4", "tiny4b", "tiny50"])
def test_cuda_path_against_reference_golden(pkg, synth, name):
    """The CUDA path against logits the reference's own code produced (tests/golden/*.npz, generated by
    tests/golden/make_golden.py from reference model.cpp + kernels/default/* on the CPU).  The golden models have
    their weights on the fp16 grid, so the "cuda fp16" strategy multiplies by exactly the same values; what is left
    is the fp16 storage of the token-shift state and fp32 summation order.  (5.1 / 5.2 are left out: the golden
    files follow kernels/default/att.cpp:101, the CUDA path follows kernels/cuda/att.cu:289.)"""
    import os
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", name + ".npz"))
    shape = synth.SHAPES[name]
    f16, _ = synth.fp16_exact_pair(shape, synth.generate(shape, seed=int(z["seed"]), ln_random=True))
    m = pkg.Model(f16, "cuda fp16", shape=shape)
    for t, want in zip(z["ids"], z["logits"]):
        got = m.run(int(t))
        err = float(np.abs(got - want).max())
        rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        assert err < ABS_TOL and rel < REL_TOL, (name, err, rel)
    m.close()


@pytest.mark.parametrize("strat", STRATS, ids=[s[0] for s in STRATS])
@pytest.mark.parametrize("name,B", [("tiny4b", 1), ("tiny52", 12)])
def test_packed_file_load_equals_fresh_load(pkg, orc, synth, tmp_path, name, B, strat):
    """A model written with save_packed and read back with load_packed holds the same bits: every projection matrix out
    of the streaming tiles, the logits of a few steps, a prompt and (12 streams) a step through the GEMM path."""
    shape, tensors, m, ref = _pair(pkg, orc, synth, name, strat, max_batch=B)
    path = str(tmp_path / "model.b200")
    m.save_packed(path)
    m2 = pkg.Model.load_packed(path, shape, strat[0], max_batch=B)
    for pname in synth.param_names(shape):
        if pname.endswith(orc.MATRIX_SUFFIXES):
            K, N = np.asarray(tensors[pname]).shape
            assert np.array_equal(m.unpack_matrix(pname, K, N), m2.unpack_matrix(pname, K, N)), pname
    for t in (3, 7, 3):
        assert np.array_equal(m.run(t), m2.run(t))
    prompt = [int(t) for t in synth.token_ids(shape, 40, seed=6)]
    assert np.array_equal(m.run(prompt), m2.run(prompt))
    if B > 8:
        ids = synth.token_ids(shape, B, seed=4)
        assert np.array_equal(m.decode(ids), m2.decode(ids))
    with open(path, "r+b") as f:          # a foreign header is refused, not half loaded
        f.write(b"NOTAFILE")
    with pytest.raises(pkg.FrB200Error):
        pkg.Model.load_packed(path, shape, strat[0])
    m.close()
    m2.close()
