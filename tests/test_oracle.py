"""CPU tests of the oracle itself (oracle/rwkv_oracle.c): an independent numpy float64 restatement of
kernels/default/att.cpp + ffn.cpp + model_forward.cpp, the fp16 conversion, the quantisers."""
import numpy as np
import pytest


def _ln(x, w, b):
    m = x.mean()
    v = ((x - m) ** 2).mean()
    return (x - m) / np.sqrt(v + 1e-5) * w + b


def numpy_forward(shape, T, ids, rescale_every=0):
    """float64 token loop; T = {name: array}.  Mirrors kernels/default/model_forward.cpp:22-193."""
    C, H = shape.n_embd, shape.n_head
    v5 = str(shape.version).startswith("5")
    gate = str(shape.version) in ("5.1", "5.2")
    T = {k: np.asarray(v, np.float64) for k, v in T.items()}
    S = C // H if v5 else 0
    st = []
    for _ in range(shape.n_layer):
        if v5:
            st.append([np.zeros(C), np.zeros((H, S, S)), np.zeros(C)])
        else:
            st.append([np.zeros(C), np.zeros(C), np.zeros(C), np.full(C, -1e30), np.zeros(C)])
    sig = lambda z: 1 / (1 + np.exp(-z))
    outs = []
    for tok in ids:
        x = T["emb.weight"][tok].copy()
        for l in range(shape.n_layer):
            b, a, f = f"blocks.{l}.", f"blocks.{l}.att.", f"blocks.{l}.ffn."
            s = st[l]
            xx = _ln(x, T[b + "ln1.weight"], T[b + "ln1.bias"])
            mixv = lambda name: xx * T[a + name] + s[0] * (1 - T[a + name])
            kx, vx, rx = mixv("time_mix_k"), mixv("time_mix_v"), mixv("time_mix_r")
            k, v, r = kx @ T[a + "key.weight"], vx @ T[a + "value.weight"], rx @ T[a + "receptance.weight"]
            if not v5:
                r = sig(r)
                aa, bb, pp = s[1], s[2], s[3]
                ww = T[a + "time_first"] + k
                p = np.maximum(pp, ww)
                e1, e2 = np.exp(pp - p), np.exp(ww - p)
                wkv = (e1 * aa + e2 * v) / (e1 * bb + e2)
                ww = T[a + "time_decay"] + pp
                p = np.maximum(ww, k)
                e1, e2 = np.exp(ww - p), np.exp(k - p)
                s[1], s[2], s[3] = e1 * aa + e2 * v, e1 * bb + e2, p
                x = x + (r * wkv) @ T[a + "output.weight"]
            else:
                u = T[a + "time_first"].reshape(H, -1, 1)
                w = T[a + "time_decay"].reshape(H, -1, 1)
                rr, kk, vv = r.reshape(H, 1, S), k.reshape(H, S, 1), v.reshape(H, 1, S)
                am = kk @ vv
                out = (rr @ (u * am + s[1])).reshape(H, S)
                s[1] = am + w * s[1]
                lw, lb = T[a + "ln_x.weight"].reshape(H, S), T[a + "ln_x.bias"].reshape(H, S)
                out = np.stack([_ln(out[h], lw[h], lb[h]) for h in range(H)]).reshape(C)
                if gate:
                    gx = mixv("time_mix_g")
                    g = gx @ T[a + "gate.weight"]
                    out = out * (g * sig(g))
                x = x + out @ T[a + "output.weight"]
            s[0] = xx
            xx = _ln(x, T[b + "ln2.weight"], T[b + "ln2.bias"])
            fs = s[-1]
            kx = xx * T[f + "time_mix_k"] + fs * (1 - T[f + "time_mix_k"])
            rx = xx * T[f + "time_mix_r"] + fs * (1 - T[f + "time_mix_r"])
            r = sig(rx @ T[f + "receptance.weight"])
            kk = np.maximum(kx @ T[f + "key.weight"], 0) ** 2
            x = x + r * (kk @ T[f + "value.weight"])
            s[-1] = xx
            if rescale_every and (l + 1) % rescale_every == 0:
                x = x / 2
        x = _ln(x, T["ln_out.weight"], T["ln_out.bias"])
        outs.append(x @ T["head.weight"])
    return np.stack(outs), st


@pytest.mark.parametrize("name", ["tiny4", "tiny4b", "tiny52", "tiny51", "tiny50"])
def test_oracle_matches_numpy_float64(orc, synth, name):
    shape = synth.SHAPES[name]
    master = synth.generate(shape, seed=3, ln_random=True)
    ids = synth.token_ids(shape, 6, seed=1)
    want, st = numpy_forward(shape, master, ids)
    m = orc.OracleModel(shape, master, synth.param_names(shape))
    got = np.stack([m.run(int(t)) for t in ids])
    assert np.abs(got - want).max() < 2e-4
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-5
    if str(shape.version) == "4":
        s = m.state_v4()
        for l in range(shape.n_layer):
            for j in range(5):
                assert np.allclose(s[l, j], st[l][j], rtol=1e-4, atol=1e-4)


def test_oracle_rescale_is_logit_invariant(orc, synth):
    """x/2 every 6 layers with att.output / ffn.value pre-divided gives the same logits
    (kernels/default/model_forward.cpp:173-175 + the fp16 file convention)."""
    shape = synth.SHAPES["tiny4b"]  # 7 layers: one rescale point
    master = synth.generate(shape, seed=5)
    f16 = synth.to_file_dtypes(shape, master, "fp16")
    ids = synth.token_ids(shape, 4, seed=2)
    names = synth.param_names(shape)
    a = orc.OracleModel(shape, f16, names, rescale_every=6)
    ref = {k: np.asarray(v, np.float32) for k, v in f16.items()}
    for k in ref:
        if k.endswith(("att.output.weight", "ffn.value.weight")):
            ref[k] = ref[k] * np.float32(2 ** (int(k.split(".")[1]) // 6))
    b = orc.OracleModel(shape, ref, names, rescale_every=0)
    for t in ids:
        la, lb = a.run(int(t)), b.run(int(t))
        assert np.abs(la - lb).max() < 1e-4


def test_reset_reproduces_first_output(orc, synth):
    """tests/test_model.cpp:93-97: ResetStates => the rerun is bit-identical."""
    shape = synth.SHAPES["tiny4"]
    m = orc.OracleModel(shape, synth.generate(shape, seed=7), synth.param_names(shape))
    a = [m.run(t) for t in (1, 2, 3)]
    m.reset()
    b = [m.run(t) for t in (1, 2, 3)]
    for x, y in zip(a, b):
        assert np.array_equal(x, y)


def test_token_out_of_range(orc, synth):
    shape = synth.SHAPES["tiny4"]
    m = orc.OracleModel(shape, synth.generate(shape, seed=7), synth.param_names(shape))
    with pytest.raises(ValueError):
        m.run(shape.vocab)


def test_f16_conversion_matches_numpy(orc):
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1, 100, 7e4)])
    x = np.concatenate([x, np.array([0, -0.0, 65504, 65519.99, 65520, 2 ** -24, 2 ** -25, 2 ** -25 * 1.0001,
                                     6.1e-5, np.inf, -np.inf], np.float32)])
    got = np.empty(x.size, np.uint16)
    orc.lib().orc_f32_to_f16(x.ctypes.data, got.ctypes.data, x.size)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)
    back = np.empty(x.size, np.float32)
    orc.lib().orc_f16_to_f32(got.ctypes.data, back.ctypes.data, x.size)
    assert np.array_equal(back, want.view(np.float16).astype(np.float32))


def test_quant_int8_properties(orc):
    rng = np.random.default_rng(1)
    W = (rng.standard_normal((128, 48)) / 11).astype(np.float32)
    W[:, 5] = 0  # all-zero output channel -> scale 1, q 0
    q, s = orc.quant_int8(W)
    assert q.shape == (48, 128) and s.shape == (48,)
    assert s[5] == np.float16(1) and not q[5].any()
    assert np.abs(q).max() <= 127
    sf = s.astype(np.float32)
    expect = np.abs(W).max(0) / np.float32(127)
    assert np.array_equal(s[np.arange(48) != 5], expect.astype(np.float16)[np.arange(48) != 5])
    D = orc.dequant_int8(q, s)
    assert np.array_equal(D, (q.astype(np.float32) * sf[:, None]).T)
    # error at most half a step (a little more where the fp16 rounding of the scale clamps the maximum)
    assert (np.abs(D - W) <= 0.5 * sf[None, :] * 1.01 + 1e-12).all()
    # requantising the dequantised matrix is idempotent
    q2, s2 = orc.quant_int8(D)
    assert np.array_equal(orc.dequant_int8(q2, s2), D)


def test_quant_int4_properties(orc):
    rng = np.random.default_rng(2)
    W = (rng.standard_normal((96, 40)) / 9).astype(np.float32)
    p, s = orc.quant_int4(W)
    assert p.shape == (40, 48) and s.shape == (40, 3)
    lo, hi = (p & 15).astype(int) - 8, (p >> 4).astype(int) - 8
    assert lo.min() >= -7 and lo.max() <= 7 and hi.min() >= -7 and hi.max() <= 7
    D = orc.dequant_int4(p, s)
    # low nibble = even k
    n, k = 7, 10
    assert D[k, n] == np.float32(lo[n, k // 2]) * np.float32(s[n, k // 32])
    assert D[k + 1, n] == np.float32(hi[n, k // 2]) * np.float32(s[n, k // 32])
    sf = np.repeat(s.astype(np.float32), 32, axis=1).T
    assert (np.abs(D - W) <= 0.5 * sf * 1.01 + 1e-12).all()


def test_round_half_away(orc):
    # W/scale landing exactly on .5 must round away from zero (std::lround), not to even
    s = np.float16(1.0)
    W = np.zeros((32, 1), np.float32)
    W[0, 0] = 7.0   # fixes the group scale at exactly 1
    W[1, 0] = 2.5
    W[2, 0] = -2.5
    W[3, 0] = 0.5
    p, sc = orc.quant_int4(W)
    assert sc[0, 0] == s
    vals = [int(p[0, 0] >> 4) - 8, int(p[0, 1] & 15) - 8, int(p[0, 1] >> 4) - 8]
    assert vals == [3, -3, 1]
