"""The oracle against golden vectors produced by the reference's own code (tests/golden/make_golden.py:
reference model.cpp + kernels/default/{model_forward,att,ffn}.cpp run on the CPU), and, where the reference
tree and the built driver are present, against that driver run live."""
import os
import subprocess

import numpy as np
import pytest

import __graft_entry__ as entry  # noqa: E402  (tests/conftest.py puts the repository root on sys.path)

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden")
CASES = ["tiny4", "tiny4b", "tiny50", "tiny51", "tiny52"]


def _load(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return int(z["seed"]), z["ids"], z["logits"]


@pytest.mark.parametrize("name", CASES)
def test_oracle_reproduces_reference_golden(orc, synth, name):
    seed, ids, want = _load(name)
    shape = synth.SHAPES[name]
    _, tensors = synth.fp16_exact_pair(shape, synth.generate(shape, seed=seed, ln_random=True))
    # the golden files come from kernels/default/att.cpp, which feeds the v5.1/5.2 gate with xx (att.cpp:101)
    m = orc.OracleModel(shape, tensors, synth.param_names(shape), gate_from_xx=True)
    got = np.stack([m.run(int(t)) for t in ids])
    assert got.shape == want.shape
    assert np.abs(got - want).max() < 5e-5
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 5e-6


def test_cuda_gate_convention_differs_only_for_gated_versions(orc, synth):
    """kernels/cuda/att.cu:289 feeds the gate with gx; kernels/default/att.cpp:101 with xx.  The flag must
    matter for 5.1/5.2 and must not for 4 / 5.0."""
    for name, differs in (("tiny4", False), ("tiny50", False), ("tiny52", True)):
        seed, ids, _ = _load(name)
        shape = synth.SHAPES[name]
        _, t = synth.fp16_exact_pair(shape, synth.generate(shape, seed=seed, ln_random=True))
        a = orc.OracleModel(shape, t, synth.param_names(shape), gate_from_xx=True)
        b = orc.OracleModel(shape, t, synth.param_names(shape), gate_from_xx=False)
        # the shift state is zero at the first token, where gx == xx * mix_g: compare the second token
        a.run(int(ids[0])); b.run(int(ids[0]))
        la, lb = a.run(int(ids[1])), b.run(int(ids[1]))
        assert (not np.array_equal(la, lb)) == differs


@pytest.mark.skipif(not (os.path.isdir(entry.reference_dir()) and
                         os.path.exists(os.path.join(os.path.dirname(HERE), "oracle", "_ref", "fr_ref_run"))),
                    reason="needs the reference tree and oracle/_ref/fr_ref_run")
def test_oracle_against_live_reference_cpu(orc, synth, tmp_path):
    exe = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "fr_ref_run")
    shape = synth.SHAPES["tiny4b"]
    tensors = synth.to_file_dtypes(shape, synth.generate(shape, seed=77, ln_random=True), "fp32")
    fr = str(tmp_path / "m.fr")
    synth.write_fr(fr, shape, tensors)
    ids = [int(i) for i in synth.token_ids(shape, 9, seed=5)]
    out = str(tmp_path / "o.bin")
    subprocess.check_call([exe, fr, "cpu fp32", out] + [str(i) for i in ids])
    want = np.fromfile(out, np.float32).reshape(len(ids), shape.vocab)
    m = orc.OracleModel(shape, tensors, synth.param_names(shape))
    got = np.stack([m.run(i) for i in ids])
    assert np.abs(got - want).max() < 5e-5


@pytest.mark.skipif(not os.path.exists(os.path.join(os.path.dirname(HERE), "oracle", "_ref", "fr_ref_run")),
                    reason="needs oracle/_ref/fr_ref_run (built where the reference tree is)")
@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 0.9), (0.7, 20, 0.95), (2.0, 0, 1.0), (1.0, 1, 0.3), (0.05, 0, 0.5)])
def test_sampler_restatement_against_the_reference_sampler(tmp_path, temperature, top_k, top_p):
    """oracle/sampler_ref.py against the reference's own Sampler::Sample (sampler.cpp + kernels/cpu/softmax.cpp, compiled
    from their sources) at vocab 65536: seeded std::minstd_rand0 draws on seeded logits give the same token ids."""
    from oracle.sampler_ref import minstd_uniforms, ref_sample
    exe = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "fr_ref_run")
    rng = np.random.default_rng(11)
    V, B, draws, seed = 65536, 3, 10, 7
    logits = (rng.standard_normal((B, V)) * 6).astype(np.float32)
    lf = str(tmp_path / "logits.bin")
    logits.tofile(lf)
    r = subprocess.run([exe, "--sample", lf, str(V), str(B), str(temperature), str(top_k), str(top_p), str(seed), str(draws)],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    theirs = np.array([[int(x) for x in line.split()[2:]] for line in r.stdout.splitlines() if line.startswith("sample")])
    us = minstd_uniforms(seed, draws)
    agree = 0
    for b in range(B):
        for d in range(draws):
            want, margin = ref_sample(logits[b], temperature, top_k, top_p, np.float32(us[d]))
            assert want == theirs[b, d] or margin <= 1e-5
            agree += want == theirs[b, d]
    assert agree >= B * draws - 2
