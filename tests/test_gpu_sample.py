"""Device-side sampling against a numpy restatement of Sampler::Sample (sampler.cpp:38-101) + the CPU softmax it
calls (kernels/cpu/softmax.cpp:6-21), oracle/sampler_ref.py, itself pinned against the reference's own sampler compiled
from its sources: same logits, same uniform draw -> same token."""
import numpy as np
import pytest

from oracle.sampler_ref import minstd_uniforms as _minstd_uniforms, pick_distance, ref_sample

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 0.9), (0.7, 20, 0.95), (2.0, 5, 1.0), (1.0, 1, 0.5),
                                                     (0.05, 0, 0.3), (1.3, 0, 1.0)])
def test_sample_matches_reference_sampler(pkg, synth, temperature, top_k, top_p):
    shape = synth.SHAPES["tiny4b"]
    tensors = synth.to_file_dtypes(shape, synth.generate(shape, seed=4, ln_random=True), "fp16")
    B = 12
    m = pkg.Model(tensors, "cuda fp16", shape=shape, max_batch=B)
    rng = np.random.default_rng(17)
    checked = 0
    for step in range(3):
        logits = m.decode(synth.token_ids(shape, B, seed=step))
        u = rng.uniform(0, 1, B).astype(np.float32)
        got = m.sample(B, temperature, top_k, top_p, u)
        for b in range(B):
            want, margin = ref_sample(logits[b], temperature, top_k, top_p, u[b])
            if margin > 1e-5:
                assert got[b] == want, (step, b, int(got[b]), want, margin)
                checked += 1
    assert checked >= 3      # draws too close to a threshold to survive a different summation order are skipped
    # greedy corner: top_k = 1 is the arg-max whatever the draw (sampler.cpp:71-74)
    logits = m.decode(synth.token_ids(shape, B, seed=9))
    assert np.array_equal(m.sample(B, 1.0, 1, 1.0, rng.uniform(0, 1, B).astype(np.float32)), logits.argmax(1))
    m.close()


def test_sample_single_stream_after_run(pkg, synth):
    """After Model.run on stream 0 (persistent kernel) the logits are where fr_b200_sample looks for them."""
    shape = synth.SHAPES["tiny4"]
    tensors = synth.to_file_dtypes(shape, synth.generate(shape, seed=4, ln_random=True), "fp16")
    m = pkg.Model(tensors, "cuda fp16", shape=shape)
    logits = m.run(5)
    want, margin = ref_sample(logits, 1.0, 0, 0.8, 0.37)
    got = m.sample(1, 1.0, 0, 0.8, [0.37])
    assert margin < 1e-5 or got[0] == want
    m.close()


@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 0.9), (0.7, 20, 0.95), (2.0, 0, 1.0), (1.0, 1, 0.3)])
def test_sample_matches_the_reference_sampler_binary_at_full_vocab(pkg, synth, tmp_path, temperature, top_k, top_p):
    """The reference's own Sampler::Sample + CPU softmax (sampler.cpp, kernels/cpu/softmax.cpp compiled from where they
    lie into the driver binary, `--sample` mode) against fr_b200_sample on the same logits at vocab 65536, seeded
    std::minstd_rand0 draws, with frequency / presence penalties applied on the device (fr_b200_logits_add) and on the
    host copy alike (chat.cpp:57-61)."""
    import os
    import subprocess
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "fr_ref_run")
    if not os.path.exists(exe):
        pytest.skip("reference sampler not built (needs the reference tree at build time)")
    shape = synth.Shape("4", 1, 64, 64, 65536)
    master = synth.generate(shape, seed=3, ln_random=True)
    master["head.weight"] = master["head.weight"] * 6.0          # peaked logits, as a trained model's
    tensors = synth.to_file_dtypes(shape, master, "fp16")
    B, draws, seed = 4, 8, 42
    m = pkg.Model(tensors, "cuda fp16", shape=shape, max_batch=B)
    logits = m.decode(synth.token_ids(shape, B, seed=1)).copy()
    # penalties: a few tokens per stream, logit -= frequency * occurrence + presence
    rng = np.random.default_rng(5)
    streams = np.repeat(np.arange(B), 3).astype(np.int32)
    tokens = np.concatenate([np.argsort(-logits[b])[:3] for b in range(B)]).astype(np.int32)
    deltas = -(0.2 * rng.integers(1, 4, len(tokens)) + 0.2).astype(np.float32)
    m.logits_add(streams, tokens, deltas)
    for s, t, d in zip(streams, tokens, deltas):
        logits[s, t] += d
    lf = str(tmp_path / "logits.bin")
    logits.astype(np.float32).tofile(lf)
    r = subprocess.run([exe, "--sample", lf, str(shape.vocab), str(B), str(temperature), str(top_k), str(top_p), str(seed), str(draws)],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    theirs = np.array([[int(x) for x in line.split()[2:]] for line in r.stdout.splitlines() if line.startswith("sample")])
    assert theirs.shape == (B, draws)
    us = _minstd_uniforms(seed, draws)
    checked = 0
    for d in range(draws):
        got = m.sample(B, temperature, top_k, top_p, [us[d]] * B)
        for b in range(B):
            want, margin = ref_sample(logits[b], temperature, top_k, top_p, np.float32(us[d]))
            assert want == theirs[b, d] or margin <= 1e-5       # the numpy restatement agrees with the reference binary
            # the device sums up to 65536 weights in segments, the reference serially: a draw closer than 1e-4 (relative
            # to the total) to a threshold may resolve to a neighbouring entry -- never further away than that
            if margin > 1e-4:
                assert got[b] == theirs[b, d], (d, b, int(got[b]), int(theirs[b, d]), margin)
                checked += 1
            else:
                dist = pick_distance(logits[b], temperature, top_k, top_p, np.float32(us[d]), int(got[b]))
                assert dist <= 1e-4, (d, b, int(got[b]), int(theirs[b, d]), margin, dist)
    # a flat distribution over the whole vocabulary (temperature 2, no cuts) gives every token ~1e-5 of the weight: all of
    # its draws are "near a threshold" and are covered by the distance check alone
    flat = top_k == 0 and top_p >= 1.0 and temperature > 1.0
    assert flat or checked >= B * draws // 2
    m.close()
