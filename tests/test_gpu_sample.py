"""Device-side sampling against a numpy restatement of Sampler::Sample (sampler.cpp:38-101) + the CPU softmax it
calls (kernels/cpu/softmax.cpp:6-21): same logits, same uniform draw -> same token."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def ref_sample(logits, temperature, top_k, top_p, u):
    """-> (token id, margin): margin = distance of the decisive running sums from their thresholds; a float32 sum
    taken in another order can only flip the outcome when it is tiny."""
    l = logits.astype(np.float32)
    e = np.exp(l - l.max()).astype(np.float32)
    p = (e / np.cumsum(e, dtype=np.float32)[-1]).astype(np.float32)
    order = np.argsort(-p, kind="stable")
    ps = p[order]
    c = np.cumsum(ps, dtype=np.float32)
    hit = np.nonzero(c >= np.float32(top_p))[0]
    n = int(hit[0]) + 1 if len(hit) else len(ps)
    margin = float(abs(c[n - 1] - top_p)) if len(hit) else 1.0
    if n > 1:
        margin = min(margin, float(abs(c[n - 2] - top_p)))
    if top_k > 0:
        n = min(n, top_k)
    t = np.float32(min(max(temperature, 0.1), 5.0))
    w = np.power(ps[:n], np.float32(1.0) / t).astype(np.float32)
    cw = np.cumsum(w, dtype=np.float32)
    rv = np.float32(u) * cw[-1]
    j = int(np.nonzero(cw >= rv)[0][0])
    margin = min(margin, float(abs(cw[j] - rv)) / float(cw[-1]))
    if j > 0:
        margin = min(margin, float(abs(cw[j - 1] - rv)) / float(cw[-1]))
    return int(order[j]), margin


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
