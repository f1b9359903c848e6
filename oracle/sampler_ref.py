"""numpy restatement of the reference's Sampler::Sample (sampler.cpp:38-101) with the CPU softmax it calls
(kernels/cpu/softmax.cpp:6-21) and of the uniform draws it takes from std::minstd_rand0 (sampler.cpp:20-22).

TEST INFRASTRUCTURE ONLY.  Pinned: tests/test_golden.py runs the reference's own sampler.cpp + kernels/cpu/softmax.cpp
(compiled from where they lie into oracle/_ref/fr_ref_run, `--sample` mode) on seeded logits at vocab 65536 and
requires the same picks.
"""
import numpy as np


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


def pick_distance(logits, temperature, top_k, top_p, u, token):
    """How far (relative to the total weight) the draw u lies outside the interval of the running sum that selects
    `token` in the reference's walk; 0 when the token is exactly the one the walk stops at, inf when the token is not
    among the candidates.  A pick that sums the weights in another order may land on a neighbour of the reference's
    token; its distance is then of the order of the float32 rounding of the sums."""
    l = logits.astype(np.float32)
    e = np.exp(l - l.max()).astype(np.float32)
    p = (e / np.cumsum(e, dtype=np.float32)[-1]).astype(np.float32)
    order = np.argsort(-p, kind="stable")
    ps = p[order]
    c = np.cumsum(ps, dtype=np.float32)
    hit = np.nonzero(c >= np.float32(top_p))[0]
    n = int(hit[0]) + 1 if len(hit) else len(ps)
    if top_k > 0:
        n = min(n, top_k)
    t = np.float32(min(max(temperature, 0.1), 5.0))
    w = np.power(ps[:n], np.float32(1.0) / t).astype(np.float64)
    cw = np.cumsum(w)
    pos = np.nonzero(order[:n] == token)[0]
    if len(pos) == 0:
        return float("inf")
    j = int(pos[0])
    rv = float(u) * cw[-1]
    lo, hi = (cw[j - 1] if j > 0 else 0.0), cw[j]
    return float(max(lo - rv, rv - hi, 0.0) / cw[-1])


def minstd_uniforms(seed, n):
    """The draws Sampler::Sample takes from its std::minstd_rand0: (g() - min) / (max - min), sampler.cpp:20-22."""
    m, state, out = 2147483647, seed % 2147483647 or 1, []
    for _ in range(n):
        state = state * 16807 % m
        out.append((state - 1) / (m - 2))
    return out


