"""fr_b200_matvec_noalloc — the matvec for hosts that may not allocate GPU memory while they run (a serving
callback that must not call cudaMalloc, a latency-bound loop).  Its scratch is a fixed array inside the library,
shared by all calls and never cleared between them, so this test calls it twice in a row with different inputs and
shapes (the second call sees the first call's leftovers) and compares each result with fr_b200_matvec, which takes
the same scratch from cudaMalloc.  Collected last on purpose: a failure here must not hide the other tests."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _noalloc(pkg, W, x, fmt):
    import torch
    K, N = W.shape
    B = x.shape[0]
    dW = torch.from_numpy(np.ascontiguousarray(W, np.float32)).cuda()
    dx = torch.from_numpy(np.ascontiguousarray(x, np.float32)).cuda()
    dy = torch.full((B, N), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    L = pkg.lib()
    rc = L.fr_b200_matvec_noalloc(dW.data_ptr(), K, N, fmt, dx.data_ptr(), B, dy.data_ptr(), 0, None)
    if rc < 0:
        raise pkg.FrB200Error(rc, "fr_b200_matvec_noalloc", L.fr_b200_noalloc_last_error().decode())
    return dy.cpu().numpy()


@pytest.mark.parametrize("fmt", [0, 1, 2])
def test_two_calls_in_a_row_match_the_allocating_entry_point(pkg, fmt):
    rng = np.random.default_rng(40 + fmt)
    # first call: a wide matrix that fills much of the scratch; second: smaller, odd row count, more streams
    for K, N, B in ((2048, 500, 1), (256, 37, 3)):
        W = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
        x = rng.standard_normal((B, K)).astype(np.float32)
        want = pkg.matvec(W, x, fmt)
        got = _noalloc(pkg, W, x, fmt)
        assert got.shape == want.shape and np.isfinite(got).all()
        # same kernels on the same packed data: the tolerance of tests/test_gpu_kernels.py, in practice equality
        assert np.abs(got - want).max() < 2e-6 * np.sqrt(K)
        assert np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-6
        # and on its own feet: the float64 product with the weights as the format stores them
        if fmt == 0:
            Wq = W.astype(np.float16).astype(np.float64)
        elif fmt == 1:
            q, s = pkg.quantize_int8(W)
            Wq = pkg.dequantize_int8(q, s).astype(np.float64)
        else:
            p4, s = pkg.quantize_int4(W)
            Wq = pkg.dequantize_int4(p4, s).astype(np.float64)
        exact = x.astype(np.float64) @ Wq
        assert np.abs(got - exact).max() < 2e-6 * np.sqrt(K) * max(1.0, np.abs(exact).max())


def test_sizes_beyond_the_built_in_scratch_are_refused(pkg):
    import torch
    L = pkg.lib()
    d = torch.zeros(16, device="cuda")
    for K, N in ((2048, 600), (8256, 16), (64, 16400)):      # too many weights, K too long, too many rows
        rc = L.fr_b200_matvec_noalloc(d.data_ptr(), K, N, 0, d.data_ptr(), 1, d.data_ptr(), 0, None)
        assert rc == -2
        assert b"scratch" in L.fr_b200_noalloc_last_error()
    assert L.fr_b200_matvec_noalloc(d.data_ptr(), 100, 8, 0, d.data_ptr(), 1, d.data_ptr(), 0, None) == -1
    assert L.fr_b200_matvec_noalloc(None, 64, 8, 0, d.data_ptr(), 1, d.data_ptr(), 0, None) == -1
    # x is read in place with 16-byte loads: a view that starts 4 bytes in is refused on the host, before any launch
    big = torch.zeros(64 * 8 + 64 + 4, device="cuda")
    assert L.fr_b200_matvec_noalloc(big.data_ptr(), 64, 8, 0, big.data_ptr() + 4, 1, big.data_ptr(), 0, None) == -1
    assert b"aligned" in L.fr_b200_noalloc_last_error()
