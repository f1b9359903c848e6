"""GPU parity of the single kernels through the C ABI: quantisers and tile packing bit-exact against the
oracle, the streaming dequant-matvec against a float64 product on the dequantised weights."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _mats(rng, K, N):
    W = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    W[:, N // 2] = 0                       # all-zero output channel
    W[3, :] *= 40                          # outliers that set the block maxima
    W[: min(32, K), 0] = 0                 # an all-zero int4 group
    return W


@pytest.mark.parametrize("K,N", [(64, 16), (128, 48), (768, 100), (2048, 33)])
def test_quantisers_bit_exact(pkg, orc, K, N):
    W = _mats(np.random.default_rng(K + N), K, N)
    q, s = pkg.quantize_int8(W)
    q0, s0 = orc.quant_int8(W)
    assert np.array_equal(q, q0) and np.array_equal(s.view(np.uint16), s0.view(np.uint16))
    p, s = pkg.quantize_int4(W)
    p0, s0 = orc.quant_int4(W)
    assert np.array_equal(p, p0) and np.array_equal(s.view(np.uint16), s0.view(np.uint16))
    assert np.array_equal(pkg.dequantize_int8(q0, orc.quant_int8(W)[1]), orc.dequant_int8(q0, orc.quant_int8(W)[1]))
    assert np.array_equal(pkg.dequantize_int4(p0, s0), orc.dequant_int4(p0, s0))


def test_quantiser_rounds_half_away(pkg, orc):
    W = np.zeros((32, 2), np.float32)
    W[0, :] = 7.0
    W[1, 0], W[2, 0], W[3, 0], W[4, 1] = 2.5, -2.5, 0.5, -0.5
    p, s = pkg.quantize_int4(W)
    p0, s0 = orc.quant_int4(W)
    assert np.array_equal(p, p0) and np.array_equal(s.view(np.uint16), s0.view(np.uint16))
    assert int(p[0, 0] >> 4) - 8 == 3 and int(p[0, 1] & 15) - 8 == -3


@pytest.mark.parametrize("fmt", [0, 1, 2])
@pytest.mark.parametrize("K,N,B", [(64, 16, 1), (128, 50, 1), (768, 96, 3), (2048, 211, 1), (8192, 64, 4), (1024, 64, 8),
                                   (2560, 40, 2), (4096, 17, 5)])
def test_matvec_matches_float64(pkg, orc, fmt, K, N, B):
    rng = np.random.default_rng(fmt * 1000 + K + N + B)
    W = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    x = rng.standard_normal((B, K)).astype(np.float32)
    if fmt == 0:
        Wd = W.astype(np.float16).astype(np.float32)
    else:
        Wd = orc.fake_quant(W, "int8" if fmt == 1 else "int4")
    y = pkg.matvec(W, x, fmt)
    # the kernel feeds x as fp16 hi + lo columns (about 22 mantissa bits); the weights are exact
    want = x.astype(np.float64) @ Wd.astype(np.float64)
    assert y.shape == (B, N)
    assert np.abs(y - want).max() < 2e-6 * np.sqrt(K)
    assert np.linalg.norm(y - want) / np.linalg.norm(want) < 2e-6


@pytest.mark.parametrize("fmt", [0, 1, 2])
def test_matvec_linearity_and_zero(pkg, fmt):
    rng = np.random.default_rng(5)
    K, N = 1024, 80
    W = (rng.standard_normal((K, N)) / 32).astype(np.float32)
    x = rng.standard_normal((1, K)).astype(np.float16).astype(np.float32)
    assert not pkg.matvec(W, np.zeros((1, K), np.float32), fmt).any()
    y1 = pkg.matvec(W, x, fmt)
    y2 = pkg.matvec(W, 2 * x, fmt)          # doubling fp16 inputs is exact
    assert np.allclose(y2, 2 * y1, rtol=0, atol=1e-6)
    # batching does not change a column's result
    xb = np.concatenate([x, rng.standard_normal((3, K)).astype(np.float32)])
    yb = pkg.matvec(W, xb, fmt)
    assert np.array_equal(yb[0], pkg.matvec(W, xb[[0, 1]], fmt)[0])


def test_matvec_argument_errors(pkg):
    W = np.zeros((100, 8), np.float32)
    with pytest.raises(pkg.FrB200Error):
        pkg.matvec(W, np.zeros((1, 100), np.float32), 0)     # K not a multiple of 64
    W = np.zeros((64, 8), np.float32)
    with pytest.raises(pkg.FrB200Error):
        pkg.matvec(W, np.zeros((9, 64), np.float32), 0)      # batch > 8


def test_a_bounded_wait_runs_out_and_leaves_the_context_usable(pkg):
    """Every device-side wait gives up after a limit and reports through a status word.  Here the limit is 1 ms and
    the barrier is one nothing arrives at: the call must come back with FR_B200_E_TIMEOUT (-6), not hang, and the
    next kernel on the same context must run as if nothing had happened."""
    L = pkg.lib()
    assert L.fr_b200_wait_selftest(0, 1000) == -6
    assert b"timed out" in L.fr_b200_last_error()
    assert L.fr_b200_wait_selftest(0, 0) == -1
    rng = np.random.default_rng(3)
    W = (rng.standard_normal((256, 48)) / 16).astype(np.float32)
    x = rng.standard_normal((1, 256)).astype(np.float32)
    y = pkg.matvec(W, x, 0)
    want = x.astype(np.float64) @ W.astype(np.float16).astype(np.float64)
    assert np.abs(y - want).max() < 1e-4
