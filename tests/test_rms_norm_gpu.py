"""GPU parity tests for rms_norm_w_residual and its quantising form, through the C ABI.

The reference has no test or golden vector for this operator (parity unpinned); the checks
are against the double-precision oracle restated from its source and, when it was built,
against the reference's own kernel recompiled for sm_100a.  FP32 tolerance: 2e-6 relative to
the row's largest |value| (both sides reduce in FP32 in different orders); x + residual and
the int8 output are integer-exact except within a hair of a rounding tie.
"""
import ctypes
import os

import numpy as np
import pytest

from tests import harness

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

EPS = 1e-5


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: GPU tests need a B200")
    from texo_b200 import _lib

    return _lib.load()


def _inputs(n, c, seed):
    rng = np.random.default_rng(seed)
    x = rng.normal(0, 1.5, (n, c)).astype(np.float32)
    r = rng.normal(0, 0.7, (n, c)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, c).astype(np.float32)
    return x, r, w


def _close(got, want):
    tol = 2e-6 * np.abs(want).max(axis=1, keepdims=True) + 1e-7
    return np.all(np.abs(got.astype(np.float64) - want) <= tol)


SHAPES = [(1, 4), (3, 8), (64, 1024), (33, 2048), (17, 4096), (8, 8192), (5, 16384), (9, 1000),  # vector path
          (7, 1001), (3, 17), (2, 20000), (4, 16388)]                                             # two-pass path


@pytest.mark.parametrize("shape", SHAPES)
def test_fp32_matches_oracle(lib, oracle, shape):
    n, c = shape
    x, r, w = _inputs(n, c, c)
    want, _ = oracle.rms_norm_w_residual(x, r, w, EPS)
    X, R, W = (torch.from_numpy(t).cuda() for t in (x, r, w))
    out = torch.full((n, c), 77.0, device="cuda")
    lib.texo_rms_norm_w_residual_solve(X.data_ptr(), R.data_ptr(), W.data_ptr(), out.data_ptr(), n, c, EPS)
    torch.cuda.synchronize()
    assert lib.texo_rms_norm_last_path() == (2 if c % 4 == 0 and c <= 16384 else 1)
    assert _close(out.cpu().numpy(), want), shape
    assert np.array_equal(X.cpu().numpy(), x) and np.array_equal(R.cpu().numpy(), r)


@pytest.mark.parametrize("shape", SHAPES)
def test_quantised_matches_oracle(lib, oracle, shape):
    n, c = shape
    x, r, w = _inputs(n, c, 7 * c)
    y, z = oracle.rms_norm_w_residual(x, r, w, EPS)
    X, R, W = (torch.from_numpy(t).cuda() for t in (x, r, w))
    for scale, zp, with_z in ((0.031, 3, True), (0.008, -5, False), (-0.02, 0, True)):
        scale = float(np.float32(scale))
        q = torch.full((n, c), 99, dtype=torch.int8, device="cuda")
        zo = torch.full((n, c), 5.0, device="cuda") if with_z else None
        rs = torch.full((n,), 12345, dtype=torch.int32, device="cuda")
        lib.texo_rms_norm_quant_solve(X.data_ptr(), R.data_ptr(), W.data_ptr(), q.data_ptr(),
                                      zo.data_ptr() if with_z else None, rs.data_ptr(), n, c, EPS, scale, zp)
        torch.cuda.synchronize()
        assert np.array_equal(rs.cpu().numpy(), q.cpu().numpy().astype(np.int64).sum(axis=1))
        t = y / np.float64(scale)
        want = np.clip(np.rint(t) + zp, -128, 127)
        got = q.cpu().numpy().astype(np.float64)
        differ = got != want
        # a different value is only acceptable one step away and next to a rounding tie
        near_tie = np.abs(np.abs(t - np.floor(t)) - 0.5) < 2e-4 * np.maximum(1.0, np.abs(t))
        assert np.all(np.abs(got - want)[differ] <= 1) and np.all(near_tie[differ]), (shape, scale)
        assert differ.mean() < 1e-3
        if with_z:
            assert np.array_equal(zo.cpu().numpy(), z)  # the FP32 add is bit-defined
    assert lib.texo_mm_int8_status() == 0


def test_unaligned_pointers_take_the_two_pass_kernel(lib, oracle):
    n, c = 6, 1024
    x, r, w = _inputs(n, c, 3)
    want, _ = oracle.rms_norm_w_residual(x, r, w, EPS)
    base = torch.zeros(n * c + 1, device="cuda")
    base[1:] = torch.from_numpy(x.reshape(-1)).cuda()
    R, W = torch.from_numpy(r).cuda(), torch.from_numpy(w).cuda()
    out = torch.empty((n, c), device="cuda")
    lib.texo_rms_norm_w_residual_solve(base.data_ptr() + 4, R.data_ptr(), W.data_ptr(), out.data_ptr(), n, c, EPS)
    torch.cuda.synchronize()
    assert lib.texo_rms_norm_last_path() == 1
    assert _close(out.cpu().numpy(), want)


def test_against_the_reference_kernel(lib):
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                        "libref_rms_norm_w_residual.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref was not built (no reference checkout at build time)")
    ref = ctypes.CDLL(path)
    ref.solve.restype = None
    ref.solve.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int, ctypes.c_int, ctypes.c_float]
    for n, c in ((128, 4096), (64, 8192), (11, 1001)):
        x, r, w = _inputs(n, c, 11)
        X, R, W = (torch.from_numpy(t).cuda() for t in (x, r, w))
        ours, theirs = torch.empty((n, c), device="cuda"), torch.empty((n, c), device="cuda")
        lib.texo_rms_norm_w_residual_solve(X.data_ptr(), R.data_ptr(), W.data_ptr(), ours.data_ptr(), n, c, EPS)
        ref.solve(X.data_ptr(), R.data_ptr(), W.data_ptr(), theirs.data_ptr(), n, c, EPS)
        torch.cuda.synchronize()
        a, b = ours.cpu().numpy().astype(np.float64), theirs.cpu().numpy().astype(np.float64)
        assert np.all(np.abs(a - b) <= 2e-6 * np.abs(b).max(axis=1, keepdims=True) + 1e-7)


@pytest.mark.parametrize("n", [64, 300])
def test_producer_feeds_the_matmul(lib, oracle, n):
    """norm+quantise -> mm_int8 on the device equals the oracle chain on the same int8 bytes;
    with the producer's row sums and prepared weights (no pre-pass at all) the bytes are the
    same again."""
    from texo_b200 import ops

    c, cols = 2048, 512
    x, r, w = _inputs(n, c, 21)
    rng = np.random.default_rng(5)
    b = rng.integers(-128, 128, (c, cols), dtype=np.int8)
    X, R, W, B = (torch.from_numpy(t).cuda() for t in (x, r, w, b))
    scale_a, zp_a = 0.03, 2
    rs = torch.empty((n,), dtype=torch.int32, device="cuda")
    A = ops.rms_norm_quant(X, R, W, EPS, scale_a, zp_a, row_sum_out=rs)
    q = (scale_a, 0.02, float(np.float32(scale_a * 0.02 * 40 * 74 * np.sqrt(c) / 40)), zp_a, -3, 1)
    C = ops.mm_int8(A, B, *q)
    torch.cuda.synchronize()
    want = oracle.mm_int8(A.cpu().numpy(), b, n, cols, c, q)
    assert np.array_equal(C.cpu().numpy(), want)
    weights = ops.Int8Weights(B)
    launches = lib.texo_kernel_launches()
    C2 = weights.matmul(A, *q, row_sum=rs)
    torch.cuda.synchronize()
    assert np.array_equal(C2.cpu().numpy(), want)
    if n > 32:
        assert lib.texo_kernel_launches() - launches == 1  # the tensor kernel alone
    weights.close()
