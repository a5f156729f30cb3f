"""GPU parity tests for the W4A16 matmul through the C ABI.

Floating point: accepted when |y - ref| <= 0.01 + 0.01 |ref| against the double-precision
oracle - the tolerance of the reference harness (tests/mm_int4.cpp:10-11,94)."""
import os
import subprocess

import numpy as np
import pytest

from tests import harness

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

ATOL = RTOL = 0.01
MARKER = 0x7BCD


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: GPU tests need a B200")
    from texo_b200 import _lib

    return _lib.load()


def run_case(lib, x, w, s, m, n, k, g, y_offset=0):
    """Guard bands, optional odd output offset, two calls (NaN poison, then stale finite)."""
    dx = torch.from_numpy(x.view(np.int16)).cuda()
    dw = torch.from_numpy(w).cuda()
    ds = torch.from_numpy(s.view(np.int16)).cuda()
    prefix = 8 + y_offset
    total = prefix + m * n + 8
    out = None
    for poison in (0x7E00, 0x4400):
        init = np.full(total, MARKER, np.uint16)
        init[prefix:prefix + m * n] = poison
        dy = torch.from_numpy(init.view(np.int16)).cuda()
        lib.texo_mm_int4_solve(dx.data_ptr(), dw.data_ptr(), ds.data_ptr(), dy.data_ptr() + 2 * prefix,
                               m, n, k, g)
        torch.cuda.synchronize()
        got = dy.cpu().numpy().view(np.uint16)
        assert np.all(got[:prefix] == MARKER) and np.all(got[prefix + m * n:] == MARKER), "guard overwritten"
        out = got[prefix:prefix + m * n].reshape(m, n)
    assert np.array_equal(dx.cpu().numpy().view(np.uint16), x) and np.array_equal(dw.cpu().numpy(), w)
    return harness.half_bits_to_float(out)


def test_pinned_example(lib):
    data = np.load(os.path.join(harness.GOLDEN_DIR, "mm_int4_example.npz"))
    got = run_case(lib, data["x"], data["w"], data["s"], 2, 4, 4, 2)
    assert np.array_equal(got.astype(np.float64), data["y"])


def _takes_tensor_path(k, g):
    return k % 64 == 0 and g in (16, 32, 64, 128)


def _takes_decode_path(m, k, g):
    return m <= 16 and g == 128 and k % 128 == 0


def test_harness_default_cases(lib, oracle):
    cases, seed = harness.mm_int4_harness_shapes()
    for m, n, k, g, sd, zero_x, off in cases:
        x, w, s = oracle.int4_inputs(m, n, k, g, sd, zero_x)
        want = oracle.mm_int4(x, w, s, m, n, k, g)
        for force in (0, 1):  # automatic dispatch, then the generic kernel alone
            lib.texo_mm_int4_force_path(force)
            got = run_case(lib, x, w, s, m, n, k, g, off)
            path = lib.texo_mm_int4_last_path()
            lib.texo_mm_int4_force_path(0)
            want_path = (1 if force == 1 else 3 if _takes_decode_path(m, k, g) else
                         (4 if g <= 64 else 2) if _takes_tensor_path(k, g) else 1)
            assert path == want_path, (m, n, k, g, force)
            assert harness.int4_within_tolerance(got, want, ATOL, RTOL), (m, n, k, g, force)
    # zero scales: first, middle, last group and an all-zero column (tests/mm_int4.cpp:166-175)
    m, n, k, g = 70, 136, 512, 32
    x, w, s = oracle.int4_inputs(m, n, k, g, seed)
    s = s.copy()
    groups = k // g
    for col in range(n):
        for gi in range(groups):
            if col == 5 or (col % 3 == 0 and gi in (0, groups // 2, groups - 1)):
                s[col, gi] = 0
    got = run_case(lib, x, w, s, m, n, k, g)
    assert harness.int4_within_tolerance(got, oracle.mm_int4(x, w, s, m, n, k, g), ATOL, RTOL)
    assert lib.texo_mm_int4_status() == 0


@pytest.mark.parametrize("shape", [(128, 128, 64, 64), (256, 256, 128, 128), (300, 520, 1024, 64),
                                   (512, 768, 2048, 128), (257, 255, 1984, 64), (1, 4096, 4096, 128),
                                   (1000, 3, 192, 64), (300, 520, 1024, 32), (256, 256, 64, 32),
                                   (257, 255, 1984, 16), (512, 768, 2048, 32), (130, 66, 128, 16),
                                   (200, 300, 8192, 128), (577, 1030, 4096, 64), (577, 1030, 4096, 16),
                                   (300, 200, 8192, 32)])
def test_tensor_path_full_matrix(lib, oracle, shape):
    """tcgen05 kind::f16 CTA-pair kernel: partial tiles in M and N, K not a multiple of the
    group pair, all four supported group sizes (a group is a quarter, half, one or two 64-k
    stages); every output within the reference tolerance."""
    m, n, k, g = shape
    x, w, s = oracle.int4_inputs(m, n, k, g, 100 + m)
    want = oracle.mm_int4(x, w, s, m, n, k, g)
    # 2 = a TMEM drain per scale group (any of the four group sizes); 4 = scale folded into the
    # weight operand as an exact FP16 hi + lo pair, one drain per tile (G <= 64, where it is the
    # default).  Forcing either also keeps few-row shapes off the decode kernel.
    for force in ((2, 4) if g <= 64 else (2,)):
        lib.texo_mm_int4_force_path(force)
        try:
            got = run_case(lib, x, w, s, m, n, k, g)
        finally:
            lib.texo_mm_int4_force_path(0)
        assert lib.texo_mm_int4_last_path() == force
        assert harness.int4_within_tolerance(got, want, ATOL, RTOL), (shape, force)
        assert lib.texo_mm_int4_status() == 0


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (16, 4096, 4096), (7, 100, 256), (16, 4100, 1024),
                                   (3, 33, 128), (16, 520, 2048), (9, 31, 8192), (16, 8192, 8192),
                                   (2, 1000, 384), (16, 288, 3968)])
def test_decode_path_full_matrix(lib, oracle, shape):
    """The streaming kernel for M <= 16, G = 128 (packed weights read once from HBM into
    registers, mma.sync on a permuted k order, K split over the warps of a CTA): ragged N,
    every way of splitting K (K / 128 odd, divisible by 2, 4, 8, 16), one to sixteen rows, odd
    output offset; every output within the reference tolerance, guard bands intact."""
    m, n, k = shape
    x, w, s = oracle.int4_inputs(m, n, k, 128, 300 + m + n)
    got = run_case(lib, x, w, s, m, n, k, 128, y_offset=1 if n % 2 else 0)
    assert lib.texo_mm_int4_last_path() == 3
    assert harness.int4_within_tolerance(got, oracle.mm_int4(x, w, s, m, n, k, 128), ATOL, RTOL)
    assert lib.texo_mm_int4_status() == 0


def test_decode_path_large_sampled_columns(lib, oracle):
    """The decode shape of an MLP up-projection, 16 x 28672 x 8192, G = 128: sampled output
    columns against the oracle, and the whole result against the CTA-pair tensor kernel."""
    m, n, k, g = 16, 28672, 8192, 128
    rng = np.random.default_rng(5)
    x = harness.float_to_half_bits(rng.normal(0, 1, (m, k)))
    w = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    s = harness.float_to_half_bits(rng.uniform(0.01, 0.11, (n, k // g)))
    dx, dw, ds = (torch.from_numpy(t.view(np.int16) if t.dtype == np.uint16 else t).cuda() for t in (x, w, s))
    ys = []
    for force in (0, 2):
        lib.texo_mm_int4_force_path(force)
        dy = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        lib.texo_mm_int4_solve(dx.data_ptr(), dw.data_ptr(), ds.data_ptr(), dy.data_ptr(), m, n, k, g)
        torch.cuda.synchronize()
        assert lib.texo_mm_int4_last_path() == (3 if force == 0 else 2)
        ys.append(dy.float().cpu().numpy())
    lib.texo_mm_int4_force_path(0)
    assert np.all(np.abs(ys[0] - ys[1]) <= 0.02 + 0.02 * np.abs(ys[1]))  # both within 0.01 of the truth
    cols = np.unique(np.linspace(0, n - 1, 48).astype(int))
    want = oracle.mm_int4(x, np.ascontiguousarray(w[cols]), np.ascontiguousarray(s[cols]), m, len(cols), k, g)
    assert harness.int4_within_tolerance(ys[0][:, cols], want, ATOL, RTOL)
    assert lib.texo_mm_int4_status() == 0


@pytest.mark.parametrize("shape", [(4096, 4096, 4096, 128, 0, 24), (8192, 520, 8192, 32, 5, 12),
                                   (4096, 8192, 8192, 128, 11, 8)])
def test_large_sampled_rows(lib, oracle, shape):
    """tests/mm_int4.cpp:178-179 plus the large weight-only shape M=4096 K=8192 N=8192, G=128."""
    m, n, k, g, seed, nrows = shape
    x, w, s = oracle.int4_inputs(m, n, k, g, seed)
    dx = torch.from_numpy(x.view(np.int16)).cuda()
    dw = torch.from_numpy(w).cuda()
    ds = torch.from_numpy(s.view(np.int16)).cuda()
    dy = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    lib.texo_mm_int4_solve(dx.data_ptr(), dw.data_ptr(), ds.data_ptr(), dy.data_ptr(), m, n, k, g)
    torch.cuda.synchronize()
    assert lib.texo_mm_int4_status() == 0
    rows = [(m - 1) * i // max(1, nrows - 1) for i in range(nrows)]
    for r in rows:
        want = oracle.mm_int4(x, w, s, m, n, k, g, rows=(r, r + 1))
        got = dy[r].float().cpu().numpy()[None, :]
        assert harness.int4_within_tolerance(got, want, ATOL, RTOL), (shape, r)


def test_unchanged_reference_harness_links_and_passes():
    exe = os.path.join(harness.ORACLE_DIR, "_ref", "mm_int4_test")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref not built (reference checkout absent at build time)")
    proc = subprocess.run([exe], capture_output=True, text=True, timeout=1800)
    assert proc.returncode == 0 and "ALL PASSED" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-2000:]
