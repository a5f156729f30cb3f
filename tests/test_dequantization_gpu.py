"""GPU parity tests for the tile-scale dequantization through the C ABI.
Tolerance 1e-6 absolute + 1e-6 relative against double (tests/dequantization.cpp:31)."""
import os
import subprocess

import numpy as np
import pytest

from tests import harness

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: GPU tests need a B200")
    from texo_b200 import _lib

    return _lib.load()


def _run(lib, x, s, rows, cols, tile, offset_floats=4):
    dx, ds = torch.from_numpy(x).cuda(), torch.from_numpy(s).cuda()
    marker = 1234567.0
    init = np.zeros(rows * cols + 2 * offset_floats, np.float32)
    init[:offset_floats] = marker
    init[-offset_floats:] = marker
    out = None
    for _ in range(2):
        dy = torch.from_numpy(init).cuda()
        lib.texo_dequantization_solve(dx.data_ptr(), ds.data_ptr(), dy.data_ptr() + 4 * offset_floats,
                                      rows, cols, tile)
        torch.cuda.synchronize()
        got = dy.cpu().numpy()
        assert np.all(got[:offset_floats] == marker) and np.all(got[-offset_floats:] == marker)
        out = got[offset_floats:offset_floats + rows * cols].reshape(rows, cols)
    assert np.array_equal(dx.cpu().numpy(), x) and np.array_equal(ds.cpu().numpy(), s)
    return out


@pytest.mark.parametrize("name,rows,cols,tile", harness.DEQUANT_SHAPES + [
    ("vector-path", 64, 256, 64), ("vector-partial", 130, 1028, 128), ("odd-offset", 33, 64, 16)])
def test_harness_cases(lib, oracle, name, rows, cols, tile):
    x, s = harness.dequant_case(rows, cols, tile)
    got = _run(lib, x, s, rows, cols, tile, offset_floats=3 if name == "odd-offset" else 4)
    want = oracle.dequantization(x, s, rows, cols, tile)
    assert np.all(np.abs(got - want) <= 1e-6 + 1e-6 * np.abs(want))


def test_full_size(lib):
    """8192 x 8192, T = 128 (the size the benchmark streams); FP32 multiply is exact to one
    rounding, so the result equals torch's elementwise product bit for bit."""
    M = N = 8192
    T = 128
    g = torch.Generator(device="cuda").manual_seed(1)
    X = torch.rand((M, N), generator=g, device="cuda") * 16 - 8
    S = torch.rand((M // T, N // T), generator=g, device="cuda") * 1.5 + 0.5
    Y = torch.empty_like(X)
    lib.texo_dequantization_solve(X.data_ptr(), S.data_ptr(), Y.data_ptr(), M, N, T)
    torch.cuda.synchronize()
    want = X * S.repeat_interleave(T, 0).repeat_interleave(T, 1)
    assert torch.equal(Y, want)


def test_unchanged_reference_harness_links_and_passes():
    exe = os.path.join(harness.ORACLE_DIR, "_ref", "dequantization_test")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref not built (reference checkout absent at build time)")
    proc = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and "ALL PASSED" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-2000:]
