"""GPU test of the allocation-free mm_int8 entry point, through the C ABI.

`texo_mm_int8_solve_noalloc` exists for hosts that may not allocate device memory once they
are running (all of HBM already belongs to their own pools, or they cannot afford the
device-wide stall of cudaMalloc).  It keeps the tensor path's scratch in a fixed array inside
the library instead of a cudaMalloc'd buffer.  The check: on two calls in a row, with
different inputs (so stale sums left in the shared scratch by the first call would show), its
output equals the regular entry point's byte for byte - integer work, so the tolerance is 0.
The file sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: GPU tests need a B200")
    from texo_b200 import _lib

    return _lib.load()


def _both(lib, A, B, q):
    M, K = A.shape
    N = B.shape[1]
    want = torch.full((M, N), 55, dtype=torch.int8, device="cuda")
    got = torch.full((M, N), -55, dtype=torch.int8, device="cuda")
    lib.texo_mm_int8_solve(A.data_ptr(), B.data_ptr(), want.data_ptr(), M, N, K, *q)
    rc = lib.texo_mm_int8_solve_noalloc(A.data_ptr(), B.data_ptr(), got.data_ptr(), M, N, K, *q)
    torch.cuda.synchronize()
    return rc, got, want


def test_two_calls_in_a_row_match_the_regular_entry_point(lib):
    g = torch.Generator(device="cuda").manual_seed(99)
    shapes = [(512, 768, 1024), (384, 512, 2048)]  # tensor path, non-zero zero points -> scratch in use
    quants = [(0.02, 0.03, 4.0, 3, -5, 1), (0.01, 0.04, 6.0, -7, 6, -2)]
    for (M, N, K), q in zip(shapes, quants):
        A = torch.randint(-128, 128, (M, K), generator=g, device="cuda", dtype=torch.int8)
        B = torch.randint(-128, 128, (K, N), generator=g, device="cuda", dtype=torch.int8)
        rc, got, want = _both(lib, A, B, q)
        assert rc == 0
        assert lib.texo_mm_int8_last_path() == 2, "expected the tensor path (the one that uses scratch)"
        assert torch.equal(got, want)
        assert want.abs().max().item() > 0 and (want.abs() < 127).float().mean().item() > 0.5
    # odd sizes go to the scratch-free generic kernel and must agree too
    A = torch.randint(-128, 128, (65, 31), generator=g, device="cuda", dtype=torch.int8)
    B = torch.randint(-128, 128, (31, 67), generator=g, device="cuda", dtype=torch.int8)
    rc, got, want = _both(lib, A, B, (0.125, 0.25, 8.0, 7, -11, 19))
    assert rc == 0 and torch.equal(got, want)


def test_sizes_beyond_the_fixed_scratch_are_rejected(lib):
    A = torch.zeros(16, dtype=torch.int8, device="cuda")
    C = torch.full((16,), 9, dtype=torch.int8, device="cuda")
    q = (1.0, 1.0, 1.0, 0, 0, 0)
    assert lib.texo_mm_int8_solve_noalloc(A.data_ptr(), A.data_ptr(), C.data_ptr(), 32769, 16, 16, *q) == -2
    assert lib.texo_mm_int8_solve_noalloc(A.data_ptr(), A.data_ptr(), C.data_ptr(), 16, 32784, 16, *q) == -2
    assert lib.texo_mm_int8_solve_noalloc(A.data_ptr(), A.data_ptr(), C.data_ptr(), 0, 16, 16, *q) == -1
    torch.cuda.synchronize()
    assert bool((C == 9).all())  # nothing was launched
