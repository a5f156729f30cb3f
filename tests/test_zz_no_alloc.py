"""GPU test of the allocation-free mm_int8 entry point, through the C ABI.

`texo_mm_int8_solve_noalloc` exists for hosts that may not allocate device memory once they
are running (all of HBM already belongs to their own pools, or they cannot afford the
device-wide stall of cudaMalloc).  It keeps the tensor path's scratch in a fixed array inside
the library instead of a cudaMalloc'd buffer.  The checks:

* on two calls in a row, with different inputs (so stale sums left in the shared scratch by
  the first call would show), its output equals the regular entry point's AND the CPU
  oracle's byte for byte - integer work, so the tolerance is 0;
* after one set-up call, calls of shapes the process has not seen before - tensor path with
  and without the sums pre-pass, wide K, the generic path - leave the device's free memory
  exactly as it was (cudaMemGetInfo before and after), and the regular entry point is not
  called in between;
* the error word is readable without allocating and reads 0 after good calls.

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


def test_two_calls_in_a_row_match_the_regular_entry_point(lib, oracle):
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
        assert np.array_equal(got.cpu().numpy(), oracle.mm_int8(A.cpu().numpy(), B.cpu().numpy(), M, N, K, q))
        assert want.abs().max().item() > 0 and (want.abs() < 127).float().mean().item() > 0.5
    # odd sizes go to the scratch-free generic kernel and must agree too
    A = torch.randint(-128, 128, (65, 31), generator=g, device="cuda", dtype=torch.int8)
    B = torch.randint(-128, 128, (31, 67), generator=g, device="cuda", dtype=torch.int8)
    rc, got, want = _both(lib, A, B, (0.125, 0.25, 8.0, 7, -11, 19))
    assert rc == 0 and torch.equal(got, want)
    assert lib.texo_mm_int8_noalloc_status() == 0


def test_calls_leave_free_device_memory_unchanged(lib, oracle):
    """Shapes, zero-point patterns and paths this process has not run through the entry point
    before: none of them may take device memory (every kernel was loaded and configured by
    the first call's set-up)."""
    rng = np.random.default_rng(31)
    cases = [  # (M, N, K, quant): together they reach every kernel the entry point can launch
        (640, 1024, 512, (0.02, 0.03, 3.0, 3, -5, 1)),       # tensor kernel + both sums
        (200, 272, 4096, (0.02, 0.03, 9.0, 0, 0, -4)),       # tensor kernel alone (no pre-pass)
        (136, 256, 33040, (0.02, 0.03, 30.0, 2, 0, 0)),      # the 64-bit tensor kernel, column sums only
        (77, 50, 129, (0.05, 0.04, 1.5, -3, 9, 2)),          # generic kernel
        (1, 16, 0, (1.0, 1.0, 1.0, 0, 0, 5)),                # K = 0
    ]
    # operands and outputs first: the caller's own allocations are not the library's
    dev = []
    for M, N, K, q in cases:
        a = rng.integers(-128, 128, (M, max(K, 1)), dtype=np.int8)[:, :K]
        b = rng.integers(-128, 128, (max(K, 1), N), dtype=np.int8)[:K]
        a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
        dev.append((a, b, torch.from_numpy(a).cuda() if K else None, torch.from_numpy(b).cuda() if K else None,
                    torch.full((M, N), 99, dtype=torch.int8, device="cuda")))
    # set-up call (a shape none of the cases repeats)
    A0 = torch.zeros((128, 128), dtype=torch.int8, device="cuda")
    C0 = torch.empty((128, 256), dtype=torch.int8, device="cuda")
    B0 = torch.zeros((128, 256), dtype=torch.int8, device="cuda")
    assert lib.texo_mm_int8_solve_noalloc(A0.data_ptr(), B0.data_ptr(), C0.data_ptr(), 128, 256, 128,
                                          1.0, 1.0, 1.0, 0, 0, 0) == 0
    assert lib.texo_mm_int8_noalloc_status() == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for (M, N, K, q), (a, b, A, B, C) in zip(cases, dev):
        rc = lib.texo_mm_int8_solve_noalloc(A.data_ptr() if K else None, B.data_ptr() if K else None,
                                            C.data_ptr(), M, N, K, *q)
        assert rc == 0, (M, N, K)
    assert lib.texo_mm_int8_noalloc_status() == 0  # blocking read: the calls above have finished
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"device memory was taken: {free_before - free_after} bytes"
    for (M, N, K, q), (a, b, A, B, C) in zip(cases, dev):
        assert np.array_equal(C.cpu().numpy(), oracle.mm_int8(a, b, M, N, K, q)), (M, N, K)


def test_sizes_beyond_the_fixed_scratch_are_rejected(lib):
    A = torch.zeros(16, dtype=torch.int8, device="cuda")
    C = torch.full((16,), 9, dtype=torch.int8, device="cuda")
    q = (1.0, 1.0, 1.0, 0, 0, 0)
    assert lib.texo_mm_int8_solve_noalloc(A.data_ptr(), A.data_ptr(), C.data_ptr(), 32769, 16, 16, *q) == -2
    assert lib.texo_mm_int8_solve_noalloc(A.data_ptr(), A.data_ptr(), C.data_ptr(), 16, 32784, 16, *q) == -2
    assert lib.texo_mm_int8_solve_noalloc(A.data_ptr(), A.data_ptr(), C.data_ptr(), 0, 16, 16, *q) == -1
    torch.cuda.synchronize()
    assert bool((C == 9).all())  # nothing was launched
