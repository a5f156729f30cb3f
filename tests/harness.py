"""Test helpers: the CPU oracle behind numpy, and the reference harness's case lists.

The case lists restate `main()` of the reference harnesses (tests/mm_int8.cpp:139-254,
tests/mm_int4.cpp:144-181, tests/dequantization.cpp:37-45 of frezcirno/Texo) so that the
parity tests read like the reference's own tests.  Nothing here is imported by the product.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")

_f = ctypes.c_float
_i = ctypes.c_int


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


class Oracle:
    def __init__(self, lib: ctypes.CDLL):
        self.lib = lib
        lib.oracle_max_threads.restype = _i

    @property
    def threads(self) -> int:
        return self.lib.oracle_max_threads()

    def set_threads(self, n: int) -> int:
        """OpenMP threads for the row-parallel loops (overrides OMP_NUM_THREADS); returns the
        count in effect."""
        self.lib.oracle_set_threads.restype = _i
        return self.lib.oracle_set_threads(int(n))

    # ---------------------------------------------------------------- mm_int8
    def mm_int8(self, A, B, M, N, K, q, mode: int = 0, rows: tuple[int, int] | None = None):
        """q = (sA, sB, sC, zA, zB, zC); mode 0 = FP32 epilogue (normative), 1 = double."""
        r0, r1 = rows if rows else (0, M)
        A = np.ascontiguousarray(A, dtype=np.int8) if K else None
        B = np.ascontiguousarray(B, dtype=np.int8) if K else None
        out = np.empty((r1 - r0, N), dtype=np.int8)
        rc = self.lib.oracle_mm_int8_rows(_p(A), _p(B), _p(out), M, N, K, _f(q[0]), _f(q[1]),
                                          _f(q[2]), q[3], q[4], q[5], r0, r1, mode)
        assert rc == 0
        return out

    def mm_int8_per_channel(self, A, B, M, N, K, sa, sb, sc, za, zb, zc, rows=None):
        """sb: float32 [N]; zb: int32 [N] or None."""
        r0, r1 = rows if rows else (0, M)
        A = np.ascontiguousarray(A, dtype=np.int8) if K else None
        B = np.ascontiguousarray(B, dtype=np.int8) if K else None
        sb = np.ascontiguousarray(sb, dtype=np.float32)
        zb = None if zb is None else np.ascontiguousarray(zb, dtype=np.int32)
        out = np.empty((r1 - r0, N), dtype=np.int8)
        rc = self.lib.oracle_mm_int8_per_channel_rows(_p(A), _p(B), _p(out), M, N, K, _f(sa), _p(sb),
                                                      _f(sc), za, _p(zb), zc, r0, r1)
        assert rc == 0
        return out

    def mm_int8_per_group(self, A, B, M, N, K, G, sa, sb, sc, za, zb, zc, rows=None):
        """sb: float32 [K/G, N] (one scale per scale group and output column)."""
        r0, r1 = rows if rows else (0, M)
        A = np.ascontiguousarray(A, dtype=np.int8)
        B = np.ascontiguousarray(B, dtype=np.int8)
        sb = np.ascontiguousarray(sb, dtype=np.float32)
        assert sb.shape == (K // G, N)
        out = np.empty((r1 - r0, N), dtype=np.int8)
        rc = self.lib.oracle_mm_int8_per_group_rows(_p(A), _p(B), _p(out), M, N, K, G, _f(sa), _p(sb), _f(sc),
                                                    za, zb, zc, r0, r1)
        assert rc == 0
        return out

    def mm_int8_swiglu(self, A, B, M, F, K, sa, s_gate, s_up, s_out, za, z_gate, z_up, rows=None):
        """Returns h / s_out before rounding, float64 [rows, F]."""
        r0, r1 = rows if rows else (0, M)
        A = np.ascontiguousarray(A, dtype=np.int8) if K else None
        B = np.ascontiguousarray(B, dtype=np.int8) if K else None
        out = np.empty((r1 - r0, F), dtype=np.float64)
        rc = self.lib.oracle_mm_int8_swiglu_rows(_p(A), _p(B), _p(out), M, F, K, _f(sa), _f(s_gate),
                                                 _f(s_up), _f(s_out), za, z_gate, z_up, r0, r1)
        assert rc == 0
        return out

    def mm_int8_harness_loop(self, A, B, M, N, K, q, rows):
        r0, r1 = rows
        out = np.empty((r1 - r0, N), dtype=np.int8)
        rc = self.lib.oracle_mm_int8_harness_loop(_p(A), _p(B), _p(out), M, N, K, _f(q[0]),
                                                  _f(q[1]), _f(q[2]), q[3], q[4], q[5], r0, r1)
        assert rc == 0
        return out

    def mm_int8_dots(self, A, B, M, N, K, za, zb, rows=None):
        r0, r1 = rows if rows else (0, M)
        out = np.empty((r1 - r0, N), dtype=np.int64)
        rc = self.lib.oracle_mm_int8_dots(_p(A), _p(B), _p(out), M, N, K, za, zb, r0, r1)
        assert rc == 0
        return out

    # ---------------------------------------------------------------- mm_int4
    def mm_int4(self, x_bits, w, s_bits, M, N, K, G, rows=None):
        r0, r1 = rows if rows else (0, M)
        out = np.empty((r1 - r0, N), dtype=np.float64)
        rc = self.lib.oracle_mm_int4_rows(_p(x_bits), _p(w), _p(s_bits), _p(out), M, N, K, G, r0, r1)
        assert rc == 0
        return out

    # -------------------------------------------------------------- mm_int4a8
    def mm_int4a8(self, A, w, M, N, K, q, rows: tuple[int, int] | None = None):
        """W4A8: A [M,K] int8, w [N,K/2] packed nibbles, q = (sA, sB, sC, zA, zB, zC)."""
        r0, r1 = rows if rows else (0, M)
        A = np.ascontiguousarray(A, dtype=np.int8) if K else None
        w = np.ascontiguousarray(w, dtype=np.uint8) if K else None
        out = np.empty((r1 - r0, N), dtype=np.int8)
        rc = self.lib.oracle_mm_int4a8_rows(_p(A), _p(w), _p(out), M, N, K, _f(q[0]), _f(q[1]),
                                            _f(q[2]), q[3], q[4], q[5], r0, r1)
        assert rc == 0
        return out

    # ---------------------------------------------------- rms_norm_w_residual
    def rms_norm_w_residual(self, x, residual, weight, eps):
        """Returns (y [N,C] float64, z [N,C] float32 = x + residual)."""
        N, C = x.shape
        y = np.empty((N, C), dtype=np.float64)
        z = np.empty((N, C), dtype=np.float32)
        rc = self.lib.oracle_rms_norm_w_residual(_p(np.ascontiguousarray(x, dtype=np.float32)),
                                                 _p(np.ascontiguousarray(residual, dtype=np.float32)),
                                                 _p(np.ascontiguousarray(weight, dtype=np.float32)),
                                                 _p(y), _p(z), N, C, _f(eps))
        assert rc == 0
        return y, z

    # --------------------------------------------------------- dequantization
    def dequantization(self, X, S, M, N, T):
        out = np.empty((M, N), dtype=np.float64)
        rc = self.lib.oracle_dequantization(_p(X), _p(S), _p(out), M, N, T)
        assert rc == 0
        return out

    # ------------------------------------------------------ harness generators
    def random_int8(self, size: int, seed: int, lo: int = -128, hi: int = 127) -> np.ndarray:
        out = np.empty(size, dtype=np.int8)
        self.lib.harness_random_int8(_p(out), ctypes.c_size_t(size), ctypes.c_uint(seed), lo, hi)
        return out

    def int4_inputs(self, m, n, k, g, seed, zero_x=False):
        x = np.empty(m * k, dtype=np.uint16)
        w = np.empty(n * (k // 2), dtype=np.uint8)
        s = np.empty(n * (k // g), dtype=np.uint16)
        self.lib.harness_int4_inputs(m, n, k, g, ctypes.c_uint(seed), int(zero_x), _p(x), _p(w), _p(s))
        return x.reshape(m, k), w.reshape(n, k // 2), s.reshape(n, k // g)


_ORACLE = None


def load_oracle() -> Oracle:
    global _ORACLE
    if _ORACLE is None:
        so = os.path.join(ORACLE_DIR, "liboracle.so")
        srcs = [os.path.join(ORACLE_DIR, f) for f in ("qmm_oracle.c", "harness_inputs.cpp")]
        if not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs):
            subprocess.run(["make", "-C", ORACLE_DIR, "liboracle.so"], check=True,
                           capture_output=True)
        _ORACLE = Oracle(ctypes.CDLL(so))
    return _ORACLE


# --------------------------------------------------------------------------------------
# mm_int8: the 56 default cases of the reference harness (tests/mm_int8.cpp:139-254).
# Each case: dict(name, m, n, k, a, b, q, offsets=(a_off, b_off, c_off), known=None|array)
# --------------------------------------------------------------------------------------

def _case(name, m, n, k, a, b, q, offsets=(0, 0, 0), known=None):
    return dict(name=name, m=m, n=n, k=k, a=np.asarray(a, dtype=np.int8).reshape(-1),
                b=np.asarray(b, dtype=np.int8).reshape(-1), q=tuple(q), offsets=tuple(offsets),
                known=None if known is None else np.asarray(known, dtype=np.int8))


def mm_int8_harness_cases(oracle: Oracle) -> list[dict]:
    rnd = oracle.random_int8
    cases = []

    def run_random(name, m, n, k, q, offsets=(0, 0, 0)):
        cases.append(_case(name, m, n, k, rnd(m * k, 42), rnd(k * n, 123), q, offsets))

    normal = (0.125, 0.25, 8.0, 0, 0, 0)
    shapes = [(1, 1, 1), (1, 17, 7), (17, 1, 7), (2, 3, 5), (15, 15, 15), (16, 16, 16),
              (17, 17, 17), (16, 15, 7), (15, 16, 7), (16, 17, 7), (17, 16, 7), (31, 32, 9),
              (32, 31, 9), (32, 32, 32), (33, 33, 33), (3, 5, 257), (3, 5, 1025), (33, 65, 1),
              (65, 67, 31)]
    for m, n, k in shapes:
        run_random("random-boundary", m, n, k, normal)
    for za, zb, zc in [(7, 0, 0), (0, -11, 0), (0, 0, 19), (7, -11, 19), (-128, 127, -128),
                       (127, -128, 127)]:
        run_random("zero-points", 17, 19, 7, (0.125, 0.25, 8.0, za, zb, zc))

    shifted = (0.25, 0.5, 0.125, 7, -11, 19)
    cases.append(_case("quantized-zero-A", 17, 19, 7, np.full(17 * 7, 7), rnd(7 * 19, 123), shifted))
    cases.append(_case("quantized-zero-B", 17, 19, 7, rnd(17 * 7, 42), np.full(7 * 19, -11), shifted))
    ident_a = np.full((17, 17), 7, dtype=np.int8)
    ident_b = np.full((19, 19), -11, dtype=np.int8)
    np.fill_diagonal(ident_a, 8)
    np.fill_diagonal(ident_b, -10)
    cases.append(_case("left-identity", 17, 19, 17, ident_a, rnd(17 * 19, 123, -32, 31), shifted))
    cases.append(_case("right-identity", 17, 19, 19, rnd(17 * 19, 42, -32, 31), ident_b, shifted))
    tail = np.full((17, 257), 7, dtype=np.int8)
    for row in range(17):
        tail[row, 256] = row + 7 + 1
    cases.append(_case("last-K-only", 17, 19, 257, tail, rnd(257 * 19, 123, -16, 15), shifted))

    odd = [-5, -3, -1, 0, 1, 3, 5]
    for zc in (0, 7, -7):
        cases.append(_case("half-to-even", 7, 1, 1, odd, [1], (0.5, 1, 1, 0, 0, zc)))
    for scale in (np.nextafter(np.float32(0.5), np.float32(0)), np.nextafter(np.float32(0.5), np.float32(1))):
        cases.append(_case("adjacent-to-half", 2, 1, 1, [-1, 1], [1], (float(scale), 1, 1, 0, 0, 0)))
    cases.append(_case("scale-B", 7, 1, 1, odd, [1], (1, 0.5, 1, 0, 0, 0)))
    cases.append(_case("scale-C", 7, 1, 1, odd, [1], (1, 1, 2, 0, 0, 0)))
    cases.append(_case("decimal-scales", 17, 19, 7, rnd(17 * 7, 42, -8, 7), rnd(7 * 19, 123, -8, 7),
                       (np.float32(0.1), np.float32(0.2), np.float32(0.3), 1, -2, 3)))
    cases.append(_case("saturation", 12, 1, 1,
                       [-128, -127, -65, -64, -63, 0, 62, 63, 64, 65, 126, 127], [2],
                       (1, 1, 1, 0, 0, 0)))
    cases.append(_case("signed-extremes", 2, 2, 1, [127, -128], [127, -128], (1, 1, 1, 0, 0, 0)))
    for zc in (-128, 127):
        cases.append(_case("shift-then-saturate", 5, 1, 1, [-127, -1, 0, 1, 127], [1],
                           (1, 1, 1, 0, 0, zc)))
    unaligned = (0.125, 0.25, 8.0, 7, -11, 19)
    run_random("unaligned-A", 17, 19, 7, unaligned, (1, 0, 0))
    run_random("unaligned-B", 17, 19, 7, unaligned, (0, 1, 0))
    run_random("unaligned-C", 17, 19, 7, unaligned, (0, 0, 1))
    run_random("unaligned-all", 17, 19, 7, unaligned, (1, 3, 7))
    for zc in (-128, -7, 0, 127):
        run_random("K-zero", 17, 19, 0, (0.125, 0.25, 8.0, 7, -11, zc), (0, 0, 1))
    leet_b = [36, 50, 42, 8, -30, 47, -2, -35, 7, -30]
    leet_q = (np.float32(0.05), np.float32(0.1), np.float32(0.01), 0, 0, 0)
    cases.append(_case("leetgpu-58-not-59", 3, 5, 2, [29, -32, -16, 35, -35, -38], leet_b, leet_q,
                       known=[-128, 127, 127, 4, 45, 127, -128, -128, 58, -128, -128, -128, -70,
                              -128, 127]))
    cases.append(_case("leetgpu-negative-tie", 3, 5, 2, [-29, 32, 16, -35, 35, 38], leet_b, leet_q,
                       known=[127, -128, -128, -4, -45, -128, 127, 127, -58, 127, 127, 127, 70,
                              127, -128]))
    for random in (False, True):
        m, n, k = 17, 19, 2048
        pairs = (k - 2) // 2
        a = (rnd(m * k, 77, -127, 127) if random else np.full(m * k, 127, dtype=np.int8)).reshape(m, k).copy()
        b = (rnd(k * n, 99, -127, 127) if random else np.full(k * n, 127, dtype=np.int8)).reshape(k, n).copy()
        a[:, pairs:2 * pairs] = a[:, :pairs]
        a[:, k - 2] = np.where(np.arange(m) % 2 == 1, -1, 1)
        a[:, k - 1] = 0
        b[pairs:2 * pairs, :] = -b[:pairs, :]
        b[k - 2, :] = np.arange(n) - n // 2
        b[k - 1, :] = 0
        cases.append(_case("random-cancellation" if random else "ordered-cancellation", m, n, k, a, b,
                           (np.float32(0.1), np.float32(0.1), np.float32(0.01), 0, 0, 0)))
    cases.append(_case("wide-positive-dot", 1, 1, 33026, np.full(33026, 127), np.full(33026, 127),
                       (1, 1, 33554432.0, -128, -128, 0)))
    cases.append(_case("wide-negative-dot", 1, 1, 33026, np.full(33026, -128), np.full(33026, 127),
                       (1, 1, 33554432.0, 127, -128, 0)))
    for c in cases:
        c["q"] = (float(np.float32(c["q"][0])), float(np.float32(c["q"][1])),
                  float(np.float32(c["q"][2])), int(c["q"][3]), int(c["q"][4]), int(c["q"][5]))
    return cases


def large_cancellation_case(oracle: Oracle):
    """tests/mm_int8.cpp:106-137: 8192x4096x2048 with an analytic answer for every output."""
    m, n, k = 8192, 4096, 2048
    pairs = (k - 2) // 2
    a = oracle.random_int8(m * k, 77, -127, 127).reshape(m, k).copy()
    b = oracle.random_int8(k * n, 99, -127, 127).reshape(k, n).copy()
    a[:, pairs:2 * pairs] = a[:, :pairs]
    sign = np.where(np.arange(m) % 2 == 1, -1, 1).astype(np.int8)
    a[:, k - 2] = sign
    a[:, k - 1] = 0
    b[pairs:2 * pairs, :] = -b[:pairs, :]
    col = (np.arange(n) % 255 - 127).astype(np.int8)
    b[k - 2, :] = col
    b[k - 1, :] = 0
    expected = (sign[:, None].astype(np.int32) * col[None, :].astype(np.int32)).astype(np.int8)
    q = (float(np.float32(0.1)), float(np.float32(0.1)), float(np.float32(0.01)), 0, 0, 0)
    return a, b, q, expected


# mm_int4 default cases (tests/mm_int4.cpp:144-176): (m, n, k, g, seed, zero_x, y_offset)
def mm_int4_harness_shapes():
    cases = [(1, 2, 4, 2, 1, True, 0)]
    seed = 2
    official = [(2, 4, 4, 2), (3, 5, 8, 4), (16, 16, 32, 16), (32, 64, 64, 32), (64, 128, 128, 64),
                (30, 50, 64, 32), (100, 200, 128, 64), (255, 100, 128, 64), (128, 256, 512, 128)]
    extra = [(1, 1, 32, 32), (129, 131, 96, 32), (7, 257, 160, 16), (200, 129, 192, 64),
             (131, 64, 384, 128), (65, 300, 1056, 32), (17, 33, 48, 16), (5, 9, 30, 2),
             (9, 7, 40, 8), (300, 200, 1024, 16), (1, 4096, 4096, 128)]
    for m, n, k, g in official + extra:
        cases.append((m, n, k, g, seed, False, 0))
        seed += 1
    cases.append((130, 66, 256, 128, seed, False, 1))
    seed += 1
    return cases, seed  # `seed` is the one the zero-scales case uses next


def half_bits_to_float(bits: np.ndarray) -> np.ndarray:
    return bits.view(np.float16).astype(np.float32)


def float_to_half_bits(values) -> np.ndarray:
    return np.asarray(values, dtype=np.float32).astype(np.float16).view(np.uint16)


def dequant_case(rows: int, cols: int, tile: int):
    """tests/dequantization.cpp:6-25 closed-form generator."""
    r = np.arange(rows)[:, None]
    c = np.arange(cols)[None, :]
    x = (((r * 11 + c * 5) % 23 - 11) * 0.25).astype(np.float32)
    sr = np.arange(-(-rows // tile))[:, None]
    sc = np.arange(-(-cols // tile))[None, :]
    s = (((sr * 7 + sc * 13) % 19 - 9) * 0.125).astype(np.float32)
    return x, s


DEQUANT_SHAPES = [("scalar", 1, 1, 16), ("small-partial-tile", 17, 31, 16),
                  ("rectangular-t32", 65, 33, 32), ("partial-t64", 129, 193, 64),
                  ("partial-t128", 257, 130, 128)]


def int4_within_tolerance(got: np.ndarray, want: np.ndarray, atol=0.01, rtol=0.01) -> bool:
    got = got.astype(np.float64)
    return bool(np.all(np.isfinite(got)) and np.all(np.abs(got - want) <= atol + rtol * np.abs(want)))


# Counter-based generator for the large benchmark shapes: any rank can materialise any
# sub-block of the same logical matrix (used by the multi-GPU tests and the benchmark).
def hashed_int8(seed: int, tensor_id: int, rows, cols) -> np.ndarray:
    """U{-128..127} bytes as a pure function of (seed, tensor_id, row, col)."""
    r = np.asarray(rows, dtype=np.uint64)[:, None]
    c = np.asarray(cols, dtype=np.uint64)[None, :]
    with np.errstate(over="ignore"):
        x = (r * np.uint64(0x9E3779B97F4A7C15)) ^ (c * np.uint64(0xC2B2AE3D27D4EB4F))
        x ^= np.uint64(seed) * np.uint64(0xD6E8FEB86659FD93) + np.uint64(tensor_id)
        x ^= x >> np.uint64(32)
        x *= np.uint64(0xD6E8FEB86659FD93)
        x ^= x >> np.uint64(29)
        x *= np.uint64(0x9E3779B97F4A7C15)
        x ^= x >> np.uint64(32)
    return (x & np.uint64(0xFF)).astype(np.uint8).view(np.int8)


def isclose_f32(a: float, b: float) -> bool:
    return math.isclose(a, b, rel_tol=0, abs_tol=0)
