"""CPU-only: pins the oracle against the reference's golden vectors and closed forms."""
import json
import os

import numpy as np
import pytest

from tests import harness


def _golden():
    data = np.load(os.path.join(harness.GOLDEN_DIR, "mm_int8_harness.npz"))
    meta = json.loads(bytes(data["meta"]).decode())
    return data, meta


def test_golden_has_all_56_harness_cases():
    _, meta = _golden()
    assert len(meta) == 56
    assert sum(m["pinned"] for m in meta) == 2


def test_generators_reproduce_golden_inputs(oracle):
    data, meta = _golden()
    cases = harness.mm_int8_harness_cases(oracle)
    assert [c["name"] for c in cases] == [m["name"] for m in meta]
    for i, c in enumerate(cases):
        assert np.array_equal(c["a"], data[f"a{i}"]) and np.array_equal(c["b"], data[f"b{i}"])


def test_normative_oracle_matches_every_harness_case(oracle):
    """FP32-epilogue oracle == what the reference harness expects, on all 56 cases."""
    data, meta = _golden()
    for i, m in enumerate(meta):
        got = oracle.mm_int8(data[f"a{i}"], data[f"b{i}"], m["m"], m["n"], m["k"], tuple(m["q"]))
        assert np.array_equal(got, data[f"e{i}"]), m["name"]


def test_pinned_vectors_separate_fp32_from_double(oracle):
    """tests/mm_int8.cpp:210-221: only the FP32 order gives 58 / -58; double gives 59 / -59."""
    data, meta = _golden()
    for i, m in enumerate(meta):
        if not m["pinned"]:
            continue
        dbl = oracle.mm_int8(data[f"a{i}"], data[f"b{i}"], m["m"], m["n"], m["k"], tuple(m["q"]), mode=1)
        assert abs(int(data[f"e{i}"][1, 3])) == 58 and abs(int(dbl[1, 3])) == 59


def test_closed_forms(oracle):
    odd = np.array([-5, -3, -1, 0, 1, 3, 5], dtype=np.int8)
    got = oracle.mm_int8(odd, np.array([1], dtype=np.int8), 7, 1, 1, (0.5, 1, 1, 0, 0, 0))
    assert got.ravel().tolist() == [-2, -2, 0, 0, 0, 2, 2]  # ties to even, both signs
    sat = np.array([-128, -127, -65, -64, -63, 0, 62, 63, 64, 65, 126, 127], dtype=np.int8)
    got = oracle.mm_int8(sat, np.array([2], dtype=np.int8), 12, 1, 1, (1, 1, 1, 0, 0, 0))
    assert got.ravel().tolist() == [-128, -128, -128, -128, -126, 0, 124, 126, 127, 127, 127, 127]
    got = oracle.mm_int8(None, None, 3, 4, 0, (0.125, 0.25, 8, 7, -11, -7))
    assert np.all(got == -7)  # K = 0 fills with zero_point_C
    wide = oracle.mm_int8(np.full(33026, 127, np.int8), np.full(33026, 127, np.int8), 1, 1, 33026,
                          (1, 1, 33554432.0, -128, -128, 0))
    assert wide[0, 0] == round(33026 * 255 * 255 / 33554432.0)


def test_large_cancellation_sampled_rows(oracle):
    a, b, q, expected = harness.large_cancellation_case(oracle)
    for r0 in (0, 4095, 8190):
        got = oracle.mm_int8(a, b, 8192, 4096, 2048, q, rows=(r0, r0 + 2))
        assert np.array_equal(got, expected[r0:r0 + 2])


def test_config1_fp32_vs_double_disagreement_count(oracle):
    """M=512,K=1024,N=512, scales .02/.03/.5, zp 3/-5/1, harness seeds 42/123: the two
    formulas differ on exactly 27 of 262,144 outputs; the FP32 one is normative."""
    M, N, K = 512, 512, 1024
    A, B = oracle.random_int8(M * K, 42), oracle.random_int8(K * N, 123)
    q = (float(np.float32(0.02)), float(np.float32(0.03)), 0.5, 3, -5, 1)
    f32 = oracle.mm_int8(A, B, M, N, K, q, mode=0)
    f64 = oracle.mm_int8(A, B, M, N, K, q, mode=1)
    assert int(np.count_nonzero(f32 != f64)) == 27
    loop = oracle.mm_int8_harness_loop(A, B, M, N, K, q, rows=(100, 102))
    assert np.array_equal(loop, f64[100:102])


def test_zero_point_identity(oracle):
    """sum (a-zA)(b-zB) = sum ab - zB rowsum(A) - zA colsum(B) + K zA zB (src/mm_int8.cu:127-129)."""
    rng = np.random.default_rng(0)
    M, N, K, za, zb = 9, 11, 300, -7, 13
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    dots = oracle.mm_int8_dots(A, B, M, N, K, za, zb)
    a64, b64 = A.astype(np.int64), B.astype(np.int64)
    ident = a64 @ b64 - zb * a64.sum(1, keepdims=True) - za * b64.sum(0, keepdims=True) + K * za * zb
    assert np.array_equal(dots, ident)


def test_mm_int4_pinned_example(oracle):
    data = np.load(os.path.join(harness.GOLDEN_DIR, "mm_int4_example.npz"))
    y = oracle.mm_int4(data["x"], data["w"], data["s"], 2, 4, 4, 2)
    assert np.array_equal(y, data["y"])
    assert y.tolist() == [[1.0, 2.0, -1.0, 0.0], [1.0, 2.0, -1.0, 0.0]]


def test_mm_int4_against_numpy(oracle):
    m, n, k, g = 5, 9, 30, 2
    x, w, s = oracle.int4_inputs(m, n, k, g, 19)
    q = np.empty((n, k), dtype=np.float64)
    q[:, 0::2] = (w >> 4).astype(np.int32) - 8
    q[:, 1::2] = (w & 15).astype(np.int32) - 8
    wd = q * np.repeat(harness.half_bits_to_float(s).astype(np.float64), g, axis=1)
    want = harness.half_bits_to_float(x).astype(np.float64) @ wd.T
    got = oracle.mm_int4(x, w, s, m, n, k, g)
    assert np.allclose(got, want, rtol=1e-12, atol=1e-12)
    # generator: scales in [0.01, 0.11], bytes cover the range
    sf = harness.half_bits_to_float(s)
    assert sf.min() >= 0.0099 and sf.max() <= 0.1101


def test_half_conversion_matches_numpy(oracle):
    import ctypes

    oracle.lib.harness_float_to_half.restype = ctypes.c_uint16
    rng = np.random.default_rng(1)
    vals = np.concatenate([rng.normal(0, 1, 2000), rng.normal(0, 1e-6, 500), rng.normal(0, 3e4, 500),
                           [0.0, -0.0, 65504.0, 65519.9, 65520.0, 5.96e-8, 2.98e-8, 2.9802323e-8]]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.lib.harness_float_to_half(ctypes.c_float(float(v))) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("name,rows,cols,tile", harness.DEQUANT_SHAPES)
def test_dequantization_closed_form(oracle, name, rows, cols, tile):
    x, s = harness.dequant_case(rows, cols, tile)
    got = oracle.dequantization(x, s, rows, cols, tile)
    want = x.astype(np.float64) * np.repeat(np.repeat(s, tile, 0), tile, 1)[:rows, :cols]
    assert np.array_equal(got, want)


def test_mm_int4a8_is_the_pinned_pieces_composed(oracle):
    """W4A8 has no reference operator; its oracle must equal the pinned INT8 oracle applied to
    weights unpacked in the pinned INT4 nibble order (high nibble = even k, value - 8), and
    must read the reference's example bytes as (1,1), (2,2), (-1,-1), (0,0)."""
    rng = np.random.default_rng(8)
    for m, n, k in ((5, 7, 2), (33, 20, 64), (16, 48, 130), (3, 4, 0)):
        a = rng.integers(-128, 128, (m, k), dtype=np.int8)
        w = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
        unpacked = np.empty((n, k), dtype=np.int8)
        unpacked[:, 0::2] = (w >> 4).astype(np.int8) - 8
        unpacked[:, 1::2] = (w & 15).astype(np.int8) - 8
        for q in ((0.02, 0.03, 0.05, 3, -5, 1), (0.5, 0.25, 1.0, 0, 0, 0), (0.02, 0.03, 0.05, -7, 7, -128)):
            want = oracle.mm_int8(a, np.ascontiguousarray(unpacked.T), m, n, k, q)
            assert np.array_equal(oracle.mm_int4a8(a, w, m, n, k, q), want)
    w = np.array([[153], [170], [119], [136]], dtype=np.uint8)
    a = np.array([[1, 0], [0, 1]], dtype=np.int8)
    got = oracle.mm_int4a8(a, w, 2, 4, 2, (1.0, 1.0, 1.0, 0, 0, 0))
    assert np.array_equal(got, np.array([[1, 2, -1, 0], [1, 2, -1, 0]], dtype=np.int8))


def test_rms_norm_w_residual_against_numpy(oracle):
    rng = np.random.default_rng(12)
    x = rng.normal(0, 2, (5, 37)).astype(np.float32)
    r = rng.normal(0, 1, (5, 37)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, 37).astype(np.float32)
    y, z = oracle.rms_norm_w_residual(x, r, w, 1e-5)
    zz = (x + r).astype(np.float32)
    assert np.array_equal(z, zz)
    want = zz.astype(np.float64) / np.sqrt((zz.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + np.float64(np.float32(1e-5))) * w
    assert np.allclose(y, want, rtol=1e-12, atol=0)


def test_per_channel_oracle_reduces_to_per_tensor(oracle):
    rng = np.random.default_rng(3)
    m, n, k = 9, 21, 50
    a = rng.integers(-128, 128, (m, k), dtype=np.int8)
    b = rng.integers(-128, 128, (k, n), dtype=np.int8)
    q = (0.02, 0.03, 0.6, 3, -5, 1)
    sb = np.full(n, q[1], dtype=np.float32)
    zb = np.full(n, q[4], dtype=np.int32)
    assert np.array_equal(oracle.mm_int8_per_channel(a, b, m, n, k, q[0], sb, q[2], q[3], zb, q[5]),
                          oracle.mm_int8(a, b, m, n, k, q))
    # column by column against the per-tensor oracle with that column's parameters
    sb = rng.uniform(0.005, 0.05, n).astype(np.float32)
    zb = rng.integers(-8, 9, n).astype(np.int32)
    got = oracle.mm_int8_per_channel(a, b, m, n, k, q[0], sb, q[2], q[3], zb, q[5])
    for col in range(n):
        want = oracle.mm_int8(a, b[:, col:col + 1], m, 1, k, (q[0], float(sb[col]), q[2], q[3], int(zb[col]), q[5]))
        assert np.array_equal(got[:, col:col + 1], want)
