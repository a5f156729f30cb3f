"""Host-side mirror of the reference operator interface, on torch CUDA tensors.

Each function keeps the name, argument order and meaning of the reference operator's
`solve` (frezcirno/Texo src/mm_int8.cu:530-535, src/mm_int4.cu:386-390,
src/dequantization.cu:40-43); torch only provides device memory and stream ordering.  The
math always runs in the CUDA library; a missing library or a CPU tensor is an error.
"""
from __future__ import annotations

import torch

from . import _lib

__all__ = ["mm_int8", "mm_int8_per_channel", "mm_int8_per_group", "mm_int8_swiglu", "mm_int8_dequant", "mm_int4",
           "mm_int4a8", "mm_int4a8_per_channel", "mm_int4a8_per_group", "dequantization", "rms_norm_w_residual",
           "rms_norm_quant", "mm_int8_host", "Int8Weights", "last_path", "status", "force_path"]


def _check_cuda(name: str, t: torch.Tensor, dtype: torch.dtype) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous and row-major")


class _DefaultStreamOrder:
    """The library issues work on the legacy default stream (reference contract).  When the
    caller's current torch stream is another one, order the two around the call."""

    def __init__(self, device: torch.device):
        self.device = device
        self.cur = torch.cuda.current_stream(device)
        self.default = torch.cuda.default_stream(device)
        self.foreign = self.cur != self.default

    def __enter__(self):
        if self.foreign:
            self.default.wait_stream(self.cur)
        return self

    def __exit__(self, *exc):
        if self.foreign:
            self.cur.wait_stream(self.default)
        return False


def mm_int8(A: torch.Tensor, B: torch.Tensor, scale_A: float, scale_B: float, scale_C: float,
            zero_point_A: int, zero_point_B: int, zero_point_C: int,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """C[M,N] int8 = requantised (A - zA) @ (B - zB); see include/texo_b200.h."""
    _check_cuda("A", A, torch.int8)
    _check_cuda("B", B, torch.int8)
    if A.dim() != 2 or B.dim() != 2 or A.shape[1] != B.shape[0]:
        raise ValueError(f"shape mismatch: A {tuple(A.shape)} B {tuple(B.shape)}")
    M, K = A.shape
    N = B.shape[1]
    if M <= 0 or N <= 0:
        raise ValueError("M and N must be positive")
    if out is None:
        out = torch.empty((M, N), dtype=torch.int8, device=A.device)
    else:
        _check_cuda("out", out, torch.int8)
        if tuple(out.shape) != (M, N):
            raise ValueError("out has the wrong shape")
    lib = _lib.load()
    with torch.cuda.device(A.device), _DefaultStreamOrder(A.device):
        lib.texo_mm_int8_solve(A.data_ptr() if K else None, B.data_ptr() if K else None,
                               out.data_ptr(), M, N, K, scale_A, scale_B, scale_C,
                               zero_point_A, zero_point_B, zero_point_C)
    return out


def mm_int8_per_channel(A: torch.Tensor, B: torch.Tensor, scale_A: float, scale_B: torch.Tensor,
                        scale_C: float, zero_point_A: int, zero_point_B: torch.Tensor | None,
                        zero_point_C: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """mm_int8 with one weight scale (fp32 [N]) and optionally one weight zero point (int32 [N])
    per output column, both CUDA tensors; see include/texo_b200.h."""
    _check_cuda("A", A, torch.int8)
    _check_cuda("B", B, torch.int8)
    _check_cuda("scale_B", scale_B, torch.float32)
    if A.dim() != 2 or B.dim() != 2 or A.shape[1] != B.shape[0]:
        raise ValueError(f"shape mismatch: A {tuple(A.shape)} B {tuple(B.shape)}")
    M, K = A.shape
    N = B.shape[1]
    if M <= 0 or N <= 0 or tuple(scale_B.shape) != (N,):
        raise ValueError("M, N must be positive and scale_B must be [N]")
    if zero_point_B is not None:
        _check_cuda("zero_point_B", zero_point_B, torch.int32)
        if tuple(zero_point_B.shape) != (N,):
            raise ValueError("zero_point_B must be [N]")
    if out is None:
        out = torch.empty((M, N), dtype=torch.int8, device=A.device)
    else:
        _check_cuda("out", out, torch.int8)
        if tuple(out.shape) != (M, N):
            raise ValueError("out has the wrong shape")
    lib = _lib.load()
    with torch.cuda.device(A.device), _DefaultStreamOrder(A.device):
        lib.texo_mm_int8_solve_per_channel(
            A.data_ptr() if K else None, B.data_ptr() if K else None, out.data_ptr(), M, N, K,
            scale_A, scale_B.data_ptr(), scale_C, zero_point_A,
            zero_point_B.data_ptr() if zero_point_B is not None else None, zero_point_C)
    return out


def mm_int8_swiglu(A: torch.Tensor, B_gu: torch.Tensor, scale_A: float, scale_gate: float,
                   scale_up: float, scale_H: float, zero_point_A: int, zero_point_gate: int,
                   zero_point_up: int, zero_point_H: int,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """H[M,F] int8 = requantised up * silu(gate), with gate / up the interleaved columns of
    A @ B_gu (B_gu [K, 2F]); see include/texo_b200.h."""
    _check_cuda("A", A, torch.int8)
    _check_cuda("B_gu", B_gu, torch.int8)
    if A.dim() != 2 or B_gu.dim() != 2 or A.shape[1] != B_gu.shape[0] or B_gu.shape[1] % 2:
        raise ValueError(f"shape mismatch: A {tuple(A.shape)} B_gu {tuple(B_gu.shape)}")
    M, K = A.shape
    F = B_gu.shape[1] // 2
    if M <= 0 or F <= 0:
        raise ValueError("M and F must be positive")
    if out is None:
        out = torch.empty((M, F), dtype=torch.int8, device=A.device)
    else:
        _check_cuda("out", out, torch.int8)
        if tuple(out.shape) != (M, F):
            raise ValueError("out has the wrong shape")
    lib = _lib.load()
    with torch.cuda.device(A.device), _DefaultStreamOrder(A.device):
        lib.texo_mm_int8_swiglu_solve(A.data_ptr() if K else None, B_gu.data_ptr() if K else None,
                                      out.data_ptr(), M, F, K, scale_A, scale_gate, scale_up, scale_H,
                                      zero_point_A, zero_point_gate, zero_point_up, zero_point_H)
    return out


def mm_int8_dequant(A: torch.Tensor, B: torch.Tensor, scale_A: float, scale_B: float,
                    zero_point_A: int, zero_point_B: int,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """Y[M,N] fp16 = half(float(sum_k (A - zA)(B - zB)) * scale_A * scale_B)."""
    _check_cuda("A", A, torch.int8)
    _check_cuda("B", B, torch.int8)
    if A.dim() != 2 or B.dim() != 2 or A.shape[1] != B.shape[0]:
        raise ValueError(f"shape mismatch: A {tuple(A.shape)} B {tuple(B.shape)}")
    M, K = A.shape
    N = B.shape[1]
    if M <= 0 or N <= 0:
        raise ValueError("M and N must be positive")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=A.device)
    else:
        _check_cuda("out", out, torch.float16)
        if tuple(out.shape) != (M, N):
            raise ValueError("out has the wrong shape")
    lib = _lib.load()
    with torch.cuda.device(A.device), _DefaultStreamOrder(A.device):
        lib.texo_mm_int8_dequant_solve(A.data_ptr() if K else None, B.data_ptr() if K else None,
                                       out.data_ptr(), M, N, K, scale_A, scale_B, zero_point_A, zero_point_B)
    return out


def mm_int4(x: torch.Tensor, w_q: torch.Tensor, scales: torch.Tensor, group_size: int,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """y[M,N] fp16 = x[M,K] @ dequant(w_q[N,K/2], scales[N,K/G])^T (W4A16)."""
    _check_cuda("x", x, torch.float16)
    _check_cuda("w_q", w_q, torch.uint8)
    _check_cuda("scales", scales, torch.float16)
    M, K = x.shape
    N = w_q.shape[0]
    if K % 2 or w_q.shape[1] != K // 2:
        raise ValueError("w_q must be [N, K/2] with even K")
    if group_size <= 0 or K % group_size or tuple(scales.shape) != (N, K // group_size):
        raise ValueError("scales must be [N, K/group_size]")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=x.device)
    else:
        _check_cuda("out", out, torch.float16)
    lib = _lib.load()
    with torch.cuda.device(x.device), _DefaultStreamOrder(x.device):
        lib.texo_mm_int4_solve(x.data_ptr(), w_q.data_ptr(), scales.data_ptr(), out.data_ptr(),
                               M, N, K, group_size)
    return out


def mm_int4a8(A: torch.Tensor, w_q: torch.Tensor, scale_A: float, scale_B: float, scale_C: float,
              zero_point_A: int, zero_point_B: int, zero_point_C: int,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """C[M,N] int8 = requantised (A - zA) @ (unpack(w_q) - zB)^T with w_q [N,K/2] packed
    nibbles in the mm_int4 format (W4A8); see include/texo_b200.h."""
    _check_cuda("A", A, torch.int8)
    _check_cuda("w_q", w_q, torch.uint8)
    if A.dim() != 2 or w_q.dim() != 2:
        raise ValueError("A and w_q must be matrices")
    M, K = A.shape
    N = w_q.shape[0]
    if K % 2 or w_q.shape[1] != K // 2:
        raise ValueError("w_q must be [N, K/2] with even K")
    if M <= 0 or N <= 0:
        raise ValueError("M and N must be positive")
    if out is None:
        out = torch.empty((M, N), dtype=torch.int8, device=A.device)
    else:
        _check_cuda("out", out, torch.int8)
        if tuple(out.shape) != (M, N):
            raise ValueError("out has the wrong shape")
    lib = _lib.load()
    with torch.cuda.device(A.device), _DefaultStreamOrder(A.device):
        lib.texo_mm_int4a8_solve(A.data_ptr() if K else None, w_q.data_ptr() if K else None,
                                 out.data_ptr(), M, N, K, scale_A, scale_B, scale_C,
                                 zero_point_A, zero_point_B, zero_point_C)
    return out


def mm_int4a8_per_channel(A: torch.Tensor, w_q: torch.Tensor, scale_A: float, scale_B: torch.Tensor,
                          scale_C: float, zero_point_A: int, zero_point_B: torch.Tensor | None,
                          zero_point_C: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """mm_int4a8 with one weight scale (fp32 [N]) and optionally one weight zero point (int32
    [N]) per output column (= row of w_q), both CUDA tensors; see include/texo_b200.h."""
    _check_cuda("A", A, torch.int8)
    _check_cuda("w_q", w_q, torch.uint8)
    _check_cuda("scale_B", scale_B, torch.float32)
    if A.dim() != 2 or w_q.dim() != 2:
        raise ValueError("A and w_q must be matrices")
    M, K = A.shape
    N = w_q.shape[0]
    if K % 2 or w_q.shape[1] != K // 2:
        raise ValueError("w_q must be [N, K/2] with even K")
    if M <= 0 or N <= 0 or tuple(scale_B.shape) != (N,):
        raise ValueError("M, N must be positive and scale_B must be [N]")
    if zero_point_B is not None:
        _check_cuda("zero_point_B", zero_point_B, torch.int32)
        if tuple(zero_point_B.shape) != (N,):
            raise ValueError("zero_point_B must be [N]")
    if out is None:
        out = torch.empty((M, N), dtype=torch.int8, device=A.device)
    else:
        _check_cuda("out", out, torch.int8)
        if tuple(out.shape) != (M, N):
            raise ValueError("out has the wrong shape")
    lib = _lib.load()
    with torch.cuda.device(A.device), _DefaultStreamOrder(A.device):
        lib.texo_mm_int4a8_solve_per_channel(
            A.data_ptr() if K else None, w_q.data_ptr() if K else None, out.data_ptr(), M, N, K,
            scale_A, scale_B.data_ptr(), scale_C, zero_point_A,
            zero_point_B.data_ptr() if zero_point_B is not None else None, zero_point_C)
    return out


def mm_int8_per_group(A: torch.Tensor, B: torch.Tensor, group_size: int, scale_A: float,
                      scale_B: torch.Tensor, scale_C: float, zero_point_A: int, zero_point_B: int,
                      zero_point_C: int) -> torch.Tensor:
    """mm_int8 with one weight scale per scale group of `group_size` consecutive k and output
    column: scale_B fp32 [K / group_size, N] on the device; see include/texo_b200.h."""
    _check_cuda("A", A, torch.int8)
    _check_cuda("B", B, torch.int8)
    _check_cuda("scale_B", scale_B, torch.float32)
    if A.dim() != 2 or B.dim() != 2 or A.shape[1] != B.shape[0]:
        raise ValueError("A must be [M, K] and B [K, N]")
    M, K = A.shape
    N = B.shape[1]
    if M <= 0 or N <= 0 or K <= 0 or group_size <= 0 or K % group_size:
        raise ValueError("M, N, K must be positive and group_size must divide K")
    if tuple(scale_B.shape) != (K // group_size, N):
        raise ValueError("scale_B must be [K / group_size, N]")
    out = torch.empty((M, N), dtype=torch.int8, device=A.device)
    lib = _lib.load()
    with torch.cuda.device(A.device), _DefaultStreamOrder(A.device):
        lib.texo_mm_int8_solve_per_group(A.data_ptr(), B.data_ptr(), out.data_ptr(), M, N, K, group_size,
                                         scale_A, scale_B.data_ptr(), scale_C, zero_point_A, zero_point_B,
                                         zero_point_C)
    return out


def mm_int4a8_per_group(A: torch.Tensor, w_q: torch.Tensor, group_size: int, scale_A: float,
                        scale_B: torch.Tensor, scale_C: float, zero_point_A: int, zero_point_B: int,
                        zero_point_C: int) -> torch.Tensor:
    """mm_int4a8 with per-group weight scales: scale_B fp32 [N, K / group_size] on the device (the
    layout of the reference's W4A16 scales); see include/texo_b200.h."""
    _check_cuda("A", A, torch.int8)
    _check_cuda("w_q", w_q, torch.uint8)
    _check_cuda("scale_B", scale_B, torch.float32)
    if A.dim() != 2 or w_q.dim() != 2:
        raise ValueError("A and w_q must be matrices")
    M, K = A.shape
    N = w_q.shape[0]
    if K <= 0 or K % 2 or w_q.shape[1] != K // 2:
        raise ValueError("w_q must be [N, K/2] with even K > 0")
    if M <= 0 or N <= 0 or group_size <= 0 or K % group_size:
        raise ValueError("M, N must be positive and group_size must divide K")
    if tuple(scale_B.shape) != (N, K // group_size):
        raise ValueError("scale_B must be [N, K / group_size]")
    out = torch.empty((M, N), dtype=torch.int8, device=A.device)
    lib = _lib.load()
    with torch.cuda.device(A.device), _DefaultStreamOrder(A.device):
        lib.texo_mm_int4a8_solve_per_group(A.data_ptr(), w_q.data_ptr(), out.data_ptr(), M, N, K, group_size,
                                           scale_A, scale_B.data_ptr(), scale_C, zero_point_A, zero_point_B,
                                           zero_point_C)
    return out


def dequantization(X: torch.Tensor, S: torch.Tensor, T: int,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """Y[M,N] fp32 = X * S[m // T][n // T]."""
    _check_cuda("X", X, torch.float32)
    _check_cuda("S", S, torch.float32)
    M, N = X.shape
    if T <= 0 or tuple(S.shape) != ((M + T - 1) // T, (N + T - 1) // T):
        raise ValueError("S must be [ceil(M/T), ceil(N/T)]")
    if out is None:
        out = torch.empty_like(X)
    else:
        _check_cuda("out", out, torch.float32)
    lib = _lib.load()
    with torch.cuda.device(X.device), _DefaultStreamOrder(X.device):
        lib.texo_dequantization_solve(X.data_ptr(), S.data_ptr(), out.data_ptr(), M, N, T)
    return out


def _check_norm_inputs(x, residual, weight):
    _check_cuda("x", x, torch.float32)
    _check_cuda("residual", residual, torch.float32)
    _check_cuda("weight", weight, torch.float32)
    if x.dim() != 2 or residual.shape != x.shape or tuple(weight.shape) != (x.shape[1],):
        raise ValueError("x, residual must be [N, C] and weight [C]")
    if x.shape[0] <= 0 or x.shape[1] <= 0:
        raise ValueError("N and C must be positive")


def rms_norm_w_residual(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                        out: torch.Tensor | None = None) -> torch.Tensor:
    """out[N,C] fp32 = (x + residual) * rsqrt(mean((x + residual)^2) + eps) * weight."""
    _check_norm_inputs(x, residual, weight)
    if out is None:
        out = torch.empty_like(x)
    else:
        _check_cuda("out", out, torch.float32)
        if out.shape != x.shape:
            raise ValueError("out has the wrong shape")
    lib = _lib.load()
    with torch.cuda.device(x.device), _DefaultStreamOrder(x.device):
        lib.texo_rms_norm_w_residual_solve(x.data_ptr(), residual.data_ptr(), weight.data_ptr(),
                                           out.data_ptr(), x.shape[0], x.shape[1], eps)
    return out


def rms_norm_quant(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                   scale: float, zero_point: int, out: torch.Tensor | None = None,
                   z_out: torch.Tensor | None = None,
                   row_sum_out: torch.Tensor | None = None) -> torch.Tensor:
    """q[N,C] int8 = clamp(rint(rms_norm_w_residual(...) / scale) + zero_point); z_out, if
    given, receives x + residual, row_sum_out (int32 [N]) the row sums of q.  The int8
    activations feed mm_int8 / mm_int4a8 as A, the row sums Int8Weights.matmul(row_sum=...)."""
    _check_norm_inputs(x, residual, weight)
    if not (scale == scale) or scale == 0.0:
        raise ValueError("scale must be finite and non-zero")
    if out is None:
        out = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    else:
        _check_cuda("out", out, torch.int8)
        if out.shape != x.shape:
            raise ValueError("out has the wrong shape")
    if z_out is not None:
        _check_cuda("z_out", z_out, torch.float32)
        if z_out.shape != x.shape:
            raise ValueError("z_out has the wrong shape")
    if row_sum_out is not None:
        _check_cuda("row_sum_out", row_sum_out, torch.int32)
        if tuple(row_sum_out.shape) != (x.shape[0],):
            raise ValueError("row_sum_out must be [N]")
    lib = _lib.load()
    with torch.cuda.device(x.device), _DefaultStreamOrder(x.device):
        lib.texo_rms_norm_quant_solve(x.data_ptr(), residual.data_ptr(), weight.data_ptr(),
                                      out.data_ptr(), z_out.data_ptr() if z_out is not None else None,
                                      row_sum_out.data_ptr() if row_sum_out is not None else None,
                                      x.shape[0], x.shape[1], eps, scale, zero_point)
    return out


def mm_int8_host(A_host: torch.Tensor, B_host: torch.Tensor, C_host: torch.Tensor,
                 scale_A: float, scale_B: float, scale_C: float,
                 zero_point_A: int, zero_point_B: int, zero_point_C: int) -> None:
    """mm_int8 on HOST tensors (pin them for full speed): what the reference harness does around
    `solve` (upload A and B, run, download C; tests/mm_int8.cpp:56-79), pipelined in row chunks
    by the library so that uploads, compute and downloads overlap.  Asynchronous: synchronise
    the device before reading C_host."""
    for name, t in (("A_host", A_host), ("B_host", B_host), ("C_host", C_host)):
        if not isinstance(t, torch.Tensor) or t.is_cuda or t.dtype != torch.int8 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous CPU int8 tensor")
    M, K = A_host.shape
    N = B_host.shape[1]
    if B_host.shape[0] != K or tuple(C_host.shape) != (M, N):
        raise ValueError("shape mismatch")
    rc = _lib.load().texo_mm_int8_solve_host(A_host.data_ptr(), B_host.data_ptr(), C_host.data_ptr(),
                                             M, N, K, scale_A, scale_B, scale_C, zero_point_A,
                                             zero_point_B, zero_point_C)
    if rc != 0:
        raise RuntimeError(f"texo_mm_int8_solve_host failed with code {rc}")


class Int8Weights:
    """A device-resident weight matrix B [K,N] prepared once for repeated mm_int8 calls: the
    library computes colsum(B) at construction and reuses it, so each call only sums the rows
    of its activations.  Results are bit-identical to `mm_int8`.  Keep B unchanged."""

    def __init__(self, B: torch.Tensor):
        _check_cuda("B", B, torch.int8)
        if B.dim() != 2 or B.shape[0] <= 0 or B.shape[1] <= 0:
            raise ValueError("B must be a non-empty [K, N] matrix")
        self.B = B  # keeps the storage alive
        self.K, self.N = B.shape
        self._lib = _lib.load()
        with torch.cuda.device(B.device), _DefaultStreamOrder(B.device):
            self._handle = self._lib.texo_mm_int8_prepare_weights(B.data_ptr(), self.K, self.N)
        if not self._handle:
            raise RuntimeError("texo_mm_int8_prepare_weights failed")

    def matmul(self, A: torch.Tensor, scale_A: float, scale_B: float, scale_C: float,
               zero_point_A: int, zero_point_B: int, zero_point_C: int,
               out: torch.Tensor | None = None, row_sum: torch.Tensor | None = None) -> torch.Tensor:
        """`row_sum` (int32 [M], optional): the row sums of A, if their producer computed them
        (rms_norm_quant(row_sum_out=...)); the call then runs no pre-pass at all."""
        _check_cuda("A", A, torch.int8)
        if A.dim() != 2 or A.shape[1] != self.K:
            raise ValueError(f"A must be [M, {self.K}]")
        M = A.shape[0]
        if out is None:
            out = torch.empty((M, self.N), dtype=torch.int8, device=A.device)
        else:
            _check_cuda("out", out, torch.int8)
        if row_sum is not None:
            _check_cuda("row_sum", row_sum, torch.int32)
            if tuple(row_sum.shape) != (M,):
                raise ValueError("row_sum must be [M]")
        with torch.cuda.device(A.device), _DefaultStreamOrder(A.device):
            self._lib.texo_mm_int8_solve_presummed(
                A.data_ptr(), row_sum.data_ptr() if row_sum is not None else None, self._handle,
                out.data_ptr(), M, scale_A, scale_B, scale_C, zero_point_A, zero_point_B, zero_point_C)
        return out

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self._lib.texo_mm_int8_release_weights(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def last_path(op: str = "mm_int8") -> int:
    return getattr(_lib.load(), f"texo_{op}_last_path")()


def force_path(path: int) -> None:
    """Force the mm_int8 device path (0 auto, 1 generic, 2 tensor, 3 skinny); diagnostics."""
    _lib.load().texo_mm_int8_force_path(int(path))


def status(op: str = "mm_int8") -> int:
    """Reads and clears the library's error state for the current device (0 = clean)."""
    return getattr(_lib.load(), f"texo_{op}_status")()
