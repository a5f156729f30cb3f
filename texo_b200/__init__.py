"""B200-native quantized matmul operators behind the reference's `solve` C ABI.

  texo_b200.ops       mm_int8 / mm_int4 / dequantization on torch CUDA tensors
  texo_b200.sharded   column-sharded multi-GPU forms (one process per GPU)
  texo_b200.build     in-tree nvcc build of the libraries (sm_100a)
"""
from . import build  # noqa: F401

__all__ = ["ops", "sharded", "build"]


def __getattr__(name):
    # torch is imported only when the operators are used, so `import texo_b200` and the
    # build step work in a bare interpreter.
    if name in ("ops", "sharded"):
        import importlib

        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
