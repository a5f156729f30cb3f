"""In-tree nvcc build of the CUDA libraries (sm_100a only).

Produces, next to this file:
  libmm_int8.so, libmm_int4.so, libdequantization.so   one `solve` each (reference ABI)
  libmm_int4a8.so                                      `solve` of the W4A8 operator (no
                                                       reference counterpart, same convention)
  librms_norm_w_residual.so                            `solve` of the reference's
                                                       rms_norm_w_residual + the quantising form
  libtexo_b200.so                                      all of them, `texo_<op>_solve` names

Mirrors the reference build rule (its Makefile:4-5,233-234: one operator source per binary,
`nvcc -O3 -arch=$(NVCC_ARCH)`), with the architecture fixed to sm_100a.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OPS = ("mm_int8", "mm_int4", "dequantization", "mm_int4a8", "rms_norm_w_residual")
EXTRA = ("capi", "peak_probe", "host_api")  # only in the combined library
HEADERS = ("ptx.cuh", "host_common.h", "requant.cuh", "skinny.cuh", "w4_decode.cuh", "w4a8_decode.cuh")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--cudart", "shared",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-Wall",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA libraries cannot be built")
    return nvcc


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout + proc.stderr, file=sys.stderr)


def lib_path(name: str) -> str:
    return os.path.join(HERE, f"lib{name}.so")


def build(force: bool = False, verbose: bool = False) -> dict[str, str]:
    """Compile whatever is out of date; returns {library name: path}."""
    nvcc = _nvcc()
    deps = [os.path.join(CSRC, h) for h in HEADERS]
    out = {}
    for op in OPS:
        src = os.path.join(CSRC, f"{op}.cu")
        target = lib_path(op)
        if force or _stale(target, [src] + deps):
            _run([nvcc, *NVCC_FLAGS, "-shared", "-o", target, src], verbose)
        out[op] = target
    combined = lib_path("texo_b200")
    srcs = [os.path.join(CSRC, f"{name}.cu") for name in OPS + EXTRA]
    if force or _stale(combined, srcs + deps):
        objs = []
        for op in OPS:
            obj = os.path.join(HERE, f"_{op}.o")
            _run([nvcc, *NVCC_FLAGS, f"-Dsolve=texo_{op}_solve", "-c", "-o", obj,
                  os.path.join(CSRC, f"{op}.cu")], verbose)
            objs.append(obj)
        for extra in EXTRA:
            obj = os.path.join(HERE, f"_{extra}.o")
            _run([nvcc, *NVCC_FLAGS, "-c", "-o", obj, os.path.join(CSRC, f"{extra}.cu")], verbose)
            objs.append(obj)
        _run([nvcc, *NVCC_FLAGS, "-shared", "-o", combined, *objs], verbose)
        for obj in objs:
            os.remove(obj)
    out["texo_b200"] = combined
    return out


if __name__ == "__main__":
    for name, path in build(force="--force" in sys.argv, verbose=True).items():
        print(f"{name}: {path}")
