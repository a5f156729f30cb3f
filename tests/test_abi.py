"""CPU-only: the C-ABI libraries load and export every symbol the header declares."""
import ctypes
import os
import re

from tests import harness


def _declared_functions():
    text = open(os.path.join(harness.ROOT, "include", "texo_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"\b(texo_\w+)\s*\(", text)


def test_header_declares_the_operator_entry_points():
    names = _declared_functions()
    for op in ("mm_int8", "mm_int4", "dequantization", "mm_int4a8", "rms_norm_w_residual"):
        assert f"texo_{op}_solve" in names
    assert len(names) == len(set(names))


def test_combined_library_exports_every_declared_symbol(libs):
    lib = ctypes.CDLL(libs["texo_b200"])
    for name in _declared_functions():
        assert hasattr(lib, name), name


def test_per_operator_libraries_export_solve(libs):
    for op in ("mm_int8", "mm_int4", "dequantization", "mm_int4a8", "rms_norm_w_residual"):
        lib = ctypes.CDLL(libs[op])
        assert hasattr(lib, "solve"), op


def test_python_binding_lists_the_same_symbols():
    from texo_b200 import _lib

    assert set(_lib._SIGNATURES) == set(_declared_functions())
