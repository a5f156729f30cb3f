"""Regenerates the golden fixtures in this directory.  Run from the repository root:

    python tests/golden/make_golden.py

mm_int8_harness.npz   the 56 default cases of the reference harness
                      (frezcirno/Texo tests/mm_int8.cpp:139-254): inputs, quantisation
                      parameters, pointer offsets and the expected bytes.  Of the 56
                      expectations, 2 are reference-held: the bytes the reference test file
                      pins (:210-221, meta "pinned": true).  The other 54 are ORACLE-GENERATED:
                      the oracle's restatement (mode 1) of the harness's double-precision
                      formula (:39-48), i.e. what the harness would compute and compare
                      against - they are not bytes produced by reference code.  (The reference's
                      compiled CPU loop itself checks the oracle in
                      tests/test_oracle.py::test_reference_cpu_loops_accept_the_oracle, and
                      its recompiled kernel checks the GPU path in the -m gpu tests.)
mm_int4_example.npz   the pinned example of tests/mm_int4.cpp:110-117 with the value of its
                      double reference (:35-45).
The inputs come from the restated generators in oracle/harness_inputs.cpp (same mt19937
streams as the harness).
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests import harness  # noqa: E402


def main():
    oracle = harness.load_oracle()
    cases = harness.mm_int8_harness_cases(oracle)
    arrays, meta = {}, []
    for i, c in enumerate(cases):
        expected = c["known"]
        if expected is None:
            expected = oracle.mm_int8(c["a"], c["b"], c["m"], c["n"], c["k"], c["q"], mode=1)
        arrays[f"a{i}"] = c["a"]
        arrays[f"b{i}"] = c["b"]
        arrays[f"e{i}"] = np.asarray(expected, dtype=np.int8).reshape(c["m"], c["n"])
        meta.append(dict(name=c["name"], m=c["m"], n=c["n"], k=c["k"], q=list(c["q"]),
                         offsets=list(c["offsets"]), pinned=c["known"] is not None))
    arrays["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(harness.GOLDEN_DIR, "mm_int8_harness.npz"), **arrays)
    print(f"mm_int8_harness.npz: {len(cases)} cases")

    x = harness.float_to_half_bits([1, 0, 1, 0, 0, 1, 0, 1]).reshape(2, 4)
    w = np.array([153, 153, 170, 170, 119, 119, 136, 136], dtype=np.uint8).reshape(4, 2)
    s = harness.float_to_half_bits([0.5] * 8).reshape(4, 2)
    y = oracle.mm_int4(x, w, s, 2, 4, 4, 2)
    np.savez_compressed(os.path.join(harness.GOLDEN_DIR, "mm_int4_example.npz"), x=x, w=w, s=s, y=y)
    print("mm_int4_example.npz:", y.tolist())


if __name__ == "__main__":
    main()
