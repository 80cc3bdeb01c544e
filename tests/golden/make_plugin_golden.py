"""Generates tests/golden/plugin_cases.npz: the outputs of the reference's own CPU callbacks
(oracle/_ref/libedref_cpu.so, built by oracle/build_ref.sh from the reference tree) for every custom-op
node of tests/plugin_cases.py.  Run where the reference tree is available:

    sh oracle/build_ref.sh && python tests/golden/make_plugin_golden.py
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "tests"))
import plugin_cases as P  # noqa: E402

LIB = os.path.join(ROOT, "oracle", "_ref", "libedref_cpu.so")

if __name__ == "__main__":
    lib = C.CDLL(LIB)
    out = {name: P.run_reference(lib, node) for name, node in P.cases().items()}
    np.savez_compressed(os.path.join(HERE, "plugin_cases.npz"), **out)
    print("wrote plugin_cases.npz", {k: (v.shape, str(v.dtype)) for k, v in out.items()})
