"""Pins the numpy oracle to the reference's own CPU callbacks: against the committed golden
vectors (tests/golden/ref_callbacks.npz, made by tests/golden/make_golden.py from the
reference tree) everywhere, and against the compiled callbacks themselves (oracle/_ref)
on fresh random inputs wherever that library has been built.  Bit-exact in both cases."""
import importlib.util
import os

import numpy as np
import pytest

from oracle import edb_oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
G = importlib.util.module_from_spec(spec)
spec.loader.exec_module(G)


def _oracle_outputs(d, pe):
    seq, heads, dh = d["rx"].shape
    return {
        "modulate": O.modulate(d["x"], d["shift"], d["scale"]),
        "residual_gate": O.residual_gate(d["y"], d["x"], d["gate"]),
        "rms_norm_mul_f16": O.rms_norm_mul_f16_callback(d["nx"], d["nw"], 1e-6).view(np.uint16),
        "rope": np.ascontiguousarray(O.apply_rope(d["rx"], pe).transpose(1, 0, 2)),   # -> [heads, seq, d]
    }


def _same_bits(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    assert a.shape == b.shape and a.dtype.itemsize == b.dtype.itemsize
    u = np.uint32 if a.dtype.itemsize == 4 else np.uint16
    return np.array_equal(a.view(u), b.view(u))


def test_oracle_matches_golden_vectors_of_the_reference_callbacks():
    gold = np.load(os.path.join(HERE, "golden", "ref_callbacks.npz"))
    d = G.inputs()
    pe = O.embed_nd(d["rpos"], (8, 28, 28), 10000.0)
    assert _same_bits(pe, gold["pe"])          # the generator's table is the oracle's own, kept for reference
    got = _oracle_outputs(d, pe)
    for k in ("modulate", "residual_gate", "rms_norm_mul_f16", "rope"):
        assert _same_bits(got[k], gold[k]), k


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_oracle_matches_compiled_reference_callbacks(seed):
    if not os.path.exists(G.LIB):
        pytest.skip("oracle/_ref/libedref_cpu.so not built (needs the reference tree)")
    lib = G.load_ref()
    d = G.inputs(seed)
    pe = O.embed_nd(d["rpos"], (8, 28, 28), 10000.0)
    ref = G.run_ref(lib, d, pe)
    got = _oracle_outputs(d, pe)
    for k in ref:
        assert _same_bits(got[k], ref[k]), k
