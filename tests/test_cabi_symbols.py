"""CPU: libedb200.so builds, loads and exports every function include/edb200_ops.h declares."""
import ctypes
import os
import re

from conftest import ROOT, load_pkg_module


def _declared():
    text = open(os.path.join(ROOT, "include", "edb200_ops.h")).read()
    return sorted(set(re.findall(r"EDB200_API[^;(]*?\b(edb200_\w+)\s*\(", text)))


def test_header_declares_functions():
    names = _declared()
    assert "edb200_mul_mat_q" in names and "edb200_last_error" in names and len(names) >= 15


def test_library_exports_every_declared_symbol():
    path = load_pkg_module("build").build()
    lib = ctypes.CDLL(path)
    missing = [n for n in _declared() if not hasattr(lib, n)]
    assert not missing, f"not exported: {missing}"


def test_binding_matches_header():
    edb = load_pkg_module("edb200")
    assert sorted(edb.declared_symbols()) == _declared()


def test_error_string_without_device():
    edb = load_pkg_module("edb200")
    lib = edb.lib()
    assert lib.edb200_version().decode().startswith("edb200")
    # argument validation happens before any CUDA call: no device is needed to see it
    st = lib.edb200_fused_modulate(None, None, None, None, 4, 8, None)
    assert st == 1 and b"fused_modulate" in lib.edb200_last_error()
