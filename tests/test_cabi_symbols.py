"""CPU: libedb200.so builds, loads and exports every function include/edb200_ops.h and
include/edb200_shims.h declare (the latter: the reference's plugin entry points under their own C++
names, plus the plain-C doors to them)."""
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


def test_library_exports_the_plugin_entry_points():
    """The ed_cuda_<op>_custom_* functions keep the reference's C++ linkage (its dispatcher calls them as
    C++ functions), so they are looked up by their mangled names; the edb200_plugin_* doors are plain C."""
    import subprocess
    path = load_pkg_module("build").build()
    text = open(os.path.join(ROOT, "include", "edb200_shims.h")).read()
    cxx = sorted(set(re.findall(r"EDB200_API\s+bool\s+(ed_cuda_\w+)\s*\(", text)))
    plain = sorted(set(re.findall(r"EDB200_API[^;(]*?\b(edb200_plugin_\w+)\s*\(", text)))
    assert len(cxx) == 15 and len(plain) == 4
    exported = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True, check=True).stdout
    for name in cxx:
        assert re.search(rf"\b_Z\d+{name}P", exported), name        # _Z<len><name>P(K)11ggml_tensor...
    lib = ctypes.CDLL(path)
    assert not [n for n in plain if not hasattr(lib, n)]


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
