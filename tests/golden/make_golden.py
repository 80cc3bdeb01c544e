"""Generates tests/golden/ref_callbacks.npz: outputs of the reference's own CPU callbacks and of
the pipelines' per-step latent arithmetic evaluated with the reference's tensor class
(oracle/_ref/libedref_cpu.so, built by oracle/build_ref.sh from the reference tree) on
seeded inputs.  Run where the reference tree is available:

    sh oracle/build_ref.sh && python tests/golden/make_golden.py
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
LIB = os.path.join(ROOT, "oracle", "_ref", "libedref_cpu.so")


def load_ref():
    lib = C.CDLL(LIB)
    vp, i64 = C.c_void_p, C.c_int64
    lib.ref_fused_modulate.argtypes = [vp, vp, vp, vp, i64, i64]
    lib.ref_fused_residual_gate.argtypes = [vp, vp, vp, vp, i64, i64]
    lib.ref_rms_norm_mul_f16.argtypes = [vp, vp, vp, i64, i64, C.c_float]
    lib.ref_rope_interleaved.argtypes = [vp, vp, vp, i64, i64, i64]
    lib.ref_tensor_euler_update.argtypes = [vp, vp, i64, C.c_float, C.c_float]
    lib.ref_tensor_flow_update.argtypes = [vp, vp, i64, C.c_float, C.c_float]
    lib.ref_tensor_cfg_combine.argtypes = [vp, vp, i64, C.c_float, vp]
    for f in (lib.ref_fused_modulate, lib.ref_fused_residual_gate, lib.ref_rms_norm_mul_f16, lib.ref_rope_interleaved,
              lib.ref_tensor_euler_update, lib.ref_tensor_flow_update, lib.ref_tensor_cfg_combine):
        f.restype = None
    return lib


# (sigma, sigma_next) pairs of the sampler updates, and the guidance scale of the combine
SIGMA_PAIRS = ((1.0, 0.9), (0.37, 0.0), (0.0, 0.0), (0.0123, 0.0045))
CFG_SCALE = 4.5


def p(a):
    return a.ctypes.data_as(C.c_void_p)


def inputs(seed=2024):
    """Seeded inputs shared by this script and the tests (values with a wide exponent spread,
    so that the rounding of every intermediate matters)."""
    rng = np.random.default_rng(seed)
    rows, h = 37, 96
    d = {
        "x": (rng.standard_normal((rows, h)) * np.exp(rng.uniform(-3, 3, (rows, h)))).astype(np.float32),
        "y": rng.standard_normal((rows, h)).astype(np.float32),
        "shift": rng.standard_normal(h).astype(np.float32),
        "scale": rng.standard_normal(h).astype(np.float32),
        "gate": rng.standard_normal(h).astype(np.float32),
        "nx": (rng.standard_normal((29, 128)) * 3).astype(np.float32),
        "nw": (1 + 0.1 * rng.standard_normal(128)).astype(np.float32),
        "rx": rng.standard_normal((21, 3, 64)).astype(np.float32),          # [seq, heads, d]
        "rpos": rng.integers(0, 40, (21, 3)).astype(np.float32),            # ids for axes (8, 28, 28)
    }
    # drawn after everything above, so that the earlier entries keep their values
    d["sx"] = (rng.standard_normal(4099) * np.exp(rng.uniform(-2, 2, 4099))).astype(np.float32)   # latent
    d["sv"] = rng.standard_normal(4099).astype(np.float32)                                       # prediction
    d["su"] = rng.standard_normal(4099).astype(np.float32)                                       # unconditional
    return d


def run_ref(lib, d, pe):
    out = {}
    rows, h = d["x"].shape
    o = np.empty_like(d["x"])
    lib.ref_fused_modulate(p(d["x"]), p(d["shift"]), p(d["scale"]), p(o), rows, h)
    out["modulate"] = o.copy()
    lib.ref_fused_residual_gate(p(d["y"]), p(d["x"]), p(d["gate"]), p(o), rows, h)
    out["residual_gate"] = o.copy()
    n = np.empty(d["nx"].shape, dtype=np.uint16)
    lib.ref_rms_norm_mul_f16(p(d["nx"]), p(d["nw"]), p(n), d["nx"].shape[0], d["nx"].shape[1], 1e-6)
    out["rms_norm_mul_f16"] = n
    seq, heads, dh = d["rx"].shape
    r = np.empty((heads, seq, dh), dtype=np.float32)
    pe_c = np.ascontiguousarray(pe, dtype=np.float32)
    lib.ref_rope_interleaved(p(d["rx"]), p(pe_c), p(r), seq, heads, dh)
    out["rope"] = r
    n = d["sx"].size
    for i, (s, s_next) in enumerate(SIGMA_PAIRS):
        x = d["sx"].copy()
        lib.ref_tensor_euler_update(p(x), p(d["sv"]), n, s, s_next)
        out[f"euler{i}"] = x
        x = d["sx"].copy()
        lib.ref_tensor_flow_update(p(x), p(d["sv"]), n, s, s_next)
        out[f"flow{i}"] = x
    o = np.empty_like(d["sx"])
    lib.ref_tensor_cfg_combine(p(d["su"]), p(d["sv"]), n, CFG_SCALE, p(o))
    out["cfg"] = o
    return out


if __name__ == "__main__":
    import sys
    sys.path.insert(0, ROOT)
    from oracle import edb_oracle as O
    d = inputs()
    pe = O.embed_nd(d["rpos"], (8, 28, 28), 10000.0)
    out = run_ref(load_ref(), d, pe)
    np.savez_compressed(os.path.join(HERE, "ref_callbacks.npz"), pe=pe, **out)
    print("wrote", os.path.join(HERE, "ref_callbacks.npz"), {k: v.shape for k, v in out.items()})
