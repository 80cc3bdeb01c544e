"""Pins the numpy oracle to the reference's own CPU callbacks and tensor arithmetic: against the committed golden
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
        "cfg": O.cfg_combine(d["su"], d["sv"], G.CFG_SCALE),
        **{f"euler{i}": O.euler_update(d["sx"], d["sv"], s, sn) for i, (s, sn) in enumerate(G.SIGMA_PAIRS)},
        **{f"flow{i}": O.flow_update(d["sx"], d["sv"], s, sn) for i, (s, sn) in enumerate(G.SIGMA_PAIRS)},
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
    assert set(got) == set(gold.files) - {"pe"}
    for k in got:
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


def test_oracle_euler_update_is_the_reference_sampler_step():
    """The per-step latent update restated in the oracle (flux_pipeline.cpp:1290-1297), checked
    against the same expression written out in float64 and against its fixed points."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal(4096, dtype=np.float32)
    v = rng.standard_normal(4096, dtype=np.float32)
    # sigma_next == sigma leaves the latent alone; sigma == 0 returns the denoised latent (= x here)
    assert np.array_equal(O.euler_update(x, v, 0.5, 0.5), x)
    assert np.array_equal(O.euler_update(x, v, 0.0, 0.0), x)
    # a full step to sigma_next = 0 lands on the denoised latent up to rounding
    got = O.euler_update(x, v, 0.8, 0.0)
    assert np.allclose(got, x.astype(np.float64) - 0.8 * v.astype(np.float64), rtol=0, atol=2e-6)
    # in exact arithmetic the update is x + v*(sigma_next - sigma)
    got = O.euler_update(x, v, 0.8, 0.55)
    assert np.allclose(got, x.astype(np.float64) + v.astype(np.float64) * (0.55 - 0.8), rtol=0, atol=2e-6)
    assert got.dtype == np.float32


def test_oracle_qwen_guidance_combine_keeps_the_conditional_norm():
    """Restated ed_qwen_apply_true_cfg (qwen_image_pipeline.cpp:29-85): every 2x2 patch of the result
    has the conditional prediction's norm, and equal branches pass through unchanged."""
    from oracle.qwen_oracle import true_cfg
    rng = np.random.default_rng(6)
    cond = rng.standard_normal((16, 8, 10), dtype=np.float32)
    uncond = rng.standard_normal((16, 8, 10), dtype=np.float32)
    out = true_cfg(cond, uncond, 4.0, 2)
    for py in range(0, 8, 2):
        for px in range(0, 10, 2):
            a = np.linalg.norm(out[:, py:py + 2, px:px + 2].astype(np.float64))
            b = np.linalg.norm(cond[:, py:py + 2, px:px + 2].astype(np.float64))
            assert abs(a - b) <= 1e-5 * b
    assert np.array_equal(true_cfg(cond, cond, 4.0, 2), cond)
    # direction is the plain guided combine's
    g = uncond + np.float32(4.0) * (cond - uncond)
    cosv = np.sum(out.astype(np.float64) * g) / (np.linalg.norm(out.astype(np.float64)) * np.linalg.norm(g.astype(np.float64)))
    assert cosv > 0.95
