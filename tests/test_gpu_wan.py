"""GPU parity of the Wan 2.1 denoise-step executor against the numpy oracle.

Tolerances are the ones the task states for this path: per-block output cosine
>= 0.999 and relative L2 <= 1e-2, full-step latent relative L2 <= 2e-2, against
the fp32 non-Sage CPU path on the same quantised weight bytes.
"""
import numpy as np
import pytest

from oracle import edb_oracle as O
from oracle.wan_oracle import WanConfig, WanOracle, wan_make_weights

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

BLOCK_COS, BLOCK_REL, STEP_REL = 0.999, 1e-2, 2e-2


def _make_model(edb, cfg, attention):
    return edb.WanModel(dim=cfg.dim, num_heads=cfg.num_heads, ffn_dim=cfg.ffn_dim, num_layers=cfg.num_layers,
                        in_dim=cfg.in_dim, out_dim=cfg.out_dim, text_dim=cfg.text_dim, freq_dim=cfg.freq_dim,
                        patch_size=cfg.patch_size, axes_dim=cfg.axes_dim, theta=cfg.theta, wtype=cfg.wtype,
                        attention=attention)


def _run_case(edb, cuda, cfg, lat_shape, n_ctx, attention, seed=0, timestep=500.0):
    weights = wan_make_weights(cfg, seed, std=0.05)
    rng = np.random.default_rng(seed + 100)
    latent = rng.standard_normal((cfg.in_dim,) + lat_shape, dtype=np.float32)
    ctx = rng.standard_normal((n_ctx, cfg.text_dim), dtype=np.float32)
    taps = {}
    ref = WanOracle(cfg, weights).forward(latent, timestep, ctx, taps)

    model = _make_model(edb, cfg, attention)
    buf_names = set()
    n = edb.lib().edb200_wan_tensor_count(model.handle)
    import ctypes as C
    buf = C.create_string_buffer(256)
    for i in range(n):
        edb.check(edb.lib().edb200_wan_tensor_info(model.handle, i, buf, 256, None, None, None, None))
        buf_names.add(buf.value.decode())
    assert buf_names == set(weights)                  # same parameter table as the reference's tensor names
    model.load_numpy(weights)
    model.prepare(*lat_shape, n_ctx)
    pt, ph, pw = cfg.patch_size
    T = (lat_shape[0] // pt) * (lat_shape[1] // ph) * (lat_shape[2] // pw)
    tap = torch.zeros(cfg.num_layers, T, cfg.dim, dtype=torch.float32, device=cuda)
    model.set_tap(tap)
    d_lat, d_ctx = (torch.from_numpy(a).to(cuda) for a in (latent, ctx))
    d_out = torch.zeros(cfg.out_dim, *lat_shape, dtype=torch.float32, device=cuda)
    model.step(d_lat, timestep, d_ctx, d_out)
    torch.cuda.synchronize()
    got_taps = tap.cpu().numpy()
    got = d_out.cpu().numpy()
    assert np.isfinite(got).all()
    report = [(f"block{i}", O.cosine(got_taps[i], taps[f"block{i}.x"]), O.rel_l2(got_taps[i], taps[f"block{i}.x"]))
              for i in range(cfg.num_layers)]
    for name, cos, rel in report:
        assert cos >= BLOCK_COS and rel <= BLOCK_REL, (name, cos, rel, report)
    step_rel = O.rel_l2(got, ref)
    assert step_rel <= STEP_REL, (step_rel, report)
    model.set_tap(None)
    host = model.compute_host(latent, timestep, ctx)
    assert np.array_equal(host, got)


@pytest.mark.parametrize("attention", ["f16", "sage"])
def test_wan_small_step_parity(edb, cuda, attention):
    cfg = WanConfig(dim=512, num_heads=4, ffn_dim=1024, num_layers=2, text_dim=128)
    att = edb.ATTN_F16 if attention == "f16" else edb.ATTN_SAGE_INT8
    # 3 latent frames of 16 x 24 -> 3 * 8 * 12 = 288 video tokens, 20 text tokens
    _run_case(edb, cuda, cfg, (3, 16, 24), 20, att)


def test_wan_q4_k_step_parity(edb, cuda):
    cfg = WanConfig(dim=512, num_heads=4, ffn_dim=1024, num_layers=1, text_dim=128, wtype=O.GGML_TYPE_Q4_K)
    _run_case(edb, cuda, cfg, (2, 8, 40), 7, edb.ATTN_SAGE_INT8, seed=3)


def test_wan_full_width_block_parity(edb, cuda):
    # Wan 2.1 14B layer widths (dim 5120, 40 heads x 128, ffn 13824, text 4096) with one block
    cfg = WanConfig(num_layers=1)
    _run_case(edb, cuda, cfg, (2, 12, 16), 33, edb.ATTN_SAGE_INT8, seed=5)


def test_wan_rejects_bad_shapes(edb, cuda):
    model = edb.WanModel(dim=512, num_heads=4, ffn_dim=1024, num_layers=1, text_dim=128)
    with pytest.raises(edb.EdbError):
        model.prepare(2, 15, 16, 8)                    # latent not a multiple of the patch size
    with pytest.raises(edb.EdbError):
        edb.WanModel(dim=500, num_heads=4)             # width not a multiple of 256


def test_wan_and_qwen_steps_follow_a_device_schedule(edb, cuda):
    """edb200_{wan,qwen}_step_sched read the timestep from a schedule in device memory (sigma * 1000) and give
    the bits of the by-value step."""
    lib = edb.lib()
    sched = torch.tensor([0.9, 0.35], dtype=torch.float32, device=cuda)
    step = torch.ones(1, dtype=torch.int32, device=cuda)               # points at 0.35
    t = float(np.float32(0.35) * np.float32(1000.0))
    wan = edb.WanModel(dim=512, num_heads=4, ffn_dim=1024, num_layers=2, text_dim=128)
    wan.init_random(seed=9, std=0.05)
    wan.prepare(2, 16, 20, 24)
    g = torch.Generator(device="cpu").manual_seed(12)
    lat, ctx = torch.randn(16, 2, 16, 20, generator=g).to(cuda), torch.randn(24, 128, generator=g).to(cuda)
    a, b = torch.empty_like(lat), torch.empty_like(lat)
    wan.step(lat, t, ctx, a)
    edb.check(lib.edb200_wan_step_sched(wan.handle, edb.ptr(lat), edb.ptr(sched), edb.ptr(step), 1000.0, edb.ptr(ctx),
                                        edb.ptr(b), edb.current_stream()))
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    qwen = edb.QwenModel(num_layers=2, num_heads=4, joint_attention_dim=256)
    qwen.init_random(seed=13, std=0.05)
    qwen.prepare(24, 24, 16)
    lat, ctx = torch.randn(16, 24, 24, generator=g).to(cuda), torch.randn(16, 256, generator=g).to(cuda)
    a, b = torch.empty_like(lat), torch.empty_like(lat)
    qwen.step(lat, t, ctx, a)
    edb.check(lib.edb200_qwen_step_sched(qwen.handle, edb.ptr(lat), edb.ptr(sched), edb.ptr(step), 1000.0, edb.ptr(ctx),
                                         edb.ptr(b), edb.current_stream()))
    torch.cuda.synchronize()
    assert torch.equal(a, b)
