"""GPU parity of the Qwen-Image denoise-pass executor against the numpy oracle.  Tolerances as stated
for this path: per-block cosine >= 0.999 and relative L2 <= 1e-2, full-pass latent relative L2 <= 2e-2,
against the fp32 non-Sage CPU path on the same quantised weight bytes."""
import numpy as np
import pytest

from oracle import edb_oracle as O
from oracle.qwen_oracle import QwenConfig, QwenOracle, qwen_make_weights

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

BLOCK_COS, BLOCK_REL, STEP_REL = 0.999, 1e-2, 2e-2


def _run_case(edb, cuda, cfg, lat_hw, n_txt, attention, seed=0, timestep=500.0, std=0.02):
    weights = qwen_make_weights(cfg, seed, std=std)
    rng = np.random.default_rng(seed + 100)
    latent = rng.standard_normal((cfg.in_channels // cfg.patch_size ** 2,) + lat_hw, dtype=np.float32)
    ctx = rng.standard_normal((n_txt, cfg.joint_attention_dim), dtype=np.float32)
    taps = {}
    ref = QwenOracle(cfg, weights).forward(latent, timestep, ctx, taps)

    model = edb.QwenModel(num_layers=cfg.num_layers, num_heads=cfg.num_attention_heads, head_dim=cfg.attention_head_dim,
                          mlp_hidden=cfg.mlp_hidden, in_channels=cfg.in_channels, out_channels=cfg.out_channels,
                          joint_attention_dim=cfg.joint_attention_dim, patch_size=cfg.patch_size, axes_dim=cfg.axes_dim,
                          theta=cfg.theta, wtype=cfg.wtype, attention=attention)
    assert set(model.tensor_names()) == set(weights)
    model.load_numpy(weights)
    model.prepare(lat_hw[0], lat_hw[1], n_txt)
    n_img = (lat_hw[0] // cfg.patch_size) * (lat_hw[1] // cfg.patch_size)
    T = n_txt + n_img
    tap = torch.zeros(cfg.num_layers, T, cfg.hidden_size, dtype=torch.float32, device=cuda)
    model.set_tap(tap)
    d_lat, d_ctx = (torch.from_numpy(a).to(cuda) for a in (latent, ctx))
    d_out = torch.zeros(cfg.out_channels, *lat_hw, dtype=torch.float32, device=cuda)
    model.step(d_lat, timestep, d_ctx, d_out)
    torch.cuda.synchronize()
    got_taps, got = tap.cpu().numpy(), d_out.cpu().numpy()
    assert np.isfinite(got).all()
    report = []
    for i in range(cfg.num_layers):
        want = np.concatenate([taps[f"block{i}.txt"], taps[f"block{i}.img"]], axis=0)
        report.append((f"block{i}", O.cosine(got_taps[i], want), O.rel_l2(got_taps[i], want)))
    for name, cos, rel in report:
        assert cos >= BLOCK_COS and rel <= BLOCK_REL, (name, cos, rel, report)
    step_rel = O.rel_l2(got, ref)
    assert step_rel <= STEP_REL, (step_rel, report)
    model.set_tap(None)
    host = model.compute_host(latent, timestep, ctx)
    assert np.array_equal(host, got)


@pytest.mark.parametrize("attention", ["f16", "sage"])
def test_qwen_small_pass_parity(edb, cuda, attention):
    cfg = QwenConfig(num_layers=2, num_attention_heads=4, joint_attention_dim=256)
    att = edb.ATTN_F16 if attention == "f16" else edb.ATTN_SAGE_INT8
    _run_case(edb, cuda, cfg, (24, 40), 21, att, std=0.05)


def test_qwen_q8_0_pass_parity(edb, cuda):
    cfg = QwenConfig(num_layers=1, num_attention_heads=4, joint_attention_dim=256, wtype=O.GGML_TYPE_Q8_0)
    _run_case(edb, cuda, cfg, (16, 16), 9, edb.ATTN_SAGE_INT8, seed=3, std=0.05)


def test_qwen_full_width_block_parity(edb, cuda):
    # Qwen-Image widths (hidden 3072, 24 heads x 128, mlp 12288, text 3584, q4_K) with one block
    cfg = QwenConfig(num_layers=1)
    _run_case(edb, cuda, cfg, (32, 48), 77, edb.ATTN_SAGE_INT8, seed=5)


def test_qwen_guidance_combine_bit_exact(edb, cuda):
    """edb200_cfg_combine_rescaled against the oracle's restatement of the reference's per-patch
    norm-preserving guidance combine, bit for bit, including a patch whose guided value is all zero."""
    from oracle.qwen_oracle import true_cfg
    rng = np.random.default_rng(41)
    C_, H_, W_ = 16, 12, 20
    cond = rng.standard_normal((C_, H_, W_), dtype=np.float32)
    uncond = rng.standard_normal((C_, H_, W_), dtype=np.float32)
    cond[:, 2:4, 6:8] = 0.0
    uncond[:, 2:4, 6:8] = 0.0
    out = torch.full((C_, H_, W_), float("nan"), dtype=torch.float32, device=cuda)
    d_c, d_u = torch.from_numpy(cond).to(cuda), torch.from_numpy(uncond).to(cuda)
    edb.check(edb.lib().edb200_cfg_combine_rescaled(edb.ptr(d_u), edb.ptr(d_c), 4.0, 2, C_, H_, W_, edb.ptr(out),
                                                    edb.current_stream()))
    want = true_cfg(cond, uncond, 4.0, 2)
    got = out.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert not got[:, 2:4, 6:8].any()
    with pytest.raises(edb.EdbError):
        edb.check(edb.lib().edb200_cfg_combine_rescaled(edb.ptr(d_u), edb.ptr(d_c), 4.0, 2, C_, 11, W_, edb.ptr(out),
                                                        edb.current_stream()))
