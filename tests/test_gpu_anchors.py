"""The computation-reuse seam of the SD3, Wan and Qwen-Image executors (the reference taps the same three
anchors in every model graph: mmdit.hpp:3318-3385, wan.hpp:4640-4729, qwen_image.hpp:3209-3274): ModelIn /
BlockOut[i] / ModelOut captures equal the stream at those points, the probe stop returns after the chosen
block without touching the output, and a step with the stored residual injected runs no block and reproduces
the full step's output.  The FLUX form of the same test is in test_gpu_flux.py."""
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _sd3(edb, cuda, g):
    m = edb.SD3Model(hidden_size=512, num_heads=8, depth=3, context_size=256, adm_in_channels=64, pos_embed_max_size=32)
    m.init_random(seed=4, std=0.05)
    n_ctx = 20
    m.prepare(32, 32, n_ctx)
    lat, ctx, y = (torch.randn(16, 32, 32, generator=g).to(cuda), torch.randn(n_ctx, 256, generator=g).to(cuda),
                   torch.randn(64, generator=g).to(cuda))
    # stream: the 256 image rows after the 20 context rows of the tap
    return m, "sd3", 3, 512, 256, slice(n_ctx, n_ctx + 256), n_ctx + 256, lambda out: m.step(lat, 500.0, ctx, y, out), lat


def _wan(edb, cuda, g):
    m = edb.WanModel(dim=512, num_heads=4, ffn_dim=1024, num_layers=3, text_dim=128, attention=edb.ATTN_F16)
    m.init_random(seed=5, std=0.05)
    n_ctx = 16
    m.prepare(3, 16, 16, n_ctx)
    lat, ctx = torch.randn(16, 3, 16, 16, generator=g).to(cuda), torch.randn(n_ctx, 128, generator=g).to(cuda)
    rows = 3 * 8 * 8
    return m, "wan", 3, 512, rows, slice(0, rows), rows, lambda out: m.step(lat, 500.0, ctx, out), lat


def _qwen(edb, cuda, g):
    m = edb.QwenModel(num_layers=3, num_heads=4, joint_attention_dim=256, attention=edb.ATTN_F16)
    m.init_random(seed=6, std=0.05)
    n_txt = 12
    m.prepare(32, 32, n_txt)
    lat, ctx = torch.randn(16, 32, 32, generator=g).to(cuda), torch.randn(n_txt, 256, generator=g).to(cuda)
    return m, "qwen", 3, 512, 256, slice(n_txt, n_txt + 256), n_txt + 256, lambda out: m.step(lat, 500.0, ctx, out), lat


@pytest.mark.parametrize("make", [_sd3, _wan, _qwen], ids=["sd3", "wan", "qwen"])
def test_reuse_anchors_capture_probe_and_inject(edb, cuda, make):
    lib = edb.lib()
    g = torch.Generator(device="cpu").manual_seed(9)
    model, fam, depth, width, rows, stream, tap_rows, step, lat = make(edb, cuda, g)
    set_capture = getattr(lib, f"edb200_{fam}_set_anchor_capture")
    set_stop = getattr(lib, f"edb200_{fam}_set_stop_after")
    set_override = getattr(lib, f"edb200_{fam}_set_stream_override")
    tap = torch.zeros(depth, tap_rows, width, device=cuda)
    model.set_tap(tap)
    a_in, a_b1, a_out = (torch.zeros(rows, width, device=cuda) for _ in range(3))
    edb.check(set_capture(model.handle, edb.ANCHOR_MODEL_IN, edb.ptr(a_in)))
    edb.check(set_capture(model.handle, 1, edb.ptr(a_b1)))
    edb.check(set_capture(model.handle, edb.ANCHOR_MODEL_OUT, edb.ptr(a_out)))
    full = torch.empty_like(lat)
    step(full)
    torch.cuda.synchronize()
    assert torch.equal(a_b1, tap[1, stream]) and torch.equal(a_out, tap[depth - 1, stream])
    assert torch.isfinite(a_in).all() and not torch.equal(a_in, a_out)
    assert set_capture(model.handle, depth, None) != 0 and set_stop(model.handle, depth) != 0   # out of range
    # probe: stop after block 1; the output is not written
    launches = lib.edb200_launch_count()
    edb.check(set_stop(model.handle, 1))
    probe_out = torch.full_like(lat, float("nan"))
    a_b1.zero_()
    step(probe_out)
    torch.cuda.synchronize()
    probe_launches = lib.edb200_launch_count() - launches
    assert torch.equal(a_b1, tap[1, stream]) and torch.isnan(probe_out).all()
    edb.check(set_stop(model.handle, -1))
    # inject: residual = ModelOut - ModelIn, no block runs
    residual = torch.empty_like(a_in)
    edb.check(lib.edb200_sub_f32(edb.ptr(a_out), edb.ptr(a_in), edb.ptr(residual), residual.numel(), edb.current_stream()))
    edb.check(set_override(model.handle, edb.ptr(residual)))
    launches = lib.edb200_launch_count()
    reused = torch.empty_like(lat)
    step(reused)
    torch.cuda.synchronize()
    assert lib.edb200_launch_count() - launches < probe_launches
    rel = float(torch.linalg.vector_norm(reused - full) / torch.linalg.vector_norm(full))
    assert rel < 1e-5, rel                                   # in + (out - in) rounds once more
    edb.check(set_override(model.handle, None))
    again = torch.empty_like(lat)
    step(again)
    torch.cuda.synchronize()
    assert torch.equal(again, full)


def test_wan_region_inject_skips_a_cached_span(edb, cuda):
    """Region inject (wan.hpp:4658-4665): at block 1 the stream becomes ModelIn + residual and block 1 is skipped.
    With residual = BlockOut[1] - ModelIn of a full step the step's output is reproduced (Wan's blocks transform
    one stream; the text context does not change)."""
    lib = edb.lib()
    g = torch.Generator(device="cpu").manual_seed(9)
    model, fam, depth, width, rows, stream, tap_rows, step, lat = _wan(edb, cuda, g)
    a_in, a_b1 = (torch.zeros(rows, width, device=cuda) for _ in range(2))
    edb.check(lib.edb200_wan_set_anchor_capture(model.handle, edb.ANCHOR_MODEL_IN, edb.ptr(a_in)))
    edb.check(lib.edb200_wan_set_anchor_capture(model.handle, 1, edb.ptr(a_b1)))
    full = torch.empty_like(lat)
    launches = lib.edb200_launch_count()
    step(full)
    torch.cuda.synchronize()
    full_launches = lib.edb200_launch_count() - launches
    residual = torch.empty_like(a_in)
    edb.check(lib.edb200_sub_f32(edb.ptr(a_b1), edb.ptr(a_in), edb.ptr(residual), residual.numel(), edb.current_stream()))
    edb.check(lib.edb200_wan_set_anchor_capture(model.handle, 1, None))
    edb.check(lib.edb200_wan_set_region_inject(model.handle, 1, 2, edb.ptr(residual)))
    launches = lib.edb200_launch_count()
    reused = torch.empty_like(lat)
    step(reused)
    torch.cuda.synchronize()
    assert lib.edb200_launch_count() - launches < full_launches
    rel = float(torch.linalg.vector_norm(reused - full) / torch.linalg.vector_norm(full))
    # in + (out - in) differs from out in the last bit, and block 2 rounds its activations to f16 on top of that
    assert rel < 2e-3, rel
    # bad regions are refused; a region after block 0 needs the ModelIn buffer
    assert lib.edb200_wan_set_region_inject(model.handle, 2, 2, edb.ptr(residual)) != 0
    assert lib.edb200_wan_set_region_inject(model.handle, 0, depth + 1, edb.ptr(residual)) != 0
    edb.check(lib.edb200_wan_set_anchor_capture(model.handle, edb.ANCHOR_MODEL_IN, None))
    assert lib.edb200_wan_set_region_inject(model.handle, 1, 2, edb.ptr(residual)) != 0
    edb.check(lib.edb200_wan_set_region_inject(model.handle, -1, 0, None))
    again = torch.empty_like(lat)
    step(again)
    torch.cuda.synchronize()
    assert torch.equal(again, full)


def test_sd3_region_over_the_whole_stack_equals_the_stream_override(edb, cuda):
    """mmdit.hpp:3336-3343 with the region [0, depth): the same stream as the whole-stack override."""
    lib = edb.lib()
    g = torch.Generator(device="cpu").manual_seed(9)
    model, fam, depth, width, rows, stream, tap_rows, step, lat = _sd3(edb, cuda, g)
    residual = torch.randn(rows, width, generator=g).to(cuda)
    edb.check(lib.edb200_sd3_set_stream_override(model.handle, edb.ptr(residual)))
    a = torch.empty_like(lat)
    step(a)
    edb.check(lib.edb200_sd3_set_stream_override(model.handle, None))
    edb.check(lib.edb200_sd3_set_region_inject(model.handle, 0, depth, edb.ptr(residual)))
    b = torch.empty_like(lat)
    step(b)
    torch.cuda.synchronize()
    assert torch.isfinite(a).all() and torch.equal(a, b)
