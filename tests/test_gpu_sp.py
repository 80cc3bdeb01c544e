"""Sequence-parallel and CFG-parallel execution on 2 (and 4) GPUs against the single-GPU step of
the same model: one process per GPU, both exchange paths of the library, token counts that divide
by the world size and token counts that need padding.  The multi-GPU tests are skipped on a 1-GPU
box; the barrier's time-out test needs one GPU only."""
import ctypes as C
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

LIB_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "edge-dit.cpp_b200")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _setup(rank, world, port, env):
    """Common start of every worker: environment, device, a gloo group (it only carries the NCCL id)."""
    import importlib.util
    for k, v in env.items():
        os.environ[k] = v
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    spec = importlib.util.spec_from_file_location("edb200", os.path.join(LIB_DIR, "edb200.py"))
    edb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(edb)
    return edb, dist, torch.device("cuda", rank)


def _spawn(world, target, args):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port) + tuple(args) + (ret,)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    return ret


def _sp_versus_single(edb, dist, model, prepare, step, out_like, graph):
    """Runs `step` on one GPU, then sequence parallel over all ranks (twice eagerly: the exchange buffers
    are reused; then, if asked, recorded once into a CUDA graph and replayed twice).  Returns
    (finite, relative error of the eager run, replay equals eager, peer mappings in use)."""
    ref = torch.empty_like(out_like)
    prepare()
    step(ref)
    torch.cuda.synchronize()
    comm = edb.Comm()
    model.set_comm(comm)
    prepare()
    mapped = bool(edb.lib().edb200_comm_peers_mapped(comm.handle))
    out = torch.empty_like(out_like)
    for _ in range(2):
        out.fill_(float("nan"))
        step(out)
        torch.cuda.synchronize()
    edb.poll_status()
    a, b = out.cpu().numpy(), ref.cpu().numpy()
    err = float(np.linalg.norm(a - b) / np.linalg.norm(b))
    same = True
    if graph and mapped:
        side = torch.cuda.Stream()
        replay = torch.empty_like(out_like)
        with torch.cuda.stream(side):
            step(replay)
            side.synchronize()
            dist.barrier()
            g = edb.Graph(lambda: step(replay))
            for _ in range(2):
                replay.fill_(float("nan"))
                g.launch()
                side.synchronize()
            edb.poll_status()
        # the out-projections of a sequence-parallel rank add their k-parts with unordered atomics,
        # so a replay equals an eager run up to the last bits only
        r = replay.cpu().numpy()
        same = bool(np.isfinite(r).all()) and float(np.linalg.norm(r - a) / np.linalg.norm(a)) <= 1e-5
    dist.barrier()
    model.set_comm(None)
    comm.close()
    return bool(np.isfinite(a).all()), err, same, mapped


def _flux_worker(rank, world, port, attention, n_txt, exchange, env, ret):
    edb, dist, dev = _setup(rank, world, port, dict(env, EDB200_SP_EXCHANGE=exchange))
    model = edb.FluxModel(hidden_size=512, num_heads=4, depth=2, depth_single_blocks=2, mlp_hidden=1024,
                          in_channels=64, context_in_dim=64, vec_in_dim=32, axes_dim=(16, 56, 56),
                          attention=attention, sage_smooth_q=True)
    model.init_random(seed=7, std=0.05)
    g = torch.Generator(device="cpu").manual_seed(11)
    latent = torch.randn(16, 24, 24, generator=g).to(dev)       # 144 image tokens
    ctx = torch.randn(n_txt, 64, generator=g).to(dev)
    y = torch.randn(32, generator=g).to(dev)
    ret[rank] = _sp_versus_single(edb, dist, model, lambda: model.prepare(24, 24, n_txt),
                                  lambda o: model.step(latent, 0.5, ctx, y, 3.5, o), latent, graph=True)
    dist.destroy_process_group()


def _check(ret, world, want_mapped=None):
    for r in range(world):
        finite, err, same, mapped = ret[r]
        assert finite
        # same arithmetic per output element on every rank count; only the tile shapes differ
        assert err <= 1e-5, (r, err)
        assert same, r
        if want_mapped is not None:
            assert mapped == want_mapped, r


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("n_txt", [16, 17], ids=["divides", "padded"])
@pytest.mark.parametrize("attention,exchange", [("f16", "peer"), ("sage", "peer"), ("sage", "nccl")])
def test_flux_step_sequence_parallel_matches_single_gpu(edb, cuda, world, n_txt, attention, exchange):
    """exchange = "peer": producers store into the owning rank's memory (CUDA IPC mappings) and a
    flag barrier orders them; "nccl": grouped ncclSend / ncclRecv plus one interleave kernel.
    n_txt = 17 makes 161 tokens: the sequence is padded to a multiple of the world size and the last
    rank owns fewer rows (sp_sequence_padding, src/core/parallel/sp_parallel.cpp:757-768)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    att = edb.ATTN_SAGE_INT8 if attention == "sage" else edb.ATTN_F16
    ret = _spawn(world, _flux_worker, (att, n_txt, exchange, {}))
    _check(ret, world, want_mapped=exchange == "peer")


def test_failed_peer_mapping_on_one_rank_falls_back_everywhere(edb, cuda):
    """A handle export that fails on rank 1 only (injected on the host): both ranks come out of the
    collective mapping call with "unsupported", both run the NCCL exchanges, nobody waits for a peer
    that took the other path, and the result is still the single-GPU one."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ret = _spawn(2, _flux_worker, (edb.ATTN_F16, 16, "peer", {"EDB200_TEST_FAIL_IPC_RANK": "1"}))
    _check(ret, 2, want_mapped=False)


def _wan_worker(rank, world, port, lat, exchange, ret):
    edb, dist, dev = _setup(rank, world, port, {"EDB200_SP_EXCHANGE": exchange})
    model = edb.WanModel(dim=512, num_heads=4, ffn_dim=1024, num_layers=5, text_dim=128)   # INT8 scores on layer 2 only
    model.init_random(seed=9, std=0.05)
    g = torch.Generator(device="cpu").manual_seed(12)
    latent = torch.randn(16, *lat, generator=g).to(dev)
    ctx = torch.randn(24, 128, generator=g).to(dev)
    ret[rank] = _sp_versus_single(edb, dist, model, lambda: model.prepare(*lat, 24),
                                  lambda o: model.step(latent, 500.0, ctx, o), latent, graph=True)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("lat", [(2, 16, 20), (3, 14, 18)], ids=["160_tokens", "189_tokens_padded"])
@pytest.mark.parametrize("exchange", ["peer", "nccl"])
def test_wan_step_sequence_parallel_matches_single_gpu(edb, cuda, world, lat, exchange):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _check(_spawn(world, _wan_worker, (lat, exchange)), world)


def _qwen_worker(rank, world, port, n_txt, exchange, ret):
    edb, dist, dev = _setup(rank, world, port, {"EDB200_SP_EXCHANGE": exchange})
    model = edb.QwenModel(num_layers=2, num_heads=4, joint_attention_dim=256)
    model.init_random(seed=13, std=0.05)
    g = torch.Generator(device="cpu").manual_seed(14)
    latent = torch.randn(16, 24, 24, generator=g).to(dev)        # 144 image tokens
    ctx = torch.randn(n_txt, 256, generator=g).to(dev)
    ret[rank] = _sp_versus_single(edb, dist, model, lambda: model.prepare(24, 24, n_txt),
                                  lambda o: model.step(latent, 500.0, ctx, o), latent, graph=False)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("n_txt", [16, 19], ids=["divides", "padded"])
@pytest.mark.parametrize("exchange", ["peer", "nccl"])
def test_qwen_pass_sequence_parallel_matches_single_gpu(edb, cuda, world, n_txt, exchange):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _check(_spawn(world, _qwen_worker, (n_txt, exchange)), world)


def _sd3_worker(rank, world, port, attention, exchange, ret):
    edb, dist, dev = _setup(rank, world, port, {"EDB200_SP_EXCHANGE": exchange})
    model = edb.SD3Model(hidden_size=512, num_heads=8, depth=6, adm_in_channels=64, context_size=128, pos_embed_max_size=16,
                         attention=attention)                  # INT8 scores (when asked for) on blocks 2 and 3
    model.init_random(seed=4, std=0.05)
    g = torch.Generator(device="cpu").manual_seed(21)
    latent = torch.randn(16, 16, 24, generator=g).to(dev)        # 96 image tokens + 11 context tokens = 107: padded
    ctx = torch.randn(11, 128, generator=g).to(dev)
    y = torch.randn(64, generator=g).to(dev)
    ret[rank] = _sp_versus_single(edb, dist, model, lambda: model.prepare(16, 24, 11),
                                  lambda o: model.step(latent, 500.0, ctx, y, o), latent, graph=False)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("attention,exchange", [("f16", "peer"), ("sage", "peer"), ("f16", "nccl")])
def test_sd3_pass_sequence_parallel_matches_single_gpu(edb, cuda, world, attention, exchange):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    att = edb.ATTN_SAGE_INT8 if attention == "sage" else edb.ATTN_F16
    _check(_spawn(world, _sd3_worker, (att, exchange)), world)


def _cfg_worker(rank, world, port, ret):
    edb, dist, dev = _setup(rank, world, port, {})
    model = edb.SD3Model(hidden_size=512, num_heads=8, depth=2, adm_in_channels=64, context_size=128, pos_embed_max_size=16)
    model.init_random(seed=4, std=0.05)
    g = torch.Generator(device="cpu").manual_seed(21)
    latent = torch.randn(16, 16, 24, generator=g).to(dev)
    ctx_c, ctx_u = torch.randn(11, 128, generator=g).to(dev), torch.zeros(11, 128, device=dev)
    y_c, y_u = torch.randn(64, generator=g).to(dev), torch.zeros(64, device=dev)
    model.prepare(16, 24, 11)
    cond, uncond = torch.empty_like(latent), torch.empty_like(latent)
    model.step(latent, 500.0, ctx_c, y_c, cond)
    model.step(latent, 500.0, ctx_u, y_u, uncond)
    want = uncond + 4.0 * (cond - uncond)          # both passes on one GPU
    comm = edb.Comm()
    mine = cond if rank == 0 else uncond            # CFG parallel: one pass per rank
    gathered = torch.empty(2, latent.numel(), device=dev)
    out = torch.empty_like(latent)
    edb.check(edb.lib().edb200_cfg_parallel_combine(comm.handle, edb.ptr(mine), 4.0, edb.ptr(gathered), edb.ptr(out),
                                                    latent.numel(), edb.current_stream()))
    torch.cuda.synchronize()
    ok = bool(torch.allclose(out, want, rtol=1e-6, atol=1e-5))
    # Qwen-Image's norm-preserving form of the same step
    want2, out2 = torch.empty_like(latent), torch.empty_like(latent)
    edb.check(edb.lib().edb200_cfg_combine_rescaled(edb.ptr(uncond), edb.ptr(cond), 4.0, 2, 16, 16, 24, edb.ptr(want2),
                                                    edb.current_stream()))
    edb.check(edb.lib().edb200_cfg_parallel_combine_rescaled(comm.handle, edb.ptr(mine), 4.0, 2, 16, 16, 24,
                                                             edb.ptr(gathered), edb.ptr(out2), edb.current_stream()))
    torch.cuda.synchronize()
    ret[rank] = ok and bool(torch.equal(out2, want2))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


def test_cfg_parallel_combine_on_two_gpus(edb, cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ret = _spawn(2, _cfg_worker, ())
    assert ret[0] and ret[1]


def _cfg_sp_worker(rank, world, port, ret):
    """CFG-parallel x sequence-parallel: the world is two branches (conditional: ranks 0 .. P-1,
    unconditional: ranks P .. 2P-1), each branch runs its pass sequence parallel over its own
    communicator, and rank i pairs with rank i + P for the guidance combine."""
    edb, dist, dev = _setup(rank, world, port, {})
    sp = world // 2
    branch, r_sp = rank // sp, rank % sp
    model = edb.QwenModel(num_layers=2, num_heads=4, joint_attention_dim=256, attention=edb.ATTN_F16)
    model.init_random(seed=13, std=0.05)
    g = torch.Generator(device="cpu").manual_seed(14)
    latent = torch.randn(16, 24, 24, generator=g).to(dev)
    ctx_c, ctx_u = torch.randn(19, 256, generator=g).to(dev), torch.zeros(19, 256, device=dev)   # 163 tokens: padded
    model.prepare(24, 24, 19)
    cond, uncond, want = (torch.empty_like(latent) for _ in range(3))
    model.step(latent, 500.0, ctx_c, cond)
    model.step(latent, 500.0, ctx_u, uncond)
    edb.check(edb.lib().edb200_cfg_combine_rescaled(edb.ptr(uncond), edb.ptr(cond), 4.0, 2, 16, 24, 24, edb.ptr(want),
                                                    edb.current_stream()))
    torch.cuda.synchronize()
    branch_comm = edb.Comm(ranks=list(range(branch * sp, (branch + 1) * sp)))
    pair_comm = edb.Comm(ranks=[r_sp, r_sp + sp])
    if sp > 1:
        model.set_comm(branch_comm)
        model.prepare(24, 24, 19)
    mine = torch.empty_like(latent)
    model.step(latent, 500.0, ctx_c if branch == 0 else ctx_u, mine)
    gathered = torch.empty(2, latent.numel(), device=dev)
    out = torch.empty_like(latent)
    edb.check(edb.lib().edb200_cfg_parallel_combine_rescaled(pair_comm.handle, edb.ptr(mine), 4.0, 2, 16, 24, 24,
                                                             edb.ptr(gathered), edb.ptr(out), edb.current_stream()))
    torch.cuda.synchronize()
    a, b = out.cpu().numpy(), want.cpu().numpy()
    ret[rank] = (bool(np.isfinite(a).all()), float(np.linalg.norm(a - b) / np.linalg.norm(b)), True, True)
    dist.barrier()
    if sp > 1:
        model.set_comm(None)
    pair_comm.close()
    branch_comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_cfg_parallel_times_sequence_parallel(edb, cuda, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _check(_spawn(world, _cfg_sp_worker, ()), world)


def test_barrier_gives_up_and_reports_timeout(edb, cuda):
    """The cross-GPU barrier's device-side wait is bounded.  A 2-rank loopback communicator on this
    one GPU (both "ranks" are this allocation) is given a 20 ms limit; nobody ever posts rank 1's
    flag, so the kernel's wait runs out, the kernel returns, and the status poll reports the
    time-out once.  Nothing hangs and the context stays usable."""
    lib = edb.lib()
    h = C.c_void_p()
    edb.check(lib.edb200_comm_create_loopback(0, 2, C.byref(h)))
    buf = torch.zeros(4096, dtype=torch.uint8, device=cuda)
    edb.check(lib.edb200_comm_map_peers(h, edb.ptr(buf), buf.numel(), 1024, edb.current_stream()))
    assert lib.edb200_comm_peers_mapped(h) == 1
    edb.check(lib.edb200_comm_set_timeout_ms(h, 20))
    edb.poll_status()                                        # clean before
    edb.check(lib.edb200_sp_barrier(h, edb.current_stream()))
    with pytest.raises(edb.EdbError) as ei:
        edb.poll_status()
    assert ei.value.status == 4                              # EDB200_ERR_TIMEOUT
    edb.poll_status()                                        # reported once, then clear again
    # a world of one completes at once: the same kernel, nobody to wait for
    h1 = C.c_void_p()
    edb.check(lib.edb200_comm_create_loopback(0, 1, C.byref(h1)))
    edb.check(lib.edb200_comm_map_peers(h1, edb.ptr(buf), buf.numel(), 2048, edb.current_stream()))
    for _ in range(3):
        edb.check(lib.edb200_sp_barrier(h1, edb.current_stream()))
    edb.poll_status()
    assert int(buf[2048 + 512: 2048 + 516].view(torch.int32).item()) == 3      # the epoch counter on the device
    x = torch.ones(8, device=cuda)
    assert float(x.sum().item()) == 8.0
    edb.check(lib.edb200_comm_unmap_peers(h))
    edb.check(lib.edb200_comm_unmap_peers(h1))
    lib.edb200_comm_destroy(h)
    lib.edb200_comm_destroy(h1)
