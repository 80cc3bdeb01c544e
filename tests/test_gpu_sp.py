"""Sequence-parallel FLUX step on 2 (and 4) GPUs against the single-GPU step of the same
model: one process per GPU, both exchange paths of the library.  Skipped on a 1-GPU box."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, lib_dir, attention, lat_hw, n_txt, exchange, ret):
    import importlib.util
    os.environ["EDB200_SP_EXCHANGE"] = exchange
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)   # carries the NCCL id only
    spec = importlib.util.spec_from_file_location("edb200", os.path.join(lib_dir, "edb200.py"))
    edb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(edb)
    dev = torch.device("cuda", rank)
    model = edb.FluxModel(hidden_size=512, num_heads=4, depth=2, depth_single_blocks=2, mlp_hidden=1024,
                          in_channels=64, context_in_dim=64, vec_in_dim=32, axes_dim=(16, 56, 56),
                          attention=attention, sage_smooth_q=True)
    model.init_random(seed=7, std=0.05)
    g = torch.Generator(device="cpu").manual_seed(11)
    latent = torch.randn(16, lat_hw, lat_hw, generator=g).to(dev)
    ctx = torch.randn(n_txt, 64, generator=g).to(dev)
    y = torch.randn(32, generator=g).to(dev)
    ref = torch.empty_like(latent)
    model.prepare(lat_hw, lat_hw, n_txt)
    model.step(latent, 0.5, ctx, y, 3.5, ref)
    torch.cuda.synchronize()
    comm = edb.Comm()
    model.set_comm(comm)
    model.prepare(lat_hw, lat_hw, n_txt)
    out = torch.empty_like(latent)
    for _ in range(2):   # twice: the exchange buffers are reused
        out.fill_(float("nan"))
        model.step(latent, 0.5, ctx, y, 3.5, out)
        torch.cuda.synchronize()
    a, b = out.cpu().numpy(), ref.cpu().numpy()
    err = float(np.linalg.norm(a - b) / np.linalg.norm(b))
    ret[rank] = (bool(np.isfinite(a).all()), err)
    dist.barrier()
    model.set_comm(None)
    comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("attention,exchange", [("f16", "peer"), ("sage", "peer"), ("sage", "nccl")])
def test_flux_step_sequence_parallel_matches_single_gpu(edb, cuda, world, attention, exchange):
    """exchange = "peer": producers store into the owning rank's memory (CUDA IPC mappings) and a
    flag barrier orders them; "nccl": grouped ncclSend / ncclRecv plus one interleave kernel."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    lib_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "edge-dit.cpp_b200")
    port = _free_port()
    att = edb.ATTN_SAGE_INT8 if attention == "sage" else edb.ATTN_F16
    # 24 x 24 latent -> 144 image tokens + 16 text tokens = 160: rank 0 owns text and image rows
    procs = [ctx.Process(target=_worker, args=(r, world, port, lib_dir, att, 24, 16, exchange, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    for r in range(world):
        finite, err = ret[r]
        assert finite
        # same arithmetic per output element on every rank count; only the tile shapes differ
        assert err <= 1e-5, (r, err)


def _wan_worker(rank, world, port, lib_dir, exchange, ret):
    import importlib.util
    import torch.distributed as dist
    os.environ["EDB200_SP_EXCHANGE"] = exchange
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    spec = importlib.util.spec_from_file_location("edb200", os.path.join(lib_dir, "edb200.py"))
    edb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(edb)
    dev = torch.device("cuda", rank)
    model = edb.WanModel(dim=512, num_heads=4, ffn_dim=1024, num_layers=2, text_dim=128)
    model.init_random(seed=9, std=0.05)
    g = torch.Generator(device="cpu").manual_seed(12)
    latent = torch.randn(16, 2, 16, 20, generator=g).to(dev)     # 2 * 8 * 10 = 160 video tokens
    ctx = torch.randn(24, 128, generator=g).to(dev)
    ref = torch.empty_like(latent)
    model.prepare(2, 16, 20, 24)
    model.step(latent, 500.0, ctx, ref)
    torch.cuda.synchronize()
    comm = edb.Comm()
    model.set_comm(comm)
    model.prepare(2, 16, 20, 24)
    out = torch.empty_like(latent)
    for _ in range(2):
        out.fill_(float("nan"))
        model.step(latent, 500.0, ctx, out)
        torch.cuda.synchronize()
    a, b = out.cpu().numpy(), ref.cpu().numpy()
    ret[rank] = (bool(np.isfinite(a).all()), float(np.linalg.norm(a - b) / np.linalg.norm(b)))
    dist.barrier()
    model.set_comm(None)
    comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("exchange", ["peer", "nccl"])
def test_wan_step_sequence_parallel_matches_single_gpu(edb, cuda, world, exchange):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    lib_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "edge-dit.cpp_b200")
    port = _free_port()
    procs = [ctx.Process(target=_wan_worker, args=(r, world, port, lib_dir, exchange, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    for r in range(world):
        finite, err = ret[r]
        assert finite
        assert err <= 1e-5, (r, err)


def _cfg_worker(rank, world, port, lib_dir, ret):
    import importlib.util
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    spec = importlib.util.spec_from_file_location("edb200", os.path.join(lib_dir, "edb200.py"))
    edb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(edb)
    dev = torch.device("cuda", rank)
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
    ret[rank] = bool(torch.allclose(out, want, rtol=1e-6, atol=1e-5))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


def test_cfg_parallel_combine_on_two_gpus(edb, cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    lib_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "edge-dit.cpp_b200")
    port = _free_port()
    procs = [ctx.Process(target=_cfg_worker, args=(r, 2, port, lib_dir, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert ret[0] and ret[1]


def _qwen_worker(rank, world, port, lib_dir, exchange, ret):
    import importlib.util
    import torch.distributed as dist
    os.environ["EDB200_SP_EXCHANGE"] = exchange
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    spec = importlib.util.spec_from_file_location("edb200", os.path.join(lib_dir, "edb200.py"))
    edb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(edb)
    dev = torch.device("cuda", rank)
    model = edb.QwenModel(num_layers=2, num_heads=4, joint_attention_dim=256)
    model.init_random(seed=13, std=0.05)
    g = torch.Generator(device="cpu").manual_seed(14)
    latent = torch.randn(16, 24, 24, generator=g).to(dev)        # 144 image tokens + 16 text tokens = 160
    ctx = torch.randn(16, 256, generator=g).to(dev)
    ref = torch.empty_like(latent)
    model.prepare(24, 24, 16)
    model.step(latent, 500.0, ctx, ref)
    torch.cuda.synchronize()
    comm = edb.Comm()
    model.set_comm(comm)
    model.prepare(24, 24, 16)
    out = torch.empty_like(latent)
    for _ in range(2):
        out.fill_(float("nan"))
        model.step(latent, 500.0, ctx, out)
        torch.cuda.synchronize()
    a, b = out.cpu().numpy(), ref.cpu().numpy()
    ret[rank] = (bool(np.isfinite(a).all()), float(np.linalg.norm(a - b) / np.linalg.norm(b)))
    dist.barrier()
    model.set_comm(None)
    comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("exchange", ["peer", "nccl"])
def test_qwen_pass_sequence_parallel_matches_single_gpu(edb, cuda, world, exchange):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    lib_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "edge-dit.cpp_b200")
    port = _free_port()
    procs = [ctx.Process(target=_qwen_worker, args=(r, world, port, lib_dir, exchange, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    for r in range(world):
        finite, err = ret[r]
        assert finite
        assert err <= 1e-5, (r, err)
