"""Host logic of the sequence-parallel path, without a GPU: token sharding, the message
list of the heads exchange, and that list executed by world_size-2 and -4 gloo ranks on CPU
tensors (the NCCL path on the GPU executes the very same list)."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("n_tokens,n_txt,world", [(4608, 512, 1), (4608, 512, 2), (4608, 512, 8), (16896, 512, 8),
                                                   (48, 16, 4), (64, 0, 4), (64, 64, 2)])
def test_shard_covers_every_token_once(edb, n_tokens, n_txt, world):
    txt_seen, img_seen = 0, 0
    for r in range(world):
        t_loc, txt_l, img_first = edb.sp_shard(n_tokens, n_txt, r, world)
        assert t_loc == n_tokens // world
        assert 0 <= txt_l <= t_loc
        # text rows come first in the global order, so a rank's text rows continue where the last rank stopped
        assert txt_l == max(0, min(t_loc, n_txt - r * t_loc))
        assert img_first == img_seen
        txt_seen += txt_l
        img_seen += t_loc - txt_l
    assert txt_seen == n_txt and img_seen == n_tokens - n_txt


def test_shard_rejects_ragged_split(edb):
    with pytest.raises(edb.EdbError):
        edb.sp_shard(4609, 512, 0, 2)
    with pytest.raises(edb.EdbError):
        edb.sp_shard(4608, 512, 2, 2)


@pytest.mark.parametrize("world,heads,t_loc,row", [(2, 4, 3, 8), (4, 8, 5, 16), (8, 24, 576, 256)])
def test_heads_plan_is_a_permutation(edb, world, heads, t_loc, row):
    hp = heads // world
    size = heads * t_loc * row  # bytes per rank, before and after
    for r in range(world):
        plan = edb.sp_heads_plan(r, world, heads, t_loc, row)
        assert len(plan) == world * hp
        send = sorted((so, nb) for _, so, _, nb in plan)
        recv = sorted((ro, nb) for _, _, ro, nb in plan)
        for spans in (send, recv):  # both sides tile the buffer exactly
            pos = 0
            for off, nb in spans:
                assert off == pos
                pos += nb
            assert pos == size
    assert edb.lib().edb200_sp_heads_plan(0, 3, 8, 4, 16, None, None, None, None, 0) == -1


def _worker(rank, world, port, heads, t_loc, d, lib_dir, ret):
    import importlib.util
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    spec = importlib.util.spec_from_file_location("edb200", os.path.join(lib_dir, "edb200.py"))
    edb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(edb)
    hp, T = heads // world, t_loc * world
    # value = global token * 1e4 + head * 1e2 + channel, exact in f32
    tok = torch.arange(rank * t_loc, (rank + 1) * t_loc, dtype=torch.float32)
    local = (tok[None, :, None] * 1e4 + torch.arange(heads, dtype=torch.float32)[:, None, None] * 1e2 +
             torch.arange(d, dtype=torch.float32)[None, None, :]).contiguous()
    out = torch.full((hp, T, d), -1.0)
    sb = local.view(torch.uint8).reshape(-1)
    rb = out.view(torch.uint8).reshape(-1)
    ops, self_copies = [], []
    for peer, so, ro, nb in edb.sp_heads_plan(rank, world, heads, t_loc, d * 4):
        if peer == rank:
            self_copies.append((so, ro, nb))
            continue
        ops.append(dist.P2POp(dist.isend, sb[so:so + nb], peer))
        ops.append(dist.P2POp(dist.irecv, rb[ro:ro + nb], peer))
    # gloo matches messages between a pair of ranks in order: both sides walk the plan head by head
    for so, ro, nb in self_copies:
        rb[ro:ro + nb] = sb[so:so + nb]
    for w in dist.batch_isend_irecv(ops) if ops else []:
        w.wait()
    want = (torch.arange(T, dtype=torch.float32)[None, :, None] * 1e4 +
            torch.arange(rank * hp, (rank + 1) * hp, dtype=torch.float32)[:, None, None] * 1e2 +
            torch.arange(d, dtype=torch.float32)[None, None, :])
    ret[rank] = bool(torch.equal(out, want))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,heads,t_loc,d", [(2, 4, 6, 8), (4, 8, 3, 4)])
def test_heads_plan_executed_by_gloo_ranks(world, heads, t_loc, d):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    lib_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "edge-dit.cpp_b200")
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, heads, t_loc, d, lib_dir, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world)), dict(ret)
