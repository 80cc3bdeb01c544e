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
                                                   (48, 16, 4), (64, 0, 4), (64, 64, 2),
                                                   # sequences that do not divide: padded to a multiple of the world size
                                                   (7145, 256, 2), (7145, 256, 4), (7145, 256, 8), (1178, 154, 4),
                                                   (1178, 154, 8), (13, 5, 4), (9, 9, 8)])
def test_shard_covers_every_token_once(edb, n_tokens, n_txt, world):
    txt_seen, img_seen, rows_seen = 0, 0, 0
    t_slot = -(-n_tokens // world)
    for r in range(world):
        t_loc, txt_l, img_first, t_rows = edb.sp_shard(n_tokens, n_txt, r, world)
        assert t_loc == t_slot                      # every rank's slot of the padded sequence
        assert t_rows == max(0, min(t_slot, n_tokens - r * t_slot))   # only the last ranks own fewer rows
        assert 0 <= txt_l <= t_rows
        # text rows come first in the global order, so a rank's text rows continue where the last rank stopped
        assert txt_l == max(0, min(t_rows, n_txt - r * t_slot))
        assert img_first == img_seen
        txt_seen += txt_l
        img_seen += t_rows - txt_l
        rows_seen += t_rows
    assert txt_seen == n_txt and img_seen == n_tokens - n_txt and rows_seen == n_tokens
    assert world * t_slot - n_tokens < world         # the reference's padding rule: less than one row per rank


def test_shard_rejects_bad_arguments(edb):
    with pytest.raises(edb.EdbError):
        edb.sp_shard(4608, 512, 2, 2)
    with pytest.raises(edb.EdbError):
        edb.sp_shard(4608, 5000, 0, 2)
    with pytest.raises(edb.EdbError):
        edb.sp_shard(0, 0, 0, 1)


def test_map_decision_needs_every_rank(edb):
    """The rule both rendezvous of edb200_comm_map_peers apply to the gathered ok bytes: peers are
    mapped only if every rank reported success, so one rank's failed export or import turns into the
    same EDB200_ERR_UNSUPPORTED on all ranks."""
    import ctypes as C
    stride = 80
    for world in (1, 2, 8):
        buf = (C.c_ubyte * (stride * world))()
        for p in range(world):
            buf[p * stride] = 1
        assert edb.lib().edb200_comm_all_ok(buf, stride, world) == 1
        for bad in range(world):
            buf[bad * stride] = 0
            assert edb.lib().edb200_comm_all_ok(buf, stride, world) == 0
            buf[bad * stride] = 1
    assert edb.lib().edb200_comm_all_ok(None, stride, 2) == 0


def test_loopback_communicator_has_no_transport(edb):
    import ctypes as C
    h = C.c_void_p()
    edb.check(edb.lib().edb200_comm_create_loopback(0, 2, C.byref(h)))
    assert edb.lib().edb200_comm_rank(h) == 0 and edb.lib().edb200_comm_world(h) == 2
    assert edb.lib().edb200_comm_peers_mapped(h) == 0
    assert edb.lib().edb200_comm_set_timeout_ms(h, 0) == 1           # out of range
    edb.check(edb.lib().edb200_comm_set_timeout_ms(h, 20))
    assert edb.lib().edb200_sp_barrier(h, None) == 1                 # nothing mapped yet
    edb.lib().edb200_comm_destroy(h)
    assert edb.lib().edb200_comm_create_loopback(2, 2, C.byref(h)) == 1


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


def _padded_worker(rank, world, port, heads, n_tokens, d, lib_dir, ret):
    """The heads exchange of a sequence that does not divide by the world size: every rank sends its
    whole slot (t_loc rows, the last rank's tail rows are padding), and the receiving side reads only
    the n_tokens real rows of each head."""
    import importlib.util
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    spec = importlib.util.spec_from_file_location("edb200", os.path.join(lib_dir, "edb200.py"))
    edb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(edb)
    t_loc, _, _, t_rows = edb.sp_shard(n_tokens, 0, rank, world)
    hp, t_pad = heads // world, t_loc * world
    tok = torch.arange(rank * t_loc, (rank + 1) * t_loc, dtype=torch.float32)
    local = (tok[None, :, None] * 1e4 + torch.arange(heads, dtype=torch.float32)[:, None, None] * 1e2 +
             torch.arange(d, dtype=torch.float32)[None, None, :]).contiguous()
    local[:, t_rows:] = float("nan")                       # rows this rank does not own: padding
    out = torch.full((hp, t_pad, d), -1.0)
    sb, rb = local.view(torch.uint8).reshape(-1), out.view(torch.uint8).reshape(-1)
    ops = []
    for peer, so, ro, nb in edb.sp_heads_plan(rank, world, heads, t_loc, d * 4):
        if peer == rank:
            rb[ro:ro + nb] = sb[so:so + nb]
            continue
        ops.append(dist.P2POp(dist.isend, sb[so:so + nb], peer))
        ops.append(dist.P2POp(dist.irecv, rb[ro:ro + nb], peer))
    for w in dist.batch_isend_irecv(ops) if ops else []:
        w.wait()
    want = (torch.arange(n_tokens, dtype=torch.float32)[None, :, None] * 1e4 +
            torch.arange(rank * hp, (rank + 1) * hp, dtype=torch.float32)[:, None, None] * 1e2 +
            torch.arange(d, dtype=torch.float32)[None, None, :])
    ret[rank] = bool(torch.equal(out[:, :n_tokens], want)) and bool(torch.isnan(out[:, n_tokens:]).all())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,heads,n_tokens,d", [(2, 4, 11, 8), (4, 8, 13, 4)])
def test_padded_heads_exchange_by_gloo_ranks(world, heads, n_tokens, d):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    lib_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "edge-dit.cpp_b200")
    port = _free_port()
    procs = [ctx.Process(target=_padded_worker, args=(r, world, port, heads, n_tokens, d, lib_dir, ret))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world)), dict(ret)


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
