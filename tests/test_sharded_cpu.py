"""CPU tier: the N-sharding bookkeeping and the gather layout on two gloo ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from avelang_b200 import sharded


def test_shard_bounds():
    assert sharded.shard_bounds(57344, 8, 0) == (0, 7168)
    assert sharded.shard_bounds(57344, 8, 7) == (50176, 57344)
    for w in (1, 2, 4, 8):
        spans = [sharded.shard_bounds(57344, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == 57344
        assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
        assert all((hi - lo) % 256 == 0 for lo, hi in spans)
    with pytest.raises(ValueError):
        sharded.shard_bounds(1000, 8, 0)
    with pytest.raises(ValueError):
        sharded.shard_bounds(1024, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k = 8, 512, 64
        g = torch.Generator().manual_seed(0)
        a = torch.randn((m, k), generator=g)
        w = torch.randn((n, k), generator=g)
        full = (a @ w.T).to(torch.bfloat16)
        mine = sharded.shard_rows(w, world, rank)
        local = (a @ mine.T).to(torch.bfloat16)
        gathered = sharded.all_gather_columns(local)
        assert gathered.shape == (world, m, n // world)
        logical = sharded.columns_view(gathered).reshape(m, n)
        ok = torch.equal(logical, full)
        # in-place form used by ShardedFp4Linear.forward: the local slab is a view of the output
        buf = torch.zeros((world, m, n // world), dtype=torch.bfloat16)
        buf[rank].copy_(local)
        dist.all_gather_into_tensor(buf.view(-1, n // world), buf[rank])
        ok = ok and torch.equal(buf, gathered)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_gather_layout_two_ranks():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret[0] and ret[1]
