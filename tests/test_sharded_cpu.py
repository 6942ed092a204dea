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


def test_k_shard_bounds_and_slab_offsets():
    assert sharded.k_shard_bounds(8192, 8, 3) == (3072, 4096)
    spans = [sharded.k_shard_bounds(8192, 4, r) for r in range(4)]
    assert spans[0][0] == 0 and spans[-1][1] == 8192 and all(spans[i][1] == spans[i + 1][0] for i in range(3))
    with pytest.raises(ValueError):
        sharded.k_shard_bounds(1000, 4, 0)
    # rank 2 of 4 writes slab 2 of every (4, rows, n) fp32 staging buffer
    assert sharded.slab_offsets(4, 2, 64, 1024) == [2 * 64 * 1024 * 4] * 4
    with pytest.raises(ValueError):
        sharded.slab_offsets(4, 4, 64, 1024)


def _k_worker(rank, world, port, ret):
    """The K-sharded layer's arithmetic on two gloo ranks, with the oracle as the per-rank GEMM: every rank's fp32
    partial (its K-slice, its own tensor scales) is placed in the owner's slab, slabs are summed in rank order."""
    import numpy as np

    from oracle import fp4_oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k = 64, 48, 512
        g = torch.Generator().manual_seed(3)
        a = torch.randn((m, k), generator=g).to(torch.bfloat16)
        w = (torch.randn((n, k), generator=g) * 0.02).to(torch.bfloat16)
        bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)
        lo, hi = sharded.k_shard_bounds(k, world, rank)
        qa, qw = O.c_quantize(bits(a[:, lo:hi]), O.NVFP4), O.c_quantize(bits(w[:, lo:hi]), O.NVFP4)
        part, _ = O.c_gemm_fp4(qa, qw, O.NVFP4)                       # (m, n) fp32, this rank's K-slice
        rows = m // world
        staging = [torch.zeros((world, rows, n)) for _ in range(world)]   # staging[j] lives on rank j
        # "peer stores": all-gather the partials, then every rank fills its own staging buffer from them
        parts = [torch.zeros((m, n)) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(part))
        mine = torch.stack([parts[r][rank * rows:(rank + 1) * rows] for r in range(world)])   # (world, rows, n)
        total = torch.zeros((rows, n))
        for r in range(world):
            total += mine[r]
        got = total.to(torch.bfloat16)
        # the unsharded oracle on per-shard-quantised operands: dequantise each K-slice, one fp32 matmul
        deq_a = np.concatenate([O.c_dequantize(*O.c_quantize(bits(a[:, s:e]), O.NVFP4), O.NVFP4)
                                for s, e in (sharded.k_shard_bounds(k, world, r) for r in range(world))], axis=1)
        deq_w = np.concatenate([O.c_dequantize(*O.c_quantize(bits(w[:, s:e]), O.NVFP4), O.NVFP4)
                                for s, e in (sharded.k_shard_bounds(k, world, r) for r in range(world))], axis=1)
        full = torch.from_numpy(deq_a) @ torch.from_numpy(deq_w).T
        exp = full[rank * rows:(rank + 1) * rows].to(torch.bfloat16)
        rel = float((got.float() - exp.float()).norm() / exp.float().norm())
        ret[rank] = rel < 1e-3
    finally:
        dist.destroy_process_group()


def test_k_sharded_reduce_scatter_math_two_ranks():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_k_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert ret[0] and ret[1]


def test_quantized_gather_layout_and_peer_order():
    """Host-side bookkeeping of the quantised all-gather: where each rank's column block sits in the gathered operand,
    how the symmetric buffer is laid out, and in which order a rank stores to its peers (no GPU needed)."""
    from avelang_b200 import fp4_gemm

    for world in (1, 2, 4, 8):
        seen_first = set()
        for rank in range(world):
            order = sharded.peer_order(rank, world)
            assert sorted(order + [rank]) == list(range(world))          # every other rank exactly once
            if world > 1:
                assert order[0] == (rank + 1) % world
                seen_first.add(order[0])
        if world > 1:
            assert len(seen_first) == world                                # the ranks start with different destinations
    lay = sharded.quantized_gather_layout(8192, 7168, 8, 3, fp4_gemm.NVFP4)
    assert lay["n_total"] == 57344 and lay["col0"] == 3 * 7168
    assert lay["packed_bytes"] == 8192 * 57344 // 2 and lay["scales_offset"] % 256 == 0
    assert lay["scales_bytes"] == fp4_gemm.sf_bytes(8192, 57344, fp4_gemm.NVFP4, fp4_gemm.SF_TILED) == 64 * 896 * 512
    assert lay["total_bytes"] == lay["scales_offset"] + lay["scales_bytes"]
    mx = sharded.quantized_gather_layout(300, 320, 4, 1, fp4_gemm.MXFP4)
    assert mx["col0"] == 320 and mx["scales_bytes"] == 3 * 10 * 512 and mx["scales_offset"] == (300 * 640 + 255) // 256 * 256
    with pytest.raises(ValueError, match="multiple of 64"):
        sharded.quantized_gather_layout(128, 96, 2, 0, fp4_gemm.NVFP4)
    with pytest.raises(ValueError, match="bad rank"):
        sharded.peer_order(2, 2)
