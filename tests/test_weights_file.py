"""CPU tier: the pre-quantised weight file round-trips and shards by rows without reading the rest."""
import numpy as np
import pytest
import torch

import avelang_b200 as ave
from avelang_b200 import weights


def _operand(rows, k, fmt, seed=0):
    g = torch.Generator().manual_seed(seed)
    blk = 16 if fmt == ave.NVFP4 else 32
    packed = torch.randint(0, 256, (rows, k // 2), generator=g, dtype=torch.uint8)
    scales = torch.randint(1, 120, (rows, k // blk), generator=g, dtype=torch.uint8)
    gs = torch.tensor([0.0123], dtype=torch.float32) if fmt == ave.NVFP4 else None
    return ave.make_operand(packed, scales, gs, fmt)


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
def test_round_trip_and_shards(tmp_path, fmt):
    op = _operand(1024, 256, fmt)
    path = str(tmp_path / "w.avefp4")
    weights.save_fp4_weights(path, op)
    h = weights.read_header(path)
    assert h["rows"] == 1024 and h["k"] == 256 and h["packed_offset"] % 64 == 0 and h["scales_offset"] % 64 == 0
    full = weights.load_fp4_weights(path)
    assert torch.equal(full.packed, op.packed) and torch.equal(full.scales, op.scales)
    if fmt == ave.NVFP4:
        assert np.float32(full.global_scale.item()) == np.float32(0.0123)
    else:
        assert full.global_scale is None
    for world in (2, 4, 8):
        parts = [weights.load_fp4_weights(path, world=world, rank=r) for r in range(world)]
        assert all(p.rows == 1024 // world for p in parts)
        assert torch.equal(torch.cat([p.packed for p in parts]), op.packed)
        assert torch.equal(torch.cat([p.scales for p in parts]), op.scales)
        if fmt == ave.NVFP4:
            assert all(np.float32(p.global_scale.item()) == np.float32(0.0123) for p in parts)


def test_rejects_bad_files(tmp_path):
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"not a weight file at all")
    with pytest.raises(ValueError, match="AVEFP4W1"):
        weights.read_header(str(bad))
    op = _operand(256, 64, ave.NVFP4)
    path = str(tmp_path / "w.avefp4")
    weights.save_fp4_weights(path, op)
    data = open(path, "rb").read()
    (tmp_path / "short.avefp4").write_bytes(data[:-100])
    with pytest.raises(ValueError, match="truncated"):
        weights.load_fp4_weights(str(tmp_path / "short.avefp4"))
    with pytest.raises(ValueError, match="multiple of"):
        weights.load_fp4_weights(path, world=3, rank=0)


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
def test_k_shards(tmp_path, fmt):
    """shard="k": every rank reads its K-slice of every row (the row-parallel layer); the slices put side by side are
    the whole operand, and the oracle's product of the whole equals the sum of the products of the slices."""
    from oracle import fp4_oracle as O

    rows, k = 96, 2048
    op = _operand(rows, k, fmt, seed=3)
    path = str(tmp_path / "w.avefp4")
    weights.save_fp4_weights(path, op)
    assert weights.load_fp4_weights(path, shard="k").k == k
    for world in (2, 4, 8):
        parts = [weights.load_fp4_weights(path, world=world, rank=r, shard="k") for r in range(world)]
        assert all(p.rows == rows and p.k == k // world for p in parts)
        assert torch.equal(torch.cat([p.packed for p in parts], dim=1), op.packed)
        assert torch.equal(torch.cat([p.scales for p in parts], dim=1), op.scales)
    # arithmetic: x (8, k) against the K-sharded weight
    x = _operand(8, k, fmt, seed=4)
    gs = lambda o: 1.0 if o.global_scale is None else float(o.global_scale.item())
    full, _ = O.c_gemm_fp4((x.packed.numpy(), x.scales.numpy(), gs(x)), (op.packed.numpy(), op.scales.numpy(), gs(op)), fmt)
    parts = [weights.load_fp4_weights(path, world=4, rank=r, shard="k") for r in range(4)]
    blk = 16 if fmt == ave.NVFP4 else 32
    acc = np.zeros_like(full, dtype=np.float64)
    for r, w in enumerate(parts):
        lo, hi = r * k // 4, (r + 1) * k // 4
        xs = (x.packed.numpy()[:, lo // 2:hi // 2], x.scales.numpy()[:, lo // blk:hi // blk], gs(x))
        part, _ = O.c_gemm_fp4(xs, (w.packed.numpy(), w.scales.numpy(), gs(w)), fmt)
        acc += part
    assert np.linalg.norm(acc - full) / np.linalg.norm(full) < 1e-6
    with pytest.raises(ValueError, match="shard must be"):
        weights.load_fp4_weights(path, shard="m")
