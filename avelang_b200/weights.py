"""On-disk format for pre-quantised FP4 weights, and a loader that shards by output rows (N) or by K.

Weights are quantised once, offline; serving loads the bytes and never touches bf16 again.  The file
holds the operand in its layout-neutral form -- packed nibbles (N, K/2), row-major scale bytes
(N, K/blk) and the fp32 tensor scale (NVFP4) -- so any shard [lo, hi) of the rows is a contiguous
byte range of each section and can be read without touching the rest.  The loader converts the
scales of its shard to the 128x4 tiled layout on the device (and can re-pack the nibbles into 16 KB
tiles for the decode kernel).

File layout (little endian):
    bytes 0..7    magic  b"AVEFP4W1"
    bytes 8..15   header length H (uint64)
    H bytes       JSON header: {"fmt": "nvfp4"|"mxfp4", "rows": N, "k": K, "block": 16|32,
                                "global_scale": float | null, "packed_offset": .., "scales_offset": ..}
    packed        N * K/2 bytes at packed_offset (64-byte aligned)
    scales        N * K/block bytes at scales_offset (64-byte aligned)

The reference keeps no weight format of its own (operands are plain bf16 tensors,
python/avelang_kernels/amdgpu_gemm.py:458-494); this is the offline half of the decode path.
"""
from __future__ import annotations

import json
import struct

import numpy as np
import torch

from .fp4_gemm import MXFP4, NVFP4, SF_ROW_MAJOR, Fp4Operand, make_operand, pack_weight_tiles, to_tiled
from .sharded import k_shard_bounds, shard_bounds

MAGIC = b"AVEFP4W1"
_ALIGN = 64


def _align(x: int) -> int:
    return (x + _ALIGN - 1) // _ALIGN * _ALIGN


def save_fp4_weights(path: str, op: Fp4Operand) -> None:
    """Write a quantised operand (row-major scales, row-major nibbles) to `path`."""
    if op.sf_layout != SF_ROW_MAJOR or op.tile_major:
        raise ValueError("save_fp4_weights needs the layout-neutral form: row-major scales, row-major nibbles "
                         "(quantise with sf_layout=SF_ROW_MAJOR).")
    block = 16 if op.fmt == NVFP4 else 32
    packed = op.packed.detach().cpu().contiguous().numpy()
    scales = op.scales.detach().cpu().contiguous().numpy()
    if packed.shape != (op.rows, op.k // 2) or scales.shape != (op.rows, op.k // block):
        raise ValueError("operand tensors do not match its declared shape.")
    header = {"fmt": "nvfp4" if op.fmt == NVFP4 else "mxfp4", "rows": op.rows, "k": op.k, "block": block,
              "global_scale": None if op.global_scale is None else float(op.global_scale.detach().cpu().reshape(-1)[0].item())}
    # offsets depend on the header length, which depends on the offsets' digits: fix the length first
    header["packed_offset"] = 0
    header["scales_offset"] = 0
    hlen = len(json.dumps(header)) + 40
    header["packed_offset"] = _align(16 + hlen)
    header["scales_offset"] = _align(header["packed_offset"] + packed.nbytes)
    blob = json.dumps(header).encode().ljust(hlen, b" ")
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<Q", hlen))
        f.write(blob)
        f.write(b"\0" * (header["packed_offset"] - f.tell()))
        f.write(packed.tobytes())
        f.write(b"\0" * (header["scales_offset"] - f.tell()))
        f.write(scales.tobytes())


def read_header(path: str) -> dict:
    with open(path, "rb") as f:
        if f.read(8) != MAGIC:
            raise ValueError(f"{path} is not an AVEFP4W1 weight file.")
        (hlen,) = struct.unpack("<Q", f.read(8))
        return json.loads(f.read(hlen).decode())


def load_fp4_weights(path: str, device: torch.device | str = "cpu", world: int = 1, rank: int = 0,
                     tile_major: bool = False, shard: str = "n") -> Fp4Operand:
    """Read this rank's shard of the weight (the whole matrix for world = 1).

    shard="n": rows [lo, hi) -- the column-parallel layer (`ShardedFp4Linear`); only the shard's bytes are read, one
    contiguous range per section.  shard="k": the K-elements [lo, hi) of every row -- the row-parallel layer
    (`RowShardedFp4Linear`); one strided read per section (memory-mapped, so again only the shard's bytes are touched).
    On a CUDA device the scales are converted to the tiled layout the GEMM consumes; `tile_major=True` also re-packs the
    nibbles for the decode kernel.  The tensor scale in the file is the scale of the whole matrix, so every shard
    dequantises exactly as the unsharded weight does.
    """
    h = read_header(path)
    fmt = NVFP4 if h["fmt"] == "nvfp4" else MXFP4
    rows, k, block = int(h["rows"]), int(h["k"]), int(h["block"])
    if shard not in ("n", "k"):
        raise ValueError(f"shard must be 'n' or 'k', got {shard!r}.")
    if shard == "n":
        lo, hi = (0, rows) if world == 1 else shard_bounds(rows, world, rank)
        n, kk = hi - lo, k
        packed = np.fromfile(path, dtype=np.uint8, count=n * (k // 2), offset=h["packed_offset"] + lo * (k // 2))
        scales = np.fromfile(path, dtype=np.uint8, count=n * (k // block), offset=h["scales_offset"] + lo * (k // block))
        if packed.size != n * (k // 2) or scales.size != n * (k // block):
            raise ValueError(f"{path} is truncated.")
        packed, scales = packed.reshape(n, k // 2), scales.reshape(n, k // block)
    else:
        lo, hi = (0, k) if world == 1 else k_shard_bounds(k, world, rank)
        n, kk = rows, hi - lo
        try:
            pm = np.memmap(path, dtype=np.uint8, mode="r", offset=h["packed_offset"], shape=(rows, k // 2))
            sm = np.memmap(path, dtype=np.uint8, mode="r", offset=h["scales_offset"], shape=(rows, k // block))
        except ValueError as exc:
            raise ValueError(f"{path} is truncated.") from exc
        packed = np.array(pm[:, lo // 2:hi // 2], order="C", copy=True)
        scales = np.array(sm[:, lo // block:hi // block], order="C", copy=True)
    device = torch.device(device)
    p = torch.from_numpy(packed).to(device)
    s = torch.from_numpy(scales).to(device)
    gs = None
    if fmt == NVFP4:
        gs = torch.tensor([h["global_scale"]], dtype=torch.float32, device=device)
    op = make_operand(p, s, gs, fmt, SF_ROW_MAJOR)
    assert op.rows == n and op.k == kk
    if device.type == "cuda":
        op = pack_weight_tiles(op) if tile_major else to_tiled(op)
    return op
