"""N-sharded FP4 linear layer: column-parallel GEMM plus an all-gather of the bf16 output.

The reference has no multi-GPU code (single process, current device, current stream:
python/avelang/backends/driver.py:24-32).  This module adds the one exchange step the
sharded workload needs on a single NVLink/NVSwitch box: with B (N, K) split by rows
across `world` ranks, rank r computes ``D[:, r*N/w:(r+1)*N/w] = A @ B_r.T`` with no
inter-rank dependency, and the slices are exchanged with one all-gather.

Layout of the gathered result: ``(world, M, N/world)`` -- rank r's column block is the
contiguous slab ``gathered[r]``; ``columns_view`` presents it as a strided (M, world, N/world) view.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .fp4_gemm import (Fp4Operand, gemm_allgather_quantized_transposed_b, gemm_allgather_transposed_b, gemm_mxfp4_transposed_b,
                       gemm_nvfp4_transposed_b, gemm_partials_transposed_b, reduce_partials, sf_bytes, NVFP4, SF_TILED)


def shard_bounds(n: int, world: int, rank: int, align: int = 128) -> tuple[int, int]:
    """Rows [lo, hi) of the (N, K) weight owned by `rank`; every shard is a multiple of `align`."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}.")
    if n % (world * align) != 0:
        raise ValueError(f"N must be a multiple of world*{align} = {world * align}, got {n}.")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_rows(weight_bf16: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """The slice of a full (N, K) bf16 weight this rank quantises and keeps."""
    lo, hi = shard_bounds(weight_bf16.shape[0], world, rank)
    return weight_bf16[lo:hi]


def all_gather_columns(local: torch.Tensor, gathered: torch.Tensor | None = None, group=None) -> torch.Tensor:
    """All-gather equal (M, n_local) slices into a (world, M, n_local) tensor (works on any backend)."""
    world = dist.get_world_size(group)
    if gathered is None:
        gathered = torch.empty((world, *local.shape), dtype=local.dtype, device=local.device)
    elif tuple(gathered.shape) != (world, *local.shape):
        raise ValueError(f"gathered must have shape {(world, *local.shape)}, got {tuple(gathered.shape)}.")
    dist.all_gather_into_tensor(gathered.view(-1, local.shape[-1]), local.contiguous(), group=group)
    return gathered


def columns_view(gathered: torch.Tensor) -> torch.Tensor:
    """(world, M, n_local) -> (M, world, n_local) strided view (no copy): ``view[i, r, j]`` is element
    ``(i, r * n_local + j)`` of the logical (M, world * n_local) result.  The slabs are not adjacent in memory,
    so the 2-D matrix itself needs a copy: ``columns_view(g).reshape(M, world * n_local)``."""
    return gathered.permute(1, 0, 2)


class ShardedFp4Linear:
    """Column-parallel ``y = x @ W.T`` with W sharded by rows (output columns).

    The NVFP4 tensor scale of W must be computed over the whole tensor before sharding
    (pass it to ``quantize_nvfp4(shard, global_scale=...)``), so that every rank's
    shard dequantises exactly as the unsharded weight would.
    """

    def __init__(self, weight_shard: Fp4Operand, group=None, fused: bool = False):
        """fused=False: local GEMM, then NCCL all-gather.  fused=True: the GEMM epilogue stores every
        output tile into all ranks' result buffers over NVLink (symmetric memory, plain peer stores),
        so the exchange overlaps the math; a device-side barrier ends the step."""
        self.weight = weight_shard
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.fused = bool(fused) and self.world > 1
        self._gathered: torch.Tensor | None = None
        self._hdl = None
        self._peer_ptrs: list[int] = []

    def local_forward(self, x: Fp4Operand, out: torch.Tensor | None = None) -> torch.Tensor:
        fn = gemm_nvfp4_transposed_b if self.weight.fmt == NVFP4 else gemm_mxfp4_transposed_b
        return fn(x, self.weight, out=out)

    def _buffers(self, m: int, n_local: int, device: torch.device) -> None:
        shape = (self.world, m, n_local)
        if self._gathered is not None and tuple(self._gathered.shape) == shape:
            return
        if self.fused:
            try:
                import torch.distributed._symmetric_memory as symm

                self._gathered = symm.empty(shape, dtype=torch.bfloat16, device=device)
                self._hdl = symm.rendezvous(self._gathered, self.group if self.group is not None else dist.group.WORLD)
            except Exception as exc:  # no peer-mapped memory on this system: exchange with NCCL after the GEMM instead
                import warnings

                warnings.warn(f"symmetric memory is unavailable ({exc!r}); ShardedFp4Linear uses the NCCL all-gather")
                self.fused = False
                self._hdl = None
                self._gathered = torch.empty(shape, dtype=torch.bfloat16, device=device)
                return
            slab_bytes = m * n_local * 2
            # this rank's slab inside every other rank's buffer; start with the next rank so that
            # the ranks do not all push to the same destination at once
            order = peer_order(self.rank, self.world)
            self._peer_ptrs = [int(self._hdl.buffer_ptrs[p]) + self.rank * slab_bytes for p in order]
        else:
            self._gathered = torch.empty(shape, dtype=torch.bfloat16, device=device)

    def forward(self, x: Fp4Operand) -> torch.Tensor:
        """Returns the gathered (world, M, N/world) bf16 result (the buffer is reused between calls, so
        every rank must be done reading the previous result before any rank calls forward again).

        The local GEMM writes straight into this rank's slab of the gathered buffer; the exchange is
        either an in-place NCCL all-gather or, with fused=True, part of the GEMM kernel itself.
        """
        m, n_local = x.rows, self.weight.rows
        self._buffers(m, n_local, x.device)
        local = self._gathered[self.rank]
        if self.fused and m > 64:
            gemm_allgather_transposed_b(x, self.weight, local, self._peer_ptrs)
            self._hdl.barrier()
            return self._gathered
        self.local_forward(x, out=local)
        if self.world > 1:
            dist.all_gather_into_tensor(self._gathered.view(-1, n_local), local, group=self.group)
        return self._gathered


def peer_order(rank: int, world: int) -> list[int]:
    """The other ranks in the order this rank stores to them: starting with the next rank, so that at any moment the
    ranks push to different destinations."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}.")
    return [(rank + i) % world for i in range(1, world)]


def quantized_gather_layout(m: int, n_local: int, world: int, rank: int, fmt: int) -> dict:
    """Byte layout of one rank's copy of the gathered (M, world * n_local) FP4 operand inside its symmetric buffer:
    packed bytes first, then (256-byte aligned) the tiled scales; plus this rank's first column in the operand."""
    if n_local % 64 != 0:
        raise ValueError(f"every rank's column block must be a multiple of 64 columns, got {n_local}.")
    n_total = n_local * world
    pk_bytes = m * n_total // 2
    pk_pad = (pk_bytes + 255) // 256 * 256
    sf_b = sf_bytes(m, n_total, fmt, SF_TILED)
    return {"n_total": n_total, "packed_bytes": pk_bytes, "scales_offset": pk_pad, "scales_bytes": sf_b,
            "total_bytes": pk_pad + sf_b, "col0": rank * n_local}


class ShardedFp4LinearQuantizedOut:
    """Column-parallel ``y = act(x @ W.T + bias)`` whose output is gathered as the NEXT layer's FP4 operand.

    When the consumer of the gathered activations is another FP4 GEMM, the ranks need not exchange bf16: the GEMM
    epilogue quantises its tile (blocks along N, the next layer's K) and stores the packed bytes and scale bytes
    straight into every rank's copy of the (M, N) operand (symmetric memory, plain peer stores over NVLink) --
    0.5625 byte per element (NVFP4) instead of 2.  ``forward`` returns that operand (scales in the tiled layout the GEMM
    consumes); its bytes equal ``quantize_nvfp4(y, global_scale=out_global_scale)`` / ``quantize_mxfp4(y)`` of the
    unsharded bf16 result.  NVFP4 needs a static tensor scale for the output, the same on every rank.
    """

    def __init__(self, weight_shard: Fp4Operand, out_global_scale: torch.Tensor | None = None, group=None):
        self.weight = weight_shard
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if weight_shard.fmt == NVFP4 and out_global_scale is None:
            raise ValueError("an NVFP4 output needs out_global_scale: a 1-element float32 tensor, the same on every rank.")
        self.out_gs = out_global_scale if weight_shard.fmt == NVFP4 else None
        self._op: Fp4Operand | None = None
        self._hdl = None
        self._peer_packed: list[int] = []
        self._peer_sf: list[int] = []

    def _buffers(self, m: int, n_local: int, device: torch.device) -> None:
        fmt = self.weight.fmt
        lay = quantized_gather_layout(m, n_local, self.world, self.rank, fmt)
        n_total, pk_bytes, pk_pad, sf_b = lay["n_total"], lay["packed_bytes"], lay["scales_offset"], lay["scales_bytes"]
        if self._op is not None and self._op.shape == (m, n_total):
            return
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm

            buf = symm.empty((lay["total_bytes"],), dtype=torch.uint8, device=device)
            self._hdl = symm.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
            order = peer_order(self.rank, self.world)
            self._peer_packed = [int(self._hdl.buffer_ptrs[p]) for p in order]
            self._peer_sf = [int(self._hdl.buffer_ptrs[p]) + pk_pad for p in order]
        else:
            buf = torch.empty((lay["total_bytes"],), dtype=torch.uint8, device=device)
        self._op = Fp4Operand(buf[:pk_bytes].view(m, n_total // 2), buf[pk_pad:pk_pad + sf_b], self.out_gs, fmt, m, n_total, SF_TILED)

    def forward(self, x: Fp4Operand, bias: torch.Tensor | None = None, activation: str | None = None) -> Fp4Operand:
        """Returns the gathered (M, N) operand (its buffer is reused between calls: every rank must be done with the
        previous result before any rank calls forward again)."""
        m, n_local = x.rows, self.weight.rows
        self._buffers(m, n_local, x.device)
        gemm_allgather_quantized_transposed_b(x, self.weight, self._op, self.rank * n_local, self._peer_packed, self._peer_sf,
                                              bias=bias, activation=activation)
        if self._hdl is not None:
            self._hdl.barrier()
        return self._op


def k_shard_bounds(k: int, world: int, rank: int, align: int = 256) -> tuple[int, int]:
    """K-elements [lo, hi) of the operands owned by `rank` in the K-sharded (row-parallel) layer; every shard is a
    multiple of `align` (whole scale blocks and whole 128-byte operand rows of the kernel's K stage)."""
    return shard_bounds(k, world, rank, align)


def slab_offsets(world: int, rank: int, rows_per_rank: int, n: int) -> list[int]:
    """Byte offset, inside EVERY rank's (world, rows_per_rank, n) fp32 staging buffer, of the slab `rank` writes;
    returned once per destination rank for symmetry with the pointer list the kernel takes."""
    if not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}.")
    return [rank * rows_per_rank * n * 4 for _ in range(world)]


class RowShardedFp4Linear:
    """Row-parallel ``y = x @ W.T`` with W (N, K) and x (M, K) sharded along K, followed by a reduce-scatter over
    the rows of y: rank j ends up with ``y[j*M/w:(j+1)*M/w]`` (bf16), summed over all ranks' K-slices in rank order.

    The typical producer of the K-sliced activation is the column-parallel layer before it (``ShardedFp4Linear``
    without its all-gather, or the quantising epilogue): rank r's output columns are exactly its K-slice here.
    NVFP4 tensor scales may differ per rank (each partial carries its own); MXFP4 has none.

    fused=True: the GEMM epilogue stores every fp32 partial tile straight into the owner rank's staging buffer
    (symmetric memory, plain peer stores over NVLink), device-side barriers bracket the step and a small kernel sums the
    `world` slabs in rank order.  fused=False: partials stay local and NCCL reduce-scatters them in fp32.
    """

    def __init__(self, weight_kshard: Fp4Operand, group=None, fused: bool = True):
        self.weight = weight_kshard
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.fused = bool(fused) and self.world > 1
        self._staging: torch.Tensor | None = None
        self._hdl = None
        self._ptrs: list[int] = []
        self._sum: torch.Tensor | None = None

    def _buffers(self, m: int, n: int, device: torch.device) -> None:
        rows = m // self.world
        shape = (self.world, rows, n)
        if self._staging is not None and tuple(self._staging.shape) == shape:
            return
        offs = slab_offsets(self.world, self.rank, rows, n)
        if self.fused:
            try:
                import torch.distributed._symmetric_memory as symm

                self._staging = symm.empty(shape, dtype=torch.float32, device=device)
                self._hdl = symm.rendezvous(self._staging, self.group if self.group is not None else dist.group.WORLD)
                self._ptrs = [int(self._hdl.buffer_ptrs[j]) + offs[j] for j in range(self.world)]
                return
            except Exception as exc:  # no peer-mapped memory on this system
                import warnings

                warnings.warn(f"symmetric memory is unavailable ({exc!r}); RowShardedFp4Linear uses the NCCL reduce-scatter")
                self.fused = False
                self._hdl = None
        # local staging: slab j = this rank's partial of rank j's rows; reduced across ranks by NCCL
        self._staging = torch.empty(shape, dtype=torch.float32, device=device)
        self._ptrs = [self._staging.data_ptr() + j * rows * n * 4 for j in range(self.world)]
        self._sum = torch.empty((1, rows, n), dtype=torch.float32, device=device)

    def forward(self, x_kshard: Fp4Operand, bias: torch.Tensor | None = None, activation: str | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
        """Returns this rank's (M / world, N) bf16 rows of ``act(x @ W.T + bias)``."""
        m, n = x_kshard.rows, self.weight.rows
        if m % (32 * self.world) != 0:
            raise ValueError(f"M must be a multiple of 32 * world = {32 * self.world}, got {m}.")
        self._buffers(m, n, x_kshard.device)
        if self.fused:
            self._hdl.barrier()      # every rank has finished reading its staging buffer from the previous step
            gemm_partials_transposed_b(x_kshard, self.weight, self._ptrs, first_owner=(self.rank + 1) % self.world)
            self._hdl.barrier()      # every rank's partials have landed
            return reduce_partials(self._staging, out=out, bias=bias, activation=activation)
        gemm_partials_transposed_b(x_kshard, self.weight, self._ptrs, first_owner=(self.rank + 1) % self.world)
        if self.world > 1:
            dist.reduce_scatter_tensor(self._sum[0], self._staging.view(-1, n), op=dist.ReduceOp.SUM, group=self.group)
            return reduce_partials(self._sum, out=out, bias=bias, activation=activation)
        return reduce_partials(self._staging, out=out, bias=bias, activation=activation)
