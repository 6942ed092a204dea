"""FP4 operators in the reference's operator convention.

The reference ships one operator, ``gemm_pipeline_transposed_b(A, B, out=None) -> Tensor``
(python/avelang_kernels/amdgpu_gemm.py:458-494): A is (M, K), B is (N, K), both
K-contiguous, the result is ``A @ B.T`` with fp32 accumulation and bf16 output,
arguments are validated with ``ValueError`` before anything is launched, ``out`` is
allocated only when not given, and the launch is asynchronous on the current stream.

The operators here keep that shape of API for block-scaled FP4 operands:

* ``quantize_nvfp4(x, global_scale=None)`` / ``quantize_mxfp4(x)`` -> ``Fp4Operand``
* ``gemm_nvfp4_transposed_b(A, B, out=None)`` / ``gemm_mxfp4_transposed_b(A, B, out=None)``

All compute runs in hand-written CUDA kernels behind the C ABI of ``libavefp4.so``;
torch tensors are used only to own device memory and to name the current stream.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib

NVFP4 = 0
MXFP4 = 1
SF_ROW_MAJOR = 0
SF_TILED = 1

GEMM_AUTO = 0
GEMM_1CTA_N128 = 1
GEMM_1CTA_N256 = 2
GEMM_2CTA_N256 = 3
GEMM_2CTA_N128 = 4
GEMM_2CTA_N192 = 5
GEMM_SKINNY = 10
GEMM_SKINNY_TILED_W = 11
GEMM_FLAG_STATIC_WEIGHTS = 0x100

_BLOCK = {NVFP4: 16, MXFP4: 32}
_FMT_NAME = {NVFP4: "NVFP4", MXFP4: "MXFP4"}


@dataclass
class Fp4Operand:
    """A quantised (rows, k) matrix, K contiguous.

    packed        uint8 (rows, k/2): element 2j in bits 3:0 of byte j, 2j+1 in bits 7:4 (E2M1)
    scales        uint8, one per 16 (NVFP4, E4M3) or 32 (MXFP4, E8M0) K elements;
                  (rows, k/blk) when ``sf_layout == SF_ROW_MAJOR``, flat 128x4 tiles when ``SF_TILED``
    global_scale  fp32 tensor with one element on the same device (NVFP4) or None (MXFP4)
    """

    packed: torch.Tensor
    scales: torch.Tensor
    global_scale: torch.Tensor | None
    fmt: int
    rows: int
    k: int
    sf_layout: int = SF_TILED
    tile_major: bool = False  # packed bytes re-ordered into 16 KB tiles by pack_weight_tiles (decode weights)
    amax_scratch: torch.Tensor | None = None  # one fp32 on the device, used when the tensor scale is taken from the data

    @property
    def shape(self) -> tuple[int, int]:
        return (self.rows, self.k)

    @property
    def device(self) -> torch.device:
        return self.packed.device


def _ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(device: torch.device) -> ctypes.c_void_p:
    # the reference launches on torch's current raw stream (python/avelang/backends/driver.py:24-32)
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(t: torch.Tensor, name: str) -> int:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor, got device {t.device}.")
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def sf_bytes(rows: int, k: int, fmt: int, sf_layout: int) -> int:
    blk = _BLOCK[fmt]
    cols = k // blk
    if sf_layout == SF_ROW_MAJOR:
        return rows * cols
    return ((rows + 127) // 128) * ((cols + 3) // 4) * 512


def _quantize(x: torch.Tensor, fmt: int, global_scale: torch.Tensor | None, sf_layout: int,
              out: Fp4Operand | None = None) -> Fp4Operand:
    if x.dtype != torch.bfloat16:
        raise ValueError(f"x must have dtype torch.bfloat16, got {x.dtype}.")
    if x.dim() != 2:
        raise ValueError(f"x must be 2-D (rows, K), got shape {tuple(x.shape)}.")
    dev = _require_cuda(x, "x")
    rows, k = x.shape
    if k % 32 != 0:
        raise ValueError(f"K must be a multiple of 32, got {k}.")
    if x.stride(1) != 1 or (rows > 1 and x.stride(0) % 8 != 0) or x.data_ptr() % 16 != 0:
        raise ValueError("x must be K-contiguous with a 16-byte aligned row stride.")
    if out is not None:
        # same convention as the reference operator's `out` (python/avelang_kernels/amdgpu_gemm.py:478-486):
        # a given result is checked and written in place, nothing is allocated
        sf_layout = out.sf_layout
        if out.fmt != fmt or out.shape != (rows, k) or out.tile_major:
            raise ValueError(f"out must be a {_FMT_NAME[fmt]} operand of shape {(rows, k)}, got {_FMT_NAME.get(out.fmt, out.fmt)} {out.shape}.")
        if out.device != x.device:
            raise ValueError(f"out must be on device {x.device}, got {out.device}.")
        if fmt == NVFP4 and out.global_scale is None:
            raise ValueError("an NVFP4 out operand needs a global_scale tensor.")
    if sf_layout not in (SF_ROW_MAJOR, SF_TILED):
        raise ValueError(f"unknown scale layout {sf_layout}.")
    ldx = x.stride(0) if rows > 1 else k
    gs = None
    with torch.cuda.device(dev):
        L = _lib.ensure_init(dev)
        if out is not None:
            packed, scales = out.packed, out.scales
        else:
            packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
            if sf_layout == SF_ROW_MAJOR:
                scales = torch.empty((rows, k // _BLOCK[fmt]), dtype=torch.uint8, device=x.device)
            else:
                scales = torch.empty((sf_bytes(rows, k, fmt, SF_TILED),), dtype=torch.uint8, device=x.device)
        stream = _stream(x.device)
        amax = None
        if fmt == NVFP4:
            if global_scale is None:
                # tensor scale from the data: one fused launch for small inputs, amax + quantise otherwise
                if out is not None:
                    gs = out.global_scale
                    if out.amax_scratch is None:
                        out.amax_scratch = torch.empty((1,), dtype=torch.float32, device=x.device)
                    amax = out.amax_scratch
                else:
                    both = torch.empty((2,), dtype=torch.float32, device=x.device)
                    gs, amax = both[0:1], both[1:2]
                _lib.check(L.ave_fp4_quantize_nvfp4_dynamic(_ptr(x), rows, k, ldx, _ptr(gs), _ptr(packed), _ptr(scales),
                                                            sf_layout, _ptr(amax), stream))
                return out if out is not None else Fp4Operand(packed, scales, gs, fmt, rows, k, sf_layout, False, amax)
            else:
                if global_scale.dtype != torch.float32 or global_scale.numel() != 1:
                    raise ValueError("global_scale must be a float32 tensor with one element.")
                if global_scale.device != x.device:
                    raise ValueError(f"global_scale must be on device {x.device}, got {global_scale.device}.")
                gs = global_scale.reshape(1)
                if out is not None and out.global_scale.data_ptr() != gs.data_ptr():
                    out.global_scale.copy_(gs)     # the operand carries its own copy of the static scale
                    gs = out.global_scale
        elif global_scale is not None:
            raise ValueError("MXFP4 has no global scale.")
        _lib.check(L.ave_fp4_quantize(_ptr(x), rows, k, ldx, fmt, _ptr(amax), _ptr(gs), _ptr(packed), _ptr(scales),
                                      sf_layout, stream))
    return out if out is not None else Fp4Operand(packed, scales, gs, fmt, rows, k, sf_layout)


def quantize_nvfp4(x: torch.Tensor, global_scale: torch.Tensor | None = None, sf_layout: int = SF_TILED,
                   out: Fp4Operand | None = None) -> Fp4Operand:
    """bf16 (rows, K) -> NVFP4: 16-element blocks, E4M3 block scales, one fp32 tensor scale.

    ``global_scale=None`` computes the tensor scale as amax / (6 * 448) on the device
    (no host synchronisation); a given one-element fp32 tensor is used as a static scale.
    ``out``: an operand of the same shape (e.g. an earlier result) to overwrite; then nothing is allocated
    and ``sf_layout`` is taken from it.
    """
    return _quantize(x, NVFP4, global_scale, sf_layout, out)


def quantize_mxfp4(x: torch.Tensor, sf_layout: int = SF_TILED, out: Fp4Operand | None = None) -> Fp4Operand:
    """bf16 (rows, K) -> MXFP4: 32-element blocks, E8M0 (power of two) block scales.  ``out`` as for quantize_nvfp4."""
    return _quantize(x, MXFP4, None, sf_layout, out)


def to_tiled(op: Fp4Operand) -> Fp4Operand:
    """Return ``op`` with its scales in the 128x4 tiled layout the GEMM consumes."""
    if op.sf_layout == SF_TILED:
        return op
    dev = _require_cuda(op.scales, "scales")
    cols = op.k // _BLOCK[op.fmt]
    with torch.cuda.device(dev):
        L = _lib.ensure_init(dev)
        tiled = torch.empty((sf_bytes(op.rows, op.k, op.fmt, SF_TILED),), dtype=torch.uint8, device=op.scales.device)
        _lib.check(L.ave_fp4_sf_to_tiled(_ptr(op.scales.contiguous()), op.rows, cols, _ptr(tiled), _stream(op.scales.device)))
    return Fp4Operand(op.packed, tiled, op.global_scale, op.fmt, op.rows, op.k, SF_TILED)


def pack_weight_tiles(op: Fp4Operand) -> Fp4Operand:
    """Offline re-packing of a weight operand for the decode (M <= 64) path.

    The packed bytes are re-ordered into 16 KB tiles (128 rows x 256 K elements, row block major,
    zero padded) so that the skinny kernel streams every weight row block from HBM as one
    contiguous run.  The result can only be used as the B operand of a GEMM with M <= 64.
    """
    if op.tile_major:
        return op
    op = to_tiled(op)
    dev = _require_cuda(op.packed, "packed")
    with torch.cuda.device(dev):
        L = _lib.ensure_init(dev)
        nbytes = L.ave_fp4_weight_tiles_bytes(op.rows, op.k)
        tiles = torch.empty((nbytes,), dtype=torch.uint8, device=op.packed.device)
        _lib.check(L.ave_fp4_pack_weight_tiles(_ptr(op.packed.contiguous()), op.rows, op.k, _ptr(tiles), _stream(op.packed.device)))
    return Fp4Operand(tiles, op.scales, op.global_scale, op.fmt, op.rows, op.k, SF_TILED, True)


def make_operand(packed: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor | None, fmt: int,
                 sf_layout: int = SF_ROW_MAJOR) -> Fp4Operand:
    """Wrap tensors quantised elsewhere (e.g. offline weights) as an operand, checking shapes.

    torch's view-only dtypes are accepted and re-viewed as bytes: ``float4_e2m1fn_x2`` for the packed
    values, ``float8_e4m3fn`` (NVFP4) / ``float8_e8m0fnu`` (MXFP4) for the scales.
    """
    f4 = getattr(torch, "float4_e2m1fn_x2", None)
    if f4 is not None and packed.dtype == f4:
        packed = packed.view(torch.uint8)
    want_sf = getattr(torch, "float8_e4m3fn", None) if fmt == NVFP4 else getattr(torch, "float8_e8m0fnu", None)
    if want_sf is not None and scales.dtype == want_sf:
        scales = scales.view(torch.uint8)
    if packed.dtype != torch.uint8 or packed.dim() != 2:
        raise ValueError("packed must be a 2-D uint8 tensor (rows, K/2).")
    rows, k = packed.shape[0], packed.shape[1] * 2
    if scales.dtype != torch.uint8 or scales.numel() != sf_bytes(rows, k, fmt, sf_layout):
        raise ValueError(f"scales must be uint8 with {sf_bytes(rows, k, fmt, sf_layout)} elements, got {scales.numel()}.")
    return Fp4Operand(packed.contiguous(), scales.contiguous(), global_scale, fmt, rows, k, sf_layout)


# One scratch buffer per device, shared by every call on that device: calls that could
# overlap on the GPU (different streams) must not share it -- run them on one stream.
_workspaces: dict[int, torch.Tensor] = {}


def _workspace(L, device: torch.device, dev: int, m: int, n: int, k: int, fmt: int, variant: int) -> torch.Tensor | None:
    need = L.ave_fp4_workspace_bytes(m, n, k, fmt, variant, dev)
    if need < 0:
        raise RuntimeError(f"ave-lang Error [CUDA]: workspace query failed ({need}).")
    if need == 0:
        return None
    key = dev
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        # zero-initialised once; the kernel leaves its counters at zero for the next call
        ws = torch.zeros((need,), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


ACTIVATIONS = {None: 0, "none": 0, "relu": 1, "gelu": 2, "gelu_tanh": 3, "silu": 4}


def _gemm(A: Fp4Operand, B: Fp4Operand, out: torch.Tensor | None, fmt: int, variant: int,
          peer_ptrs: list[int] | None = None, static_weights: bool = False,
          bias: torch.Tensor | None = None, activation: str | None = None,
          quant: Fp4Operand | None = None, want_bf16: bool = True) -> torch.Tensor | None:
    name = _FMT_NAME[fmt]
    if activation not in ACTIVATIONS:
        raise ValueError(f"activation must be one of {sorted(k for k in ACTIVATIONS if k)}, got {activation!r}.")
    if A.fmt != fmt:
        raise ValueError(f"A must be an {name} operand, got {_FMT_NAME.get(A.fmt, A.fmt)}.")
    if B.fmt != fmt:
        raise ValueError(f"B must be an {name} operand, got {_FMT_NAME.get(B.fmt, B.fmt)}.")
    m, k = A.rows, A.k
    n = B.rows
    if B.k != k:
        raise ValueError(f"A and B must share K, got {k} and {B.k}.")
    if k % 32 != 0 or k == 0:
        raise ValueError(f"K must be a positive multiple of 32, got {k}.")
    if n % 8 != 0:
        raise ValueError(f"N must be a multiple of 8, got {n}.")
    dev = _require_cuda(A.packed, "A")
    if B.device != A.device:
        raise ValueError(f"B must be on device {A.device}, got {B.device}.")
    if fmt == NVFP4 and (A.global_scale is None or B.global_scale is None):
        raise ValueError("NVFP4 operands need a global_scale tensor.")
    out_shape = (m, n)
    if out is None and not want_bf16:
        pass    # quantised result only
    elif out is None:
        out = torch.empty(out_shape, dtype=torch.bfloat16, device=A.device)
    elif tuple(out.shape) != out_shape:
        raise ValueError(f"out must have shape {out_shape}, got {tuple(out.shape)}.")
    elif out.dtype != torch.bfloat16:
        raise ValueError(f"out must have dtype torch.bfloat16, got {out.dtype}.")
    elif out.device != A.device:
        raise ValueError(f"out must be on device {A.device}, got {out.device}.")
    if out is not None and m > 0 and n > 0 and (out.stride(1) != 1 or out.stride(0) % 8 != 0 or out.data_ptr() % 16 != 0):
        raise ValueError("out must be row-major with a row stride that is a multiple of 8 elements and 16-byte aligned.")
    if bias is not None:
        if bias.dtype != torch.bfloat16 or tuple(bias.shape) != (n,):
            raise ValueError(f"bias must be a bfloat16 tensor of shape ({n},), got {bias.dtype} {tuple(bias.shape)}.")
        if bias.device != A.device:
            raise ValueError(f"bias must be on device {A.device}, got {bias.device}.")
        if not bias.is_contiguous() or bias.data_ptr() % 16 != 0:
            raise ValueError("bias must be contiguous and 16-byte aligned.")
        if peer_ptrs:
            raise ValueError("the fused all-gather takes no bias or activation.")
    if m == 0 or n == 0:
        return out
    if A.tile_major:
        raise ValueError("A must not be a tile-major (pack_weight_tiles) operand.")
    if B.tile_major:
        if m > 64:
            raise ValueError(f"a tile-major weight operand serves only M <= 64, got M = {m}.")
        if variant not in (GEMM_AUTO, GEMM_SKINNY, GEMM_SKINNY_TILED_W):
            raise ValueError(f"a tile-major weight operand cannot be used with variant {variant}.")
        variant = GEMM_SKINNY_TILED_W
    elif variant == GEMM_SKINNY_TILED_W:
        raise ValueError("variant GEMM_SKINNY_TILED_W needs a B operand made by pack_weight_tiles.")
    A = to_tiled(A)
    B = to_tiled(B)
    with torch.cuda.device(dev):
        L = _lib.ensure_init(dev)
        if peer_ptrs:
            if m <= 64:
                raise ValueError(f"the fused all-gather needs M > 64, got {m}.")
            if len(peer_ptrs) > 7:
                raise ValueError(f"at most 7 peers, got {len(peer_ptrs)}.")
            arr = (ctypes.c_void_p * len(peer_ptrs))(*peer_ptrs)
            _lib.check(L.ave_fp4_gemm_allgather(_ptr(A.packed), _ptr(A.scales), _ptr(A.global_scale), _ptr(B.packed),
                                                _ptr(B.scales), _ptr(B.global_scale), _ptr(out), arr, len(peer_ptrs), m, n, k,
                                                out.stride(0), fmt, variant, _stream(A.device)))
            return out
        ws = _workspace(L, A.device, dev, m, n, k, fmt, variant)
        if static_weights:
            variant |= GEMM_FLAG_STATIC_WEIGHTS
        if bias is not None or ACTIVATIONS[activation] != 0 or quant is not None:
            epi = _lib.Epilogue(None if bias is None else bias.data_ptr(), ACTIVATIONS[activation], 0)
            if quant is not None:
                epi.quantize_out = 1
                epi.q_packed = quant.packed.data_ptr()
                epi.q_scales = quant.scales.data_ptr()
                epi.q_global_scale = None if quant.global_scale is None else quant.global_scale.data_ptr()
                epi.q_sf_layout = quant.sf_layout
            ldd = n if out is None else out.stride(0)
            _lib.check(L.ave_fp4_gemm_epilogue(_ptr(A.packed), _ptr(A.scales), _ptr(A.global_scale), _ptr(B.packed),
                                               _ptr(B.scales), _ptr(B.global_scale), _ptr(out), m, n, k, ldd, fmt,
                                               variant, _ptr(ws), 0 if ws is None else ws.numel(), _stream(A.device),
                                               ctypes.byref(epi)))
            return out
        _lib.check(L.ave_fp4_gemm(_ptr(A.packed), _ptr(A.scales), _ptr(A.global_scale), _ptr(B.packed), _ptr(B.scales),
                                  _ptr(B.global_scale), _ptr(out), m, n, k, out.stride(0), fmt, variant, _ptr(ws),
                                  0 if ws is None else ws.numel(), _stream(A.device)))
    return out


def gemm_nvfp4_transposed_b(A: Fp4Operand, B: Fp4Operand, out: torch.Tensor | None = None,
                            variant: int = GEMM_AUTO, static_weights: bool = False,
                            bias: torch.Tensor | None = None, activation: str | None = None) -> torch.Tensor:
    """``out = A @ B.T`` for NVFP4 operands A (M, K) and B (N, K); fp32 accumulate, bf16 out.

    ``static_weights=True`` promises that B is not written by anything queued earlier on the stream; the
    decode kernel (M <= 64) then overlaps its start-up and first weight loads with the previous kernel.
    ``bias`` ((N,) bf16) and ``activation`` ("relu", "gelu", "gelu_tanh", "silu") are fused into the epilogue:
    ``out = act(A @ B.T + bias)``, evaluated in fp32 and rounded to bf16 once.
    """
    return _gemm(A, B, out, NVFP4, variant, static_weights=static_weights, bias=bias, activation=activation)


def gemm_mxfp4_transposed_b(A: Fp4Operand, B: Fp4Operand, out: torch.Tensor | None = None,
                            variant: int = GEMM_AUTO, static_weights: bool = False,
                            bias: torch.Tensor | None = None, activation: str | None = None) -> torch.Tensor:
    """``out = act(A @ B.T + bias)`` for MXFP4 operands A (M, K) and B (N, K); fp32 accumulate, bf16 out."""
    return _gemm(A, B, out, MXFP4, variant, static_weights=static_weights, bias=bias, activation=activation)


GEMM_FLAG_TILE_MAJOR_WEIGHTS = 0x200
_decode_workspaces: dict[int, torch.Tensor] = {}


def _linear_decode(x: torch.Tensor, W: Fp4Operand, out: torch.Tensor | None, fmt: int, static_weights: bool,
                   bias: torch.Tensor | None, activation: str | None) -> torch.Tensor:
    name = _FMT_NAME[fmt]
    if activation not in ACTIVATIONS:
        raise ValueError(f"activation must be one of {sorted(k for k in ACTIVATIONS if k)}, got {activation!r}.")
    if x.dtype != torch.bfloat16:
        raise ValueError(f"x must have dtype torch.bfloat16, got {x.dtype}.")
    if x.dim() != 2:
        raise ValueError(f"x must be 2-D (M, K), got shape {tuple(x.shape)}.")
    if W.fmt != fmt:
        raise ValueError(f"W must be an {name} operand, got {_FMT_NAME.get(W.fmt, W.fmt)}.")
    m, k = x.shape
    n = W.rows
    if W.k != k:
        raise ValueError(f"x and W must share K, got {k} and {W.k}.")
    if k % 32 != 0 or k == 0:
        raise ValueError(f"K must be a positive multiple of 32, got {k}.")
    if n % 8 != 0:
        raise ValueError(f"N must be a multiple of 8, got {n}.")
    dev = _require_cuda(x, "x")
    if W.device != x.device:
        raise ValueError(f"W must be on device {x.device}, got {W.device}.")
    if x.stride(1) != 1 or (m > 1 and x.stride(0) % 8 != 0) or x.data_ptr() % 16 != 0:
        raise ValueError("x must be K-contiguous with a 16-byte aligned row stride.")
    if fmt == NVFP4 and W.global_scale is None:
        raise ValueError("an NVFP4 weight operand needs a global_scale tensor.")
    if m > 32:
        # more rows than the one-call decode entry point serves: the two operators, same results
        q = _quantize(x, fmt, None, SF_TILED)
        return _gemm(q, W, out, fmt, GEMM_AUTO, static_weights=static_weights, bias=bias, activation=activation)
    out_shape = (m, n)
    if out is None:
        out = torch.empty(out_shape, dtype=torch.bfloat16, device=x.device)
    elif tuple(out.shape) != out_shape:
        raise ValueError(f"out must have shape {out_shape}, got {tuple(out.shape)}.")
    elif out.dtype != torch.bfloat16:
        raise ValueError(f"out must have dtype torch.bfloat16, got {out.dtype}.")
    elif out.device != x.device:
        raise ValueError(f"out must be on device {x.device}, got {out.device}.")
    if out.stride(1) != 1 or out.stride(0) % 8 != 0 or out.data_ptr() % 16 != 0:
        raise ValueError("out must be row-major with a row stride that is a multiple of 8 elements and 16-byte aligned.")
    if bias is not None and (bias.dtype != torch.bfloat16 or tuple(bias.shape) != (n,) or bias.device != x.device
                             or not bias.is_contiguous() or bias.data_ptr() % 16 != 0):
        raise ValueError(f"bias must be a contiguous, 16-byte aligned bfloat16 tensor of shape ({n},) on {x.device}.")
    if m == 0 or n == 0:
        return out
    W = to_tiled(W)
    with torch.cuda.device(dev):
        L = _lib.ensure_init(dev)
        need = L.ave_fp4_linear_decode_workspace_bytes(m, n, k, fmt, dev)
        if need < 0:
            raise RuntimeError(f"ave-lang Error [CUDA]: workspace query failed ({need}).")
        ws = _decode_workspaces.get(dev)
        if ws is None or ws.numel() < need:
            # zero-initialised once; the kernel leaves its counters at zero for the next call
            ws = torch.zeros((need,), dtype=torch.uint8, device=x.device)
            _decode_workspaces[dev] = ws
        flags = (GEMM_FLAG_STATIC_WEIGHTS if static_weights else 0) | (GEMM_FLAG_TILE_MAJOR_WEIGHTS if W.tile_major else 0)
        epi = None
        if bias is not None or ACTIVATIONS[activation] != 0:
            epi = ctypes.byref(_lib.Epilogue(None if bias is None else bias.data_ptr(), ACTIVATIONS[activation], 0))
        _lib.check(L.ave_fp4_linear_decode(_ptr(x), x.stride(0) if m > 1 else k, _ptr(W.packed), _ptr(W.scales), _ptr(W.global_scale),
                                           _ptr(out), m, n, k, out.stride(0), fmt, flags, _ptr(ws), ws.numel(), _stream(x.device), epi))
    return out


def linear_nvfp4_decode(x: torch.Tensor, W: Fp4Operand, out: torch.Tensor | None = None, static_weights: bool = False,
                        bias: torch.Tensor | None = None, activation: str | None = None) -> torch.Tensor:
    """``act(quantize_nvfp4(x) @ W.T + bias)`` for bf16 activations x (M, K) and an NVFP4 weight operand W (N, K).

    Up to M = 32 this is one call into the library that allocates nothing: the activations are quantised (tensor scale
    from the data) into a scratch buffer and the decode GEMM is chained behind the quantise kernel with programmatic
    dependent launch; results are bit-identical to ``gemm_nvfp4_transposed_b(quantize_nvfp4(x), W)``.  More rows take
    that route through the two operators.  One scratch buffer per device is shared by every call on that device: keep
    such calls on one stream.
    """
    return _linear_decode(x, W, out, NVFP4, static_weights, bias, activation)


def linear_mxfp4_decode(x: torch.Tensor, W: Fp4Operand, out: torch.Tensor | None = None, static_weights: bool = False,
                        bias: torch.Tensor | None = None, activation: str | None = None) -> torch.Tensor:
    """``act(quantize_mxfp4(x) @ W.T + bias)``; see linear_nvfp4_decode."""
    return _linear_decode(x, W, out, MXFP4, static_weights, bias, activation)


def gemm_quantized_out_transposed_b(A: Fp4Operand, B: Fp4Operand, out_global_scale: torch.Tensor | None = None,
                                    bias: torch.Tensor | None = None, activation: str | None = None,
                                    sf_layout: int = SF_TILED, out_bf16: torch.Tensor | bool | None = None,
                                    variant: int = GEMM_AUTO) -> Fp4Operand | tuple[Fp4Operand, torch.Tensor]:
    """``act(A @ B.T + bias)`` delivered as an FP4 operand (M, N) of A's format with its scale blocks along N --
    the A operand of the next layer's GEMM -- straight from the GEMM epilogue, without the bf16 matrix going
    through memory.  Bit-identical to quantising the bf16 result with ``quantize_nvfp4(out, global_scale=...)``
    / ``quantize_mxfp4(out)``.  NVFP4 needs ``out_global_scale`` (a 1-element fp32 tensor: the static, calibrated
    tensor scale of the result).  ``out_bf16``: True or a (M, N) bf16 tensor to receive the bf16 result as well;
    then ``(operand, bf16)`` is returned."""
    fmt = A.fmt
    m, n = A.rows, B.rows
    blk = 16 if fmt == NVFP4 else 32
    if n % blk != 0:
        raise ValueError(f"a quantised result needs N % {blk} == 0, got {n}.")
    if fmt == NVFP4:
        if out_global_scale is None or out_global_scale.dtype != torch.float32 or out_global_scale.numel() != 1:
            raise ValueError("an NVFP4 result needs out_global_scale: a 1-element float32 tensor.")
        if out_global_scale.device != A.device:
            raise ValueError(f"out_global_scale must be on device {A.device}, got {out_global_scale.device}.")
    else:
        out_global_scale = None
    if sf_layout not in (SF_ROW_MAJOR, SF_TILED):
        raise ValueError(f"unknown sf_layout {sf_layout}.")
    if variant in (GEMM_SKINNY, GEMM_SKINNY_TILED_W) or B.tile_major:
        raise ValueError("the quantising epilogue is served by the tiled kernels only.")
    packed = torch.empty((m, n // 2), dtype=torch.uint8, device=A.device)
    scales = torch.empty((sf_bytes(m, n, fmt, sf_layout),), dtype=torch.uint8, device=A.device)
    if sf_layout == SF_ROW_MAJOR:
        scales = scales.view(m, n // blk)
    q = Fp4Operand(packed, scales, out_global_scale, fmt, m, n, sf_layout)
    want = out_bf16 is not None and out_bf16 is not False
    res = _gemm(A, B, out_bf16 if isinstance(out_bf16, torch.Tensor) else None, fmt, variant, bias=bias,
                activation=activation, quant=q, want_bf16=want)
    return (q, res) if want else q


def gemm_allgather_quantized_transposed_b(A: Fp4Operand, B: Fp4Operand, gathered: Fp4Operand, col0: int,
                                          peer_packed_ptrs: list[int], peer_scale_ptrs: list[int],
                                          bias: torch.Tensor | None = None, activation: str | None = None,
                                          variant: int = GEMM_AUTO) -> Fp4Operand:
    """``act(A @ B.T + bias)`` quantised in the GEMM epilogue as columns ``[col0, col0 + N)`` of ``gathered`` (an
    (M, N_total) operand of A's format with tiled or row-major scales, NVFP4 with its static ``global_scale``) and,
    fused into the same epilogue, stored to the other ranks' copies of that operand: ``peer_packed_ptrs`` /
    ``peer_scale_ptrs`` are raw device addresses (valid on this GPU) of the bases of their packed bytes and scales.
    The all-gather of an N-sharded layer's output in the form the next layer's GEMM consumes."""
    fmt = A.fmt
    name = _FMT_NAME[fmt]
    if activation not in ACTIVATIONS:
        raise ValueError(f"activation must be one of {sorted(k for k in ACTIVATIONS if k)}, got {activation!r}.")
    if B.fmt != fmt or gathered.fmt != fmt:
        raise ValueError(f"A, B and the gathered operand must all be {name} operands.")
    m, k, n = A.rows, A.k, B.rows
    if B.k != k:
        raise ValueError(f"A and B must share K, got {k} and {B.k}.")
    if m <= 64:
        raise ValueError(f"the fused all-gather needs M > 64, got {m}.")
    n_total = gathered.k
    if gathered.rows != m:
        raise ValueError(f"the gathered operand must have {m} rows, got {gathered.rows}.")
    if n % 64 or col0 % 64 or n_total % 64 or col0 < 0 or col0 + n > n_total:
        raise ValueError(f"N, col0 and N_total must be multiples of 64 with col0 + N <= N_total, got {n}, {col0}, {n_total}.")
    if len(peer_packed_ptrs) != len(peer_scale_ptrs) or len(peer_packed_ptrs) > 7:
        raise ValueError("one packed and one scale address per peer, at most 7 peers.")
    if fmt == NVFP4 and (A.global_scale is None or B.global_scale is None or gathered.global_scale is None):
        raise ValueError("NVFP4 operands need a global_scale tensor (the gathered operand a static one).")
    if A.tile_major or B.tile_major or gathered.tile_major:
        raise ValueError("tile-major operands serve the decode kernel only.")
    if bias is not None and (bias.dtype != torch.bfloat16 or tuple(bias.shape) != (n,) or bias.device != A.device
                             or not bias.is_contiguous() or bias.data_ptr() % 16 != 0):
        raise ValueError(f"bias must be a contiguous, 16-byte aligned bfloat16 tensor of shape ({n},) on {A.device}.")
    dev = _require_cuda(A.packed, "A")
    if B.device != A.device or gathered.device != A.device:
        raise ValueError(f"B and the gathered operand must be on device {A.device}.")
    A = to_tiled(A)
    B = to_tiled(B)
    with torch.cuda.device(dev):
        L = _lib.ensure_init(dev)
        epi = _lib.Epilogue(None if bias is None else bias.data_ptr(), ACTIVATIONS[activation], 1)
        epi.q_packed = gathered.packed.data_ptr()
        epi.q_scales = gathered.scales.data_ptr()
        epi.q_global_scale = None if gathered.global_scale is None else gathered.global_scale.data_ptr()
        epi.q_sf_layout = gathered.sf_layout
        np_ = len(peer_packed_ptrs)
        pk = (ctypes.c_void_p * max(np_, 1))(*peer_packed_ptrs)
        ps = (ctypes.c_void_p * max(np_, 1))(*peer_scale_ptrs)
        _lib.check(L.ave_fp4_gemm_allgather_quantized(_ptr(A.packed), _ptr(A.scales), _ptr(A.global_scale), _ptr(B.packed),
                                                      _ptr(B.scales), _ptr(B.global_scale), m, n, k, fmt, variant, ctypes.byref(epi),
                                                      n_total, col0, pk, ps, np_, _stream(A.device)))
    return gathered


def gemm_allgather_transposed_b(A: Fp4Operand, B: Fp4Operand, out: torch.Tensor, peer_ptrs: list[int],
                                variant: int = GEMM_AUTO) -> torch.Tensor:
    """``out = A @ B.T`` and, fused into the epilogue, the same tiles stored to ``peer_ptrs``: raw device
    addresses (valid on this GPU) of the matching (M, N) block in every other rank's result buffer."""
    return _gemm(A, B, out, A.fmt, variant, peer_ptrs)


def gemm_partials_transposed_b(A: Fp4Operand, B: Fp4Operand, slab_ptrs: list[int], first_owner: int = 0) -> None:
    """First half of a K-sharded GEMM + reduce-scatter.  A (M, K_r) and B (N, K_r) are this rank's K-slices; the
    fp32 product is scattered by rows: rows ``[j*M/w, (j+1)*M/w)`` are stored (row stride N) at ``slab_ptrs[j]``,
    raw device addresses valid on this GPU (peer-mapped for other ranks' buffers), ``w = len(slab_ptrs)``.  The tile
    schedule starts at the rows of owner ``first_owner``; ranks should pass different values (rank + 1 mod w) so that
    their stores are spread over all destination GPUs at any time."""
    fmt = A.fmt
    if B.fmt != fmt:
        raise ValueError("A and B must have the same format.")
    m, k, n = A.rows, A.k, B.rows
    world = len(slab_ptrs)
    if B.k != k:
        raise ValueError(f"A and B must share K, got {k} and {B.k}.")
    if not 1 <= world <= 8:
        raise ValueError(f"1..8 slabs, got {world}.")
    if not 0 <= first_owner < world:
        raise ValueError(f"first_owner must be in [0, {world}), got {first_owner}.")
    if m <= 0 or m % (32 * world) != 0:
        raise ValueError(f"M must be a positive multiple of 32 * world = {32 * world}, got {m}.")
    if n % 8 != 0 or k % 32 != 0 or k == 0:
        raise ValueError(f"N must be a multiple of 8 and K a positive multiple of 32, got N = {n}, K = {k}.")
    if A.tile_major or B.tile_major:
        raise ValueError("tile-major operands serve the decode kernel only.")
    if fmt == NVFP4 and (A.global_scale is None or B.global_scale is None):
        raise ValueError("NVFP4 operands need a global_scale tensor.")
    dev = _require_cuda(A.packed, "A")
    if B.device != A.device:
        raise ValueError(f"B must be on device {A.device}, got {B.device}.")
    A = to_tiled(A)
    B = to_tiled(B)
    with torch.cuda.device(dev):
        L = _lib.ensure_init(dev)
        arr = (ctypes.c_void_p * world)(*slab_ptrs)
        _lib.check(L.ave_fp4_gemm_partials(_ptr(A.packed), _ptr(A.scales), _ptr(A.global_scale), _ptr(B.packed), _ptr(B.scales),
                                           _ptr(B.global_scale), arr, world, first_owner, m, n, k, fmt, _stream(A.device)))


def reduce_partials(slabs: torch.Tensor, out: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                    activation: str | None = None) -> torch.Tensor:
    """Second half: ``out (rows, N) bf16 = act(slabs.sum(0) + bias)`` for fp32 slabs (world, rows, N), summed in slab
    order, rounded once."""
    if slabs.dtype != torch.float32 or slabs.dim() != 3 or not slabs.is_contiguous():
        raise ValueError("slabs must be a contiguous float32 tensor (world, rows, N).")
    if activation not in ACTIVATIONS:
        raise ValueError(f"activation must be one of {sorted(k for k in ACTIVATIONS if k)}, got {activation!r}.")
    world, rows, n = slabs.shape
    dev = _require_cuda(slabs, "slabs")
    if n % 8 != 0:
        raise ValueError(f"N must be a multiple of 8, got {n}.")
    if out is None:
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=slabs.device)
    elif tuple(out.shape) != (rows, n) or out.dtype != torch.bfloat16 or out.device != slabs.device:
        raise ValueError(f"out must be a bfloat16 tensor of shape {(rows, n)} on {slabs.device}.")
    if out.stride(1) != 1 or out.stride(0) % 8 != 0 or out.data_ptr() % 16 != 0:
        raise ValueError("out must be row-major with a row stride that is a multiple of 8 elements and 16-byte aligned.")
    if bias is not None and (bias.dtype != torch.bfloat16 or tuple(bias.shape) != (n,) or bias.device != slabs.device
                             or not bias.is_contiguous() or bias.data_ptr() % 16 != 0):
        raise ValueError(f"bias must be a contiguous, 16-byte aligned bfloat16 tensor of shape ({n},) on {slabs.device}.")
    with torch.cuda.device(dev):
        L = _lib.ensure_init(dev)
        epi = _lib.Epilogue(None if bias is None else bias.data_ptr(), ACTIVATIONS[activation], 0)
        _lib.check(L.ave_fp4_reduce_partials(_ptr(slabs), world, rows, n, _ptr(out), out.stride(0), ctypes.byref(epi),
                                             _stream(slabs.device)))
    return out


def check_device_status(device: torch.device | None = None) -> None:
    """Synchronise the current stream and raise if a kernel recorded a wait time-out."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    dev = device.index if device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(dev):
        L = _lib.ensure_init(dev)
        _lib.check(L.ave_fp4_check(_stream(device)))
