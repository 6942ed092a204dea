"""The operators through the native module instead of ctypes.

``_avefp4_shim`` (python/src/avefp4_shim.cc, built by ``avelang_b200.build.build_shim``) exposes the C ABI of
libavefp4.so as a pybind11 module, the way the reference exposes its native code (python/src/avelang_bindings.cc).
The functions here are the GEMM and decode operators written against it: same arguments, checks and results as
``avelang_kernels.nvfp4_gemm`` -- they share the operand type and the scratch buffers -- only the last hop
(tensor -> pointer -> library) differs.  ctypes stays the default binding; this module exists for hosts that want a
single native extension and no ctypes.
"""
from __future__ import annotations

import torch

from avelang_b200 import fp4_gemm as _ops
from avelang_b200.fp4_gemm import Fp4Operand


def shim():
    """The native module (raises ImportError with the build hint when it has not been built)."""
    try:
        from . import _avefp4_shim
    except ImportError as exc:  # not built: say how
        raise ImportError("avelang_kernels._avefp4_shim is missing: build it with "
                          "`python -c 'from avelang_b200 import build; build.build_shim()'` (needs g++ and pybind11).") from exc
    return _avefp4_shim


def _p(t: torch.Tensor | None) -> int:
    return 0 if t is None else t.data_ptr()


def gemm_fp4_transposed_b(A: Fp4Operand, B: Fp4Operand, out: torch.Tensor | None = None, variant: int = _ops.GEMM_AUTO,
                          bias: torch.Tensor | None = None, activation: str | None = None) -> torch.Tensor:
    """``out = act(A @ B.T + bias)`` for two operands of the same FP4 format, launched through the native module."""
    S = shim()
    if A.fmt != B.fmt:
        raise ValueError("A and B must have the same format.")
    if activation not in _ops.ACTIVATIONS:
        raise ValueError(f"activation must be one of {sorted(k for k in _ops.ACTIVATIONS if k)}, got {activation!r}.")
    m, k, n = A.rows, A.k, B.rows
    if B.k != k:
        raise ValueError(f"A and B must share K, got {k} and {B.k}.")
    if n % 8 != 0 or k % 32 != 0 or k == 0:
        raise ValueError(f"N must be a multiple of 8 and K a positive multiple of 32, got N = {n}, K = {k}.")
    dev = _ops._require_cuda(A.packed, "A")
    if B.device != A.device:
        raise ValueError(f"B must be on device {A.device}, got {B.device}.")
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=A.device)
    elif tuple(out.shape) != (m, n) or out.dtype != torch.bfloat16 or out.device != A.device:
        raise ValueError(f"out must be a bfloat16 tensor of shape {(m, n)} on {A.device}.")
    if bias is not None and (bias.dtype != torch.bfloat16 or tuple(bias.shape) != (n,) or bias.device != A.device):
        raise ValueError(f"bias must be a bfloat16 tensor of shape ({n},) on {A.device}.")
    if m == 0 or n == 0:
        return out
    A, B = _ops.to_tiled(A), _ops.to_tiled(B)
    with torch.cuda.device(dev):
        S.init(dev)
        need = S.workspace_bytes(m, n, k, A.fmt, variant, dev)
        ws = None
        if need > 0:
            ws = _ops._workspaces.get(dev)
            if ws is None or ws.numel() < need:
                ws = torch.zeros((need,), dtype=torch.uint8, device=A.device)
                _ops._workspaces[dev] = ws
        S.gemm(_p(A.packed), _p(A.scales), _p(A.global_scale), _p(B.packed), _p(B.scales), _p(B.global_scale), _p(out), m, n, k,
               out.stride(0), A.fmt, variant, _p(ws), 0 if ws is None else ws.numel(), torch.cuda.current_stream(A.device).cuda_stream,
               _p(bias), _ops.ACTIVATIONS[activation])
    return out
