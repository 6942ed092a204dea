"""The reference operator itself on B200: ``gemm_pipeline_transposed_b(A, B, out=None)``.

Same name, argument meaning, validation style and error behaviour as
python/avelang_kernels/amdgpu_gemm.py:458-494 (bf16 A (M, K) and B (N, K), K contiguous,
``out = A @ B.T`` with fp32 accumulation, bf16 result, ``ValueError`` on bad dtype / shape / ``out``),
served by the same TMA + tcgen05 pipeline as the FP4 kernels in dense bf16 mode
(``tcgen05.mma kind::f16``).  Differences, both deliberate: the result is rounded to nearest even
instead of truncated (amdgpu_gemm.py:322-328 truncates), which is what the reference's own oracle
``(A.float() @ B.float().T).to(torch.bfloat16)`` does; and M, N need not be multiples of 128
(edges are zero-filled on load and clipped on store) -- only K % 8 and N % 8 are required.

The argument checks and their messages follow the reference operator (causalflow-ai/avelang,
python/avelang_kernels/amdgpu_gemm.py, Apache-2.0) so that callers see the same errors.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .fp4_gemm import GEMM_AUTO

GROUP_K = 8
GROUP_N = 8


def gemm_pipeline_transposed_b(
    A: torch.Tensor,
    B: torch.Tensor,
    out: torch.Tensor | None = None,
    variant: int = GEMM_AUTO,
) -> torch.Tensor:
    if A.dtype != torch.bfloat16:
        raise ValueError(f"A must have dtype torch.bfloat16, got {A.dtype}.")
    if B.dtype != torch.bfloat16:
        raise ValueError(f"B must have dtype torch.bfloat16, got {B.dtype}.")
    if A.dim() != 2 or B.dim() != 2:
        raise ValueError(f"A and B must be 2-D, got shapes {tuple(A.shape)} and {tuple(B.shape)}.")
    m = A.shape[0]
    k = A.shape[1]
    n = B.shape[0]
    if B.shape[1] != k:
        raise ValueError(f"A and B must share K, got {k} and {B.shape[1]}.")
    if n % GROUP_N != 0:
        raise ValueError(f"N must be a multiple of {GROUP_N}, got {n}.")
    if k % GROUP_K != 0 or k == 0:
        raise ValueError(f"K must be a positive multiple of {GROUP_K}, got {k}.")
    if not A.is_cuda:
        raise ValueError(f"A must be a CUDA tensor, got device {A.device}.")
    if B.device != A.device:
        raise ValueError(f"B must be on device {A.device}, got {B.device}.")
    if not A.is_contiguous() or not B.is_contiguous():
        raise ValueError("A and B must be contiguous (K-major).")

    out_shape = (m, n)
    if out is None:
        out = torch.empty(out_shape, dtype=torch.bfloat16, device=A.device)
    elif tuple(out.shape) != out_shape:
        raise ValueError(f"out must have shape {out_shape}, got {tuple(out.shape)}.")
    elif out.dtype != torch.bfloat16:
        raise ValueError(f"out must have dtype torch.bfloat16, got {out.dtype}.")
    elif out.device != A.device:
        raise ValueError(f"out must be on device {A.device}, got {out.device}.")
    if m == 0 or n == 0:
        return out
    if out.stride(1) != 1 or out.stride(0) % 8 != 0 or out.data_ptr() % 16 != 0:
        raise ValueError("out must be row-major with a row stride that is a multiple of 8 elements and 16-byte aligned.")

    dev = A.device.index if A.device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(dev):
        L = _lib.ensure_init(dev)
        stream = ctypes.c_void_p(torch.cuda.current_stream(A.device).cuda_stream)
        _lib.check(L.ave_bf16_gemm(ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(B.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                   m, n, k, out.stride(0), variant, stream))
    return out
