"""Seeded synthetic inputs for the benchmark configurations.

The reference benchmark draws unseeded ``torch.randn`` bf16 operands
(benchmark/gemm/bench_amdgpu_gemm.py:27-29) and its test seeds torch with 0
(test/examples/gemm/amdgpu/test_amdgpu_gemm.py:16).  Here every operand comes from a
CPU ``torch.Generator`` so the CPU oracle and the GPU see identical bits; values are
drawn in fp32 and cast to bf16.
"""
from __future__ import annotations

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def normal_bf16(rows: int, k: int, seed: int, std: float = 1.0) -> torch.Tensor:
    """N(0, std^2) as bf16 on the CPU."""
    x = torch.randn((rows, k), generator=_gen(seed), dtype=torch.float32)
    if std != 1.0:
        x = x * std
    return x.to(torch.bfloat16)


def outlier_activations_bf16(rows: int, k: int, seed: int, frac: float = 0.001, gain: float = 50.0) -> torch.Tensor:
    """N(0,1) activations with round(frac*k) channels (K columns, the same for every row) scaled by `gain`."""
    g = _gen(seed)
    x = torch.randn((rows, k), generator=g, dtype=torch.float32)
    n_out = max(1, int(round(frac * k)))
    cols = torch.randperm(k, generator=g)[:n_out]
    x[:, cols] *= gain
    return x.to(torch.bfloat16)


def student_t3_bf16(rows: int, k: int, seed: int) -> torch.Tensor:
    """Student-t with 3 degrees of freedom built from four seeded normal draws: z0 / sqrt((z1^2+z2^2+z3^2)/3)."""
    g = _gen(seed)
    z0 = torch.randn((rows, k), generator=g, dtype=torch.float32)
    s = torch.zeros((rows, k), dtype=torch.float32)
    for _ in range(3):
        z = torch.randn((rows, k), generator=g, dtype=torch.float32)
        s.addcmul_(z, z)
    return (z0 / torch.sqrt(s / 3.0)).to(torch.bfloat16)


# The five workloads (shapes, formats, distributions) the benchmark and the tests use.
CONFIGS = {
    "c0_oracle_128x256x512": dict(m=128, n=256, k=512, fmt="nvfp4", a="normal", b="normal"),
    "c1_square_8192": dict(m=8192, n=8192, k=8192, fmt="nvfp4", a="normal", b="normal"),
    "c2_decode_16x28672x8192": dict(m=16, n=28672, k=8192, fmt="nvfp4", a="outlier", b="weight"),
    "c3_prefill_8192x57344x8192": dict(m=8192, n=57344, k=8192, fmt="nvfp4", a="normal", b="normal"),
    "c4_mxfp4_16384": dict(m=16384, n=16384, k=16384, fmt="mxfp4", a="student_t3", b="weight"),
}


def make_operand_bf16(kind: str, rows: int, k: int, seed: int) -> torch.Tensor:
    if kind == "normal":
        return normal_bf16(rows, k, seed)
    if kind == "weight":
        return normal_bf16(rows, k, seed, std=0.02)
    if kind == "outlier":
        return outlier_activations_bf16(rows, k, seed)
    if kind == "student_t3":
        return student_t3_bf16(rows, k, seed)
    raise ValueError(f"unknown operand kind {kind!r}")
