#!/usr/bin/env python3
"""FP4 GEMM benchmark driver.

Mirrors the reference driver benchmark/gemm/bench_amdgpu_gemm.py:23-84 -- same flags
(--m --n --k --warmup --repeat --iters --validate), same method (warm-up calls, one call
captured in a CUDA graph, events around repeat x iters replays, flops = 2*M*N*K, one
printed key=value line, optional validation with max-abs printed) -- for the block-scaled
FP4 operators, and adds --format, --seed, --variant, --rotate and --no-graph.

The bf16 mode's driver (flags, print format, validation block) follows the reference script
(causalflow-ai/avelang, benchmark/gemm/bench_amdgpu_gemm.py, Apache-2.0).

Validation uses the CPU oracle (dequantise E2M1 x scale, fp32 matmul, bf16 round) on the same
quantised operands; it is meant for sizes the CPU finishes in seconds.
"""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import avelang_b200 as ave  # noqa: E402
from avelang_b200 import inputs  # noqa: E402

NOMINAL_FP4_TFLOPS = 9000.0
NOMINAL_HBM_GBS = 8000.0


def _ensure_b200():
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA is not available.")
    if torch.cuda.get_device_capability()[0] != 10:
        raise RuntimeError("The FP4 GEMM benchmark requires an sm_100 (B200) device.")


def _validate_shape(m, n, k):
    if k % 32 != 0 or k <= 0:
        raise ValueError(f"K must be a positive multiple of 32, got {k}.")
    if n % 8 != 0:
        raise ValueError(f"N must be a multiple of 8, got {n}.")
    if m <= 0:
        raise ValueError(f"M must be positive, got {m}.")


def run_fp4_gemm_benchmark(m, n, k, warmup, repeat, iters, validate, fmt="nvfp4", seed=0, variant=0, rotate=1,
                           use_graph=True, a_kind="normal", b_kind="normal"):
    _ensure_b200()
    _validate_shape(m, n, k)
    dev = torch.device("cuda")
    if fmt == "bf16":
        return run_bf16_gemm_benchmark(m, n, k, warmup, repeat, iters, validate, seed, variant, use_graph)
    quant = ave.quantize_nvfp4 if fmt == "nvfp4" else ave.quantize_mxfp4
    gemm = ave.gemm_nvfp4_transposed_b if fmt == "nvfp4" else ave.gemm_mxfp4_transposed_b
    blk = 16 if fmt == "nvfp4" else 32

    sets = []
    for r in range(rotate):
        a = inputs.make_operand_bf16(a_kind, m, k, seed + 2 * r).to(dev)
        b = inputs.make_operand_bf16(b_kind, n, k, seed + 2 * r + 1).to(dev)
        sets.append((quant(a, sf_layout=ave.SF_ROW_MAJOR), quant(b, sf_layout=ave.SF_ROW_MAJOR)))
        del a, b
    tiled = [(ave.to_tiled(A), ave.to_tiled(B)) for A, B in sets]
    C = torch.zeros((m, n), dtype=torch.bfloat16, device=dev)

    def one_pass():
        for A, B in tiled:
            gemm(A, B, out=C, variant=variant)

    for _ in range(warmup):
        one_pass()
    torch.cuda.synchronize()

    if use_graph:
        graph = torch.cuda.CUDAGraph()
        capture_stream = torch.cuda.Stream()
        with torch.cuda.graph(graph, stream=capture_stream):
            one_pass()
        torch.cuda.synchronize()
        replay = graph.replay
    else:
        replay = one_pass

    start_evt = torch.cuda.Event(enable_timing=True)
    end_evt = torch.cuda.Event(enable_timing=True)
    start_evt.record()
    for _ in range(repeat):
        for _ in range(iters):
            replay()
    end_evt.record()
    torch.cuda.synchronize()
    ave.check_device_status(dev)
    elapsed = (start_evt.elapsed_time(end_evt) * 1.0e-3) / (repeat * iters * rotate)

    flops = 2.0 * m * n * k
    tflops = flops / elapsed / 1.0e12
    bytes_moved = m * k // 2 + n * k // 2 + (m + n) * (k // blk) + 2 * m * n
    bandwidth = bytes_moved / elapsed / 1.0e9
    print(f"M={m} N={n} K={k} format={fmt} variant={variant} time_ms={elapsed * 1.0e3:.4f} tflops={tflops:.3f} "
          f"bandwidth_gbs={bandwidth:.3f} pct_fp4_peak={100.0 * tflops / NOMINAL_FP4_TFLOPS:.2f} "
          f"pct_hbm_8tbs={100.0 * bandwidth / NOMINAL_HBM_GBS:.2f}")

    if validate:
        import numpy as np

        from oracle import fp4_oracle as O

        A, B = sets[-1]
        ofmt = O.NVFP4 if fmt == "nvfp4" else O.MXFP4

        def host(op):
            gs = float(op.global_scale.item()) if op.global_scale is not None else 1.0
            return op.packed.cpu().numpy(), op.scales.cpu().numpy(), gs

        d32, dbf = O.c_gemm_fp4(host(A), host(B), ofmt)
        expected = O.bf16_bits_to_f32(dbf)
        actual = C.float().cpu().numpy()
        max_abs = float(np.abs(actual - expected).max())
        rel_fro = float(np.linalg.norm(actual - expected) / (np.linalg.norm(expected) or 1.0))
        rel_fro_f32 = float(np.linalg.norm(actual - d32) / (np.linalg.norm(d32) or 1.0))
        if not rel_fro <= 1e-3:
            raise AssertionError(f"Validation failed (rel_fro {rel_fro:.3e}, max abs diff {max_abs}).")
        print(f"validation=max_abs_diff:{max_abs:.6f} rel_fro:{rel_fro:.3e} rel_fro_vs_fp32:{rel_fro_f32:.3e}")
    return elapsed


def run_bf16_gemm_benchmark(m, n, k, warmup, repeat, iters, validate, seed=0, variant=0, use_graph=True):
    """The reference operator on B200, measured exactly as benchmark/gemm/bench_amdgpu_gemm.py:23-68 does."""
    from avelang_b200.bf16_gemm import gemm_pipeline_transposed_b

    torch.manual_seed(seed)
    A = torch.randn((m, k), dtype=torch.bfloat16, device="cuda")
    B = torch.randn((n, k), dtype=torch.bfloat16, device="cuda")
    C = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    for _ in range(warmup):
        gemm_pipeline_transposed_b(A, B, out=C, variant=variant)
    torch.cuda.synchronize()
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        capture_stream = torch.cuda.Stream()
        with torch.cuda.graph(graph, stream=capture_stream):
            gemm_pipeline_transposed_b(A, B, out=C, variant=variant)
        torch.cuda.synchronize()
        replay = graph.replay
    else:
        def replay():
            gemm_pipeline_transposed_b(A, B, out=C, variant=variant)
    start_evt = torch.cuda.Event(enable_timing=True)
    end_evt = torch.cuda.Event(enable_timing=True)
    start_evt.record()
    for _ in range(repeat):
        for _ in range(iters):
            replay()
    end_evt.record()
    torch.cuda.synchronize()
    ave.check_device_status(torch.device("cuda"))
    elapsed = (start_evt.elapsed_time(end_evt) * 1.0e-3) / (repeat * iters)
    flops = 2.0 * m * n * k
    tflops = flops / elapsed / 1.0e12
    bytes_moved = (m * k + k * n + m * n) * 2
    bandwidth = bytes_moved / elapsed / 1.0e9
    print(f"M={m} N={n} K={k} format=bf16 variant={variant} time_ms={elapsed * 1.0e3:.4f} tflops={tflops:.3f} bandwidth_gbs={bandwidth:.3f}")
    if validate:
        expected = (A.float().cpu() @ B.float().cpu().T).to(dtype=torch.bfloat16)
        actual = C.to("cpu")
        max_abs = torch.max(torch.abs(actual - expected)).item()
        if not torch.allclose(actual, expected, rtol=1e-1, atol=1e-1):
            raise AssertionError(f"Validation failed (max abs diff {max_abs}).")
        print(f"validation=max_abs_diff:{max_abs:.6f}")
    return elapsed


def main():
    parser = argparse.ArgumentParser(description="Block-scaled FP4 GEMM benchmark (K multiple of 32, N multiple of 8)")
    parser.add_argument("--m", type=int, default=1024)
    parser.add_argument("--n", type=int, default=1024)
    parser.add_argument("--k", type=int, default=1024)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--repeat", type=int, default=100)
    parser.add_argument("--iters", type=int, default=100, help="Graph replays per timing repeat")
    parser.add_argument("--validate", action="store_true", default=False)
    parser.add_argument("--format", choices=["nvfp4", "mxfp4", "bf16"], default="nvfp4")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--variant", type=int, default=0, help="kernel variant (0 = chosen by shape)")
    parser.add_argument("--rotate", type=int, default=1, help="operand sets cycled per pass (use >1 to defeat L2 reuse)")
    parser.add_argument("--no-graph", action="store_true", help="plain launches instead of CUDA graph replays")
    parser.add_argument("--a-kind", default="normal", choices=["normal", "weight", "outlier", "student_t3"])
    parser.add_argument("--b-kind", default="normal", choices=["normal", "weight", "outlier", "student_t3"])
    args = parser.parse_args()
    run_fp4_gemm_benchmark(args.m, args.n, args.k, args.warmup, args.repeat, args.iters, args.validate, args.format,
                           args.seed, args.variant, args.rotate, not args.no_graph, args.a_kind, args.b_kind)


if __name__ == "__main__":
    main()
