#!/usr/bin/env python3
"""K-sharded (row-parallel) FP4 linear layer on one box: GEMM on this rank's K-slice + reduce-scatter of the rows.

Launch with torchrun, one rank per GPU:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmark/gemm/bench_row_parallel.py --m 8192 --n 8192 --k-per-rank 8192
Weak scaling in K: every rank holds a (m, k_per_rank) activation slice and a (n, k_per_rank) weight slice and ends
with m / N rows of the bf16 result.  Two exchanges are timed: the fused one (the epilogue stores fp32 partial tiles
straight into the owner's staging buffer over NVLink, then a slab reduction) and local partials + NCCL reduce-scatter.
Timing: CUDA events on the launching stream after warm-up, barrier on both sides, max over ranks.  The reference
has no multi-GPU code; the method follows its single-GPU driver benchmark/gemm/bench_amdgpu_gemm.py:31-52.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import avelang_b200 as ave  # noqa: E402
from avelang_b200 import inputs, sharded  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k-per-rank", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    m, n, k = args.m, args.n, args.k_per_rank
    A = ave.quantize_nvfp4(inputs.normal_bf16(m, k, 2 * rank).to(dev))
    W = ave.quantize_nvfp4(inputs.normal_bf16(n, k, 2 * rank + 1).to(dev))

    def timed(layer):
        def barrier():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
        for _ in range(args.warmup):
            layer.forward(A)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            layer.forward(A)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    fused_ms = timed(sharded.RowShardedFp4Linear(W, fused=True))
    nccl_ms = timed(sharded.RowShardedFp4Linear(W, fused=False))
    ave.check_device_status(dev)
    if rank == 0:
        flops = 2.0 * m * n * k * world
        link_bytes = 4.0 * m * n * (world - 1) / world           # fp32 partial rows leaving each GPU
        floor_ms = max(2.0 * m * n * k / 6.48e15, link_bytes / 770e9) * 1e3
        print(json.dumps({"workload": f"row_parallel_{m}x{n}x{k}_per_rank_nvfp4_x{world}", "n_gpus": world,
                          "fused_ms_per_step": round(fused_ms, 4), "nccl_ms_per_step": round(nccl_ms, 4),
                          "fused_tflops_whole_box": round(flops / fused_ms / 1e9, 1),
                          "nvlink_bytes_out_per_gpu": int(link_bytes), "floor_ms": round(floor_ms, 4),
                          "fraction_of_floor": round(floor_ms / fused_ms, 3)}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
