#!/usr/bin/env python3
"""Benchmark of the FP4 hot path.

    python bench.py --gpus N --steps K --warmup W            (this repo's CUDA path)
    python bench.py --impl reference --gpus N --steps K ...  (the oracle's CPU path on the host cores)

One step = one pass of the hot path over one batch of synthetic input:

  N = 1   the square NVFP4 GEMM  D = A * B^T  at M = N = K = 8192 (bf16 out) on operands
          already quantised and resident in HBM.  Three operand sets are rotated so that the
          working set (3 x 72 MB operands + 128 MB output) exceeds the 126 MB L2.
  N > 1   the same per-GPU GEMM as one N-shard of an (8192, 8192*N, 8192) problem (weak scaling:
          per-GPU work fixed, activations replicated, weights split by output column), followed by the
          all-gather of the bf16 output over NVLink -- the one exchange step the sharded path has.

`value` is whole-job TFLOP/s (2*M*N*K per GPU per step, all ranks, divided by the slowest
rank's device time).  The K steps are repeated inside one CUDA-event pair until the timed region
is a few hundred milliseconds long, so that the clock samples taken during it mean something.
`e2e` is the same metric through the public operators with HOST buffers: each step copies the bf16
activations A from pinned host memory, quantises them on the device, multiplies with the resident
pre-quantised weights B and copies D back.

Besides the headline the line carries the other workloads of the path: `decode` (M = 16, N = 28672,
K = 8192, HBM-bound), `quantise` (bf16 -> NVFP4 / MXFP4 at 8192^2), `c4` (MXFP4 16384^3), `c3`
(8192 x 57344 x 8192 with N split over the ranks, at every N) and, at N > 1, a `parity` object: the
gathered result of the sharded step compared, on every rank, with the unsharded GEMM of every shard.

The driver of the reference benchmark (benchmark/gemm/bench_amdgpu_gemm.py:23-68: warm-up,
event timing, 2*M*N*K flops, validation inside the benchmark) is mirrored by
benchmark/gemm/bench_fp4_gemm.py; this file is the machine-readable contract around the same measurement.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "NVFP4 GEMM TFLOPS & % FP4 peak at 8192^3; decode-GEMM HBM GB/s"
M = N = K = 8192
C3_N = 57344
NOMINAL_FP4_TFLOPS = 9000.0      # NVIDIA B200 datasheet, dense FP4
NOMINAL_HBM_GBS = 8000.0         # figure the decode target is quoted against
FALLBACK_BF16_TFLOPS = 1590.0    # earlier measurement on this pool, used only if MEASURED_PEAKS.json is absent
FALLBACK_HBM_GBS = 6650.0
NVLINK_GBS_PER_DIR = 770.0       # measured peer copy per direction on this pool
MIN_TIMED_MS = 250.0             # the K steps are repeated until the timed region is at least this long
# dram__bytes_read.sum + dram__bytes_write.sum per launch, copied from the ncu captures summarised under profiles/
# (a capture cannot be taken inside a benchmark run; `traffic_source` in the line names the summary)
NCU_TRAFFIC = {
    "gemm_8192": (205_100_000, "profiles/choice_tile_shape_and_pipeline_depth.md, row 2-CTA 256x256 at 8192^3 (ncu, mean of two launches)"),
    "decode": (134_600_000, "profiles/choice_decode_burst_and_stream_k.md, row burst 4 with stream-K (ncu, mean of two launches)"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return dict(bf16=float(p["bf16_tflops"]), bf16_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    hbm=float(p["hbm_gbs"]), source="measured")
    except Exception:
        return dict(bf16=FALLBACK_BF16_TFLOPS, bf16_sustained=1400.0, hbm=FALLBACK_HBM_GBS, source="fallback")


def make_config(world: int, workload: str) -> dict:
    """The `config` object of the JSON line; both arms print the same one for the same command line."""
    c3 = (workload == "c3")
    n = (C3_N // world) if c3 else N
    if c3:
        name = f"c3_prefill_8192x57344x8192_nvfp4_n_sharded_x{world}"
    elif world == 1:
        name = "c1_square_nvfp4_8192"
    else:
        name = f"c1_per_gpu_slice_of_8192x{8192 * world}x8192_plus_allgather"
    return {"workload": name, "m": M, "n_per_gpu": n, "k": K, "world": world,
            "l2": "3 operand sets rotated; working set 3 x 72 MB + 2 x 128 MB output > 126 MB L2",
            "parallelism": (f"n-sharded x{world} + bf16 all-gather" if world > 1 else "single gpu")}


class ClockSampler:
    """Samples SM clock, power and throttle reasons while the timed region runs.

    Uses NVML in a background thread (a sample every few milliseconds); falls back to an
    `nvidia-smi -lms` child process when the NVML python binding is not importable.  Read-only queries.
    """

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []          # (sm_mhz, sm_max_mhz, power_w, [hw_slowdown, hw_thermal, sw_thermal, sw_power_cap])
        self.proc = None
        self.thread = None
        self._stop = False
        try:
            import threading

            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = gpu_index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if gpu_index < len(ids) and ids[gpu_index].isdigit():
                    phys = int(ids[gpu_index])
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            smax = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            R = pynvml

            def loop():
                while not self._stop:
                    try:
                        mhz = float(R.nvmlDeviceGetClockInfo(h, R.NVML_CLOCK_SM))
                        pw = R.nvmlDeviceGetPowerUsage(h) / 1000.0
                        rs = R.nvmlDeviceGetCurrentClocksEventReasons(h) if hasattr(R, "nvmlDeviceGetCurrentClocksEventReasons") \
                            else R.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                        flags = ["Active" if rs & m else "Not Active" for m in (
                            R.nvmlClocksThrottleReasonHwSlowdown, R.nvmlClocksThrottleReasonHwThermalSlowdown,
                            R.nvmlClocksThrottleReasonSwThermalSlowdown, R.nvmlClocksThrottleReasonSwPowerCap)]
                        self.rows.append((mhz, smax, pw, flags))
                    except Exception:
                        pass
                    time.sleep(0.002)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20", "-i", str(gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        rows = self.rows
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=2)
        elif self.proc is not None:
            self.proc.terminate()
            try:
                out, _ = self.proc.communicate(timeout=5)
            except Exception:
                self.proc.kill()
                out = ""
            for line in out.splitlines():
                parts = [x.strip() for x in line.split(",")]
                if len(parts) >= 7:
                    try:
                        rows.append((float(parts[0]), float(parts[1]), float(parts[2]), parts[3:7]))
                    except ValueError:
                        pass
        else:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source available"]}
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        pmax = max(r[2] for r in rows)
        busy = [r for r in rows if r[2] >= 0.6 * pmax] or rows
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in busy for i in range(4) if r[3][i].lower().startswith("active")})
        return {"sm_mhz": statistics.median(r[0] for r in busy), "sm_min_mhz": min(r[0] for r in busy),
                "sm_max_mhz": rows[0][1], "power_w_max": round(pmax, 1), "samples": len(busy), "samples_total": len(rows),
                "reasons": reasons, "source": "nvml" if self.thread is not None else "nvidia-smi"}


def bind_to_gpu_local_cpus(gpu_index: int):
    """Run this rank's threads on the CPUs NVML names as local to its GPU, so that the pinned host buffers it allocates
    afterwards sit on that NUMA node and the PCIe copies do not cross sockets (a process setting, not a GPU one).
    Returns the number of CPUs bound to, or None when NVML or the call is unavailable."""
    try:
        import pynvml

        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        phys = gpu_index
        if visible:
            ids = [v.strip() for v in visible.split(",") if v.strip()]
            if gpu_index < len(ids) and ids[gpu_index].isdigit():
                phys = int(ids[gpu_index])
        h = pynvml.nvmlDeviceGetHandleByIndex(phys)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1}
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return len(allowed)
    except Exception:
        return None


def dist_env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return world, rank, local


# ------------------------------------------------------------------------------------ ours
class Bench:
    """Shared state of one rank of the benchmark: device, process group, timing helpers, operand factories."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        import avelang_b200 as ave

        self.torch, self.dist, self.ave, self.args = torch, dist, ave, args
        self.world, self.rank, self.local = dist_env()
        if self.world != args.gpus and self.world != 1:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}")
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the FP4 path has no CPU fallback")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.cpu_affinity = None
        if self.world > 1 and args.bind_cpus:
            self.cpu_affinity = bind_to_gpu_local_cpus(self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.peaks = measured_peaks()
        self.launches = 0        # kernels of this library launched inside the headline timed region

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_true(self, ok: bool) -> bool:
        if self.world == 1:
            return bool(ok)
        t = self.torch.tensor([1 if ok else 0], dtype=self.torch.int32, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item())

    def timed(self, fn, steps: int, warmup: int, min_ms: float = 0.0):
        """Warm up, then time `steps` calls of fn(i), repeated so that the region lasts at least `min_ms`.
        Barrier + synchronize on both sides, CUDA events on the launching stream, max over ranks.
        Returns (ms per step, repeats)."""
        torch = self.torch
        for i in range(warmup):
            fn(i)
        reps = 1
        if min_ms > 0.0:
            self.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(steps):
                fn(i)
            e1.record()
            self.barrier()
            est = max(self.max_over_ranks(e0.elapsed_time(e1)), 1e-3)
            reps = max(1, min(4000, int(math.ceil(min_ms / est))))
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for i in range(steps):
                fn(i)
        e1.record()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1)) / (steps * reps), reps

    def operand(self, rows: int, k: int, seed: int, std: float = 1.0):
        """A seeded N(0, std) bf16 matrix generated on the device, quantised to NVFP4 (tensor scale from the data)."""
        torch = self.torch
        gen = torch.Generator(device=self.dev)
        gen.manual_seed(seed)
        x = torch.randn((rows, k), generator=gen, device=self.dev, dtype=torch.float32)
        if std != 1.0:
            x *= std
        x = x.to(torch.bfloat16)
        return self.ave.quantize_nvfp4(x), x


def weight_seed(rank: int, i: int) -> int:
    return 100_000 + 1000 * rank + i


def act_seed(i: int) -> int:
    return 7_000 + i


def sharded_block(B: Bench, n_local: int, R: int, steps: int, warmup: int, min_ms: float, tag: str, keep_host_a: bool = False):
    """One N-sharded workload on this rank: R operand sets (activations identical on every rank, weights per rank),
    the parity check of the gathered result, and the timings (fused step, GEMM only, NCCL all-gather only)."""
    torch, ave, dist = B.torch, B.ave, B.dist
    from avelang_b200 import sharded

    world, rank, dev = B.world, B.rank, B.dev
    A_ops, B_ops, host_a = [], [], []
    for i in range(R):
        a_op, a = B.operand(M, K, act_seed(i))                      # replicated activations: same seed on every rank
        b_op, b = B.operand(n_local, K, weight_seed(rank, i))       # this rank's rows of the weight
        A_ops.append(a_op)
        B_ops.append(b_op)
        if keep_host_a and i < 2:
            host_a.append(a.cpu().pin_memory())
        del a, b
    torch.cuda.synchronize(dev)
    res = {"A": A_ops, "B": B_ops, "host_a": host_a}
    outs = [torch.empty((M, n_local), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    res["outs"] = outs

    def gemm_only(i: int):
        ave.gemm_nvfp4_transposed_b(A_ops[i % R], B_ops[i % R], out=outs[i % 2])

    if world == 1:
        ms, reps = B.timed(gemm_only, steps, warmup, min_ms)
        res.update(step_ms=ms, gemm_ms=ms, reps=reps, ag_ms=None, layers=None, parity=None)
        return res

    fused = not B.args.nccl_allgather
    layers = [sharded.ShardedFp4Linear(B_ops[i], fused=fused) for i in range(R)]
    res["layers"] = layers

    # ---- parity, before any timing: the gathered result of the sharded step (the data plane every number below
    # uses) must equal, bit for bit, the unsharded GEMM of the same activations with every rank's shard, which
    # each rank regenerates from the shard's seed.  The NCCL form of the exchange is checked the same way once.
    parity = {"what": "every rank compares each peer's slab of the gathered (world, M, N/world) result with its own "
                      "single-GPU GEMM on that peer's regenerated weight shard (bit-equal)"}
    g = layers[0].forward(A_ops[0])
    B.barrier()
    ok_fused = True
    mism = 0
    for p in range(world):
        wp = B_ops[0] if p == rank else B.operand(n_local, K, weight_seed(p, 0))[0]
        want = ave.gemm_nvfp4_transposed_b(A_ops[0], wp, out=outs[0])
        torch.cuda.synchronize(dev)
        eq = bool(torch.equal(g[p], want))
        if not eq:
            mism += int((g[p] != want).sum().item())
        ok_fused = ok_fused and eq
        del wp
    second = layers[0].forward(A_ops[0]).clone()     # the buffer is reused: a second step must give the same bits
    B.barrier()
    ok_fused = ok_fused and bool(torch.equal(second, g))
    other = sharded.ShardedFp4Linear(B_ops[0], fused=not fused)
    g2 = other.forward(A_ops[0])
    B.barrier()
    ok_other = bool(torch.equal(g2, second))
    del other, g2, second
    parity["gathered_equals_unsharded"] = B.all_true(ok_fused)
    parity["fused_equals_nccl_allgather"] = B.all_true(ok_other)
    parity["exchange_checked"] = "fused peer stores" if fused else "nccl"
    parity["mismatching_elements_this_rank"] = mism
    parity["ranks"] = world
    res["parity"] = parity
    B.barrier()

    def step(i: int):
        layers[i % R].forward(A_ops[i % R])

    res["step_ms"], res["reps"] = B.timed(step, steps, warmup, min_ms)
    res["gemm_ms"], _ = B.timed(gemm_only, steps, 3, min_ms / 4)
    gath = torch.empty((world, M, n_local), dtype=torch.bfloat16, device=dev)

    def ag(i):
        dist.all_gather_into_tensor(gath.view(-1, n_local), gath[rank])
    res["ag_ms"], _ = B.timed(ag, max(5, steps // 2), 3, 0.0)
    del gath
    res["fused"] = fused
    return res


def nvlink_roofline(world: int, n_local: int, fp4_peak: float, step_ms: float, gemm_ms: float, ag_ms: float, fused: bool) -> dict:
    flops = 2.0 * M * n_local * K
    link_bytes = 2.0 * M * n_local * (world - 1)          # bf16 bytes each GPU must send, and receive
    t_flop = flops / (fp4_peak * 1e12)
    t_link = link_bytes / (NVLINK_GBS_PER_DIR * 1e9)
    return {
        "target_ms": round(max(t_flop, t_link) * 1e3, 4), "achieved_ms": round(step_ms, 4),
        "frac": round(max(t_flop, t_link) * 1e3 / step_ms, 4), "bound": "nvlink" if t_link > t_flop else "tensor",
        "exchange": "fused into the GEMM epilogue (peer stores) + device barrier" if fused else "NCCL all-gather after the GEMM",
        "gemm_only_ms": round(gemm_ms, 4), "nccl_allgather_only_ms": round(ag_ms, 4),
        "unfused_gemm_plus_nccl_ms": round(gemm_ms + ag_ms, 4),
        "gemm_only_tflops_per_gpu": round(flops / (gemm_ms * 1e-3) / 1e12, 1),
        "nvlink_bytes_in_per_gpu": int(link_bytes),
        "nvlink_ingress_gbs": round(link_bytes / (step_ms * 1e-3) / 1e9, 1),
        "allgather_busbw_gbs": round(link_bytes / (ag_ms * 1e-3) / 1e9, 1),
    }


def run_ours(args) -> dict:
    B = Bench(args)
    torch, ave, dist = B.torch, B.ave, B.dist
    world, rank, local, dev, peaks = B.world, B.rank, B.local, B.dev, B.peaks
    c3_headline = (args.workload == "c3")
    n_local = (C3_N // world) if c3_headline else N
    R = 3  # operand sets rotated so that consecutive steps do not hit L2-resident operands
    warmup = max(args.warmup, 3)
    fp4_peak = 4.0 * peaks["bf16"]

    sampler = ClockSampler(local) if rank == 0 else None
    head = sharded_block(B, n_local, R, args.steps, warmup, args.min_timed_ms, "headline", keep_host_a=True)
    clocks = sampler.stop() if sampler else None
    ave.check_device_status(dev)
    A_ops, B_ops, outs, layers, host_a = head["A"], head["B"], head["outs"], head["layers"], head["host_a"]
    ms_per_step, gemm_ms = head["step_ms"], head["gemm_ms"]
    flops_per_gpu = 2.0 * M * n_local * K
    value = world * flops_per_gpu / (ms_per_step * 1e-3) / 1e12
    gemm_tflops = flops_per_gpu / (gemm_ms * 1e-3) / 1e12

    # The kernel is timed inside a region of several hundred milliseconds, so the denominator is the SUSTAINED
    # figure of the measured peaks (the burst one applies to a kernel timed alone); both fractions are in the line.
    fp4_peak_sustained = 4.0 * peaks["bf16_sustained"]
    roofline = {
        "bound": "tensor", "kernel": "gemm_fp4_kernel<2-CTA, 256x256x256>", "achieved": round(gemm_tflops, 1),
        "peak": round(fp4_peak_sustained, 1), "unit": "TFLOP/s", "frac": round(gemm_tflops / fp4_peak_sustained, 4),
        "peak_source": (f"4 x cuBLAS bf16 sustained ({peaks['bf16_sustained']:.0f} TF, {peaks['source']}; the kernel is timed inside a "
                        f">= {MIN_TIMED_MS:.0f} ms loop under the power cap): FP4 issues at 4x the bf16 rate"),
        "frac_of_nominal_9000": round(gemm_tflops / NOMINAL_FP4_TFLOPS, 4),
        "frac_of_4x_burst_bf16": round(gemm_tflops / fp4_peak, 4),
        "algorithmic_bytes": M * K // 2 + n_local * K // 2 + (M + n_local) * K // 16 + 2 * M * n_local,
        "traffic": NCU_TRAFFIC["gemm_8192"][0] if n_local == N else None,
        "traffic_source": NCU_TRAFFIC["gemm_8192"][1] if n_local == N else None,
        "launch_us": round(gemm_ms * 1e3, 2),
    }
    if world > 1:
        roofline["fused_step"] = nvlink_roofline(world, n_local, fp4_peak, ms_per_step, gemm_ms, head["ag_ms"], head["fused"])

    # ---- SM clock the GEMM really ran at: CTA 0 stamps clock64() through the library's trace hook
    # during the last launch of a back-to-back burst; cycles / event time = effective MHz.
    try:
        import ctypes

        from avelang_b200 import _lib
        L = _lib.ensure_init(local)
        cap = 2048
        tbuf = torch.zeros((3 * cap * 4,), dtype=torch.int64, device=dev)
        _lib.check(L.ave_fp4_set_trace(ctypes.c_void_p(tbuf.data_ptr()), tbuf.numel() * 8))
        for i in range(30):
            ave.gemm_nvfp4_transposed_b(A_ops[i % R], B_ops[i % R], out=outs[i % 2])
        t0e, t1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0e.record()
        ave.gemm_nvfp4_transposed_b(A_ops[0], B_ops[0], out=outs[0])
        t1e.record()
        torch.cuda.synchronize(dev)
        _lib.check(L.ave_fp4_set_trace(None, 0))
        tr = tbuf.cpu().view(3, cap, 4)
        first = int(tr[0, 0, 0])
        last = int(tr[2, :, 3].max())
        if clocks is not None and first > 0 and last > first:
            mhz = (last - first) / (t0e.elapsed_time(t1e) * 1e3)
            clocks["sm_mhz_in_kernel"] = round(mhz, 1)
            clocks["sm_mhz_in_kernel_how"] = "clock64 span of CTA 0 / CUDA-event time of the last of 31 back-to-back launches"
            roofline["fp4_ceiling_at_in_kernel_clock_tflops"] = round(32768 * ave_sm_count(L) * mhz * 1e6 / 1e12, 1)
        del tbuf
    except Exception as exc:
        if clocks is not None:
            clocks["sm_mhz_in_kernel"] = None
            clocks["sm_mhz_in_kernel_error"] = repr(exc)

    e2e = e2e_block(B, head, n_local, R, args)
    fp4_gather = None
    if world > 1 and not args.skip_fp4_gather:
        try:
            fp4_gather = fp4_gather_block(B, head, n_local, R, args, fp4_peak)
        except Exception as exc:
            fp4_gather = {"error": repr(exc)[:300]}
        B.barrier()

    cfg = make_config(world, args.workload)
    out = {
        "metric": METRIC, "value": round(value, 1), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
        "scaling": "strong" if c3_headline else "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3 block scale, fp32 accumulate, bf16 out)", "data": "synthetic",
        "config": cfg, "roofline": roofline, "e2e": e2e, "gpu_launches": args.steps * head["reps"], "clocks": clocks,
        "pct_of_nominal_fp4_peak": round(100.0 * value / world / NOMINAL_FP4_TFLOPS, 2),
        "timed_repeats": head["reps"], "timed_region_ms": round(ms_per_step * args.steps * head["reps"], 1),
        "timed_region": (f"{args.steps} steps x {head['reps']} repeats inside one CUDA-event pair (>= {args.min_timed_ms:.0f} ms), "
                         "barrier + synchronize on both sides, max over ranks"),
    }
    if world > 1:
        out["exchange"] = "fused peer stores" if head["fused"] else "nccl"
        out["cpus_bound_per_rank"] = B.cpu_affinity
    if head["parity"] is not None:
        out["parity"] = head["parity"]
    if fp4_gather is not None:
        out["fp4_gather"] = fp4_gather

    # free the headline's buffers before the side workloads
    del head, A_ops, B_ops, outs, layers, host_a
    torch.cuda.empty_cache()

    def side(name, fn):
        try:
            out[name] = fn()
        except Exception as exc:  # keep the headline line even if a side measurement fails
            out[name] = {"error": repr(exc)[:300]}
        B.barrier()

    if not c3_headline and not args.skip_c3:
        side("c3", lambda: c3_block(B, fp4_peak, args))
    if world > 1 and not args.skip_ksharded:
        side("k_sharded", lambda: ksharded_block(B, fp4_peak, args))
    if world == 1:
        if not args.skip_decode:
            side("decode", lambda: decode_bench(ave, torch, dev, peaks))
        if not args.skip_quantise:
            side("quantise", lambda: quantise_bench(ave, torch, dev, peaks))
        if not args.skip_c4:
            side("c4", lambda: c4_bench(B, fp4_peak))
        if not args.skip_context:
            side("context", lambda: library_context(B))
        if not args.skip_cpu_baseline and rank == 0:
            try:
                out["cpu_baseline"] = cpu_baseline(full=not args.cpu_sample, sample_rows=args.cpu_rows)
            except Exception as exc:
                out["cpu_baseline"] = {"error": repr(exc)[:300]}
    ave.check_device_status(dev)
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def ave_sm_count(L) -> int:
    n = int(L.ave_fp4_sm_count())
    return n if n > 0 else 148


def e2e_block(B: Bench, head: dict, n_local: int, R: int, args) -> dict:
    """End to end through the public operators with host buffers.  Every step copies its activations from pinned
    host memory, quantises, multiplies (N > 1: sharded GEMM + fused all-gather) and copies this rank's result slab
    back to pinned host memory.  Copy-in, compute and copy-out of consecutive steps run on three streams
    (double-buffered), so the PCIe link carries input and output at the same time; every step still does all of
    its copies inside the timed region.  N > 1: the activations are uploaded once per box -- every rank copies
    1/N of the rows from host and the ranks all-gather them over NVLink."""
    torch, ave, dist = B.torch, B.ave, B.dist
    from avelang_b200 import sharded

    world, rank, dev = B.world, B.rank, B.dev
    B_ops, outs, host_a = head["B"], head["outs"], head["host_a"]
    # enough steps for the three-stage pipeline's fill and drain (one copy-in and one copy-out, ~5 ms, both inside the
    # timed region) not to dominate: 10 steps read 9 % low
    e2e_steps = max(40, 2 * args.steps)
    s_in, s_comp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    a_buf = [torch.empty((M, K), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    h_buf = [torch.empty((M, n_local), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    rows = M // world
    if world > 1:
        # one result buffer per pipeline slot, so that a slab can be copied out while the next step computes
        e_layers = [sharded.ShardedFp4Linear(B_ops[b], fused=head["fused"]) for b in range(2)]
        my_rows = [h[rank * rows:(rank + 1) * rows] for h in host_a]

    def e2e_step(i: int):
        b = i % 2
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_comp[b])                 # the quantise that read a_buf[b] two steps ago is done
            if world == 1:
                a_buf[b].copy_(host_a[i % len(host_a)], non_blocking=True)
            else:
                mine = a_buf[b][rank * rows:(rank + 1) * rows]
                mine.copy_(my_rows[i % len(my_rows)], non_blocking=True)
                dist.all_gather_into_tensor(a_buf[b], mine)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(ev_in[b])
            s_comp.wait_event(ev_out[b])                # the result buffer of this slot has been copied out
            q = ave.quantize_nvfp4(a_buf[b])
            if world == 1:
                d = ave.gemm_nvfp4_transposed_b(q, B_ops[i % R], out=outs[b])
            else:
                d = e_layers[b].forward(q)[rank]
            ev_comp[b].record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b])
            h_buf[b].copy_(d, non_blocking=True)
            ev_out[b].record(s_out)

    def timed_e2e(steps: int, warmup: int) -> float:
        cur = torch.cuda.current_stream(dev)
        for i in range(warmup):
            e2e_step(i)
        B.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(cur)
        for st in (s_in, s_comp, s_out):
            st.wait_event(e0)
        for i in range(steps):
            e2e_step(i)
        for st in (s_in, s_comp, s_out):
            cur.wait_stream(st)
        e1.record(cur)
        B.barrier()
        return B.max_over_ranks(e0.elapsed_time(e1))

    e2e_ms = timed_e2e(e2e_steps, 4) / e2e_steps
    flops_per_gpu = 2.0 * M * n_local * K
    what = ("pinned host bf16 A -> device, amax + NVFP4 quantise, GEMM with resident pre-quantised B, bf16 D -> pinned host; "
            "copy-in, compute and copy-out of consecutive steps overlap on three streams")
    if world > 1:
        what = (f"every rank: 1/{world} of the rows of pinned host bf16 A -> device, NCCL all-gather of A over NVLink, amax + NVFP4 "
                "quantise, sharded GEMM + all-gather of D, this rank's bf16 slab of D -> pinned host; three streams, double-buffered")
    return {"value": round(world * flops_per_gpu / (e2e_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
            "h2d_bytes_per_step": 2 * M * K, "d2h_bytes_per_step": 2 * M * n_local * world,
            "h2d_bytes_per_step_per_rank": 2 * M * K // world, "d2h_bytes_per_step_per_rank": 2 * M * n_local,
            "ms_per_step": round(e2e_ms, 4), "steps": e2e_steps, "what": what}


def fp4_gather_block(B: Bench, head: dict, n_local: int, R: int, args, fp4_peak: float) -> dict:
    """The same sharded layer gathering its output as the NEXT layer's NVFP4 operand: the GEMM epilogue quantises
    its tile and stores packed bytes + scale bytes into every rank's copy (0.5625 byte per element over NVLink
    instead of 2).  Checked against the quantise kernel applied to the gathered bf16 result, then timed."""
    torch, ave = B.torch, B.ave
    from avelang_b200 import sharded

    world, dev = B.world, B.dev
    A_ops, B_ops, layers = head["A"], head["B"], head["layers"]
    n_total = n_local * world
    g = layers[0].forward(A_ops[0])
    B.barrier()
    full = sharded.columns_view(g).reshape(M, n_total)          # the gathered bf16 result as one (M, N) matrix
    gs = (full.abs().max().float() / 2688.0).reshape(1)         # static tensor scale of the output, same on every rank
    want = ave.quantize_nvfp4(full, global_scale=gs)
    qlayers = [sharded.ShardedFp4LinearQuantizedOut(B_ops[i], out_global_scale=gs) for i in range(2)]
    op = qlayers[0].forward(A_ops[0])
    B.barrier()
    ok = bool(torch.equal(op.packed, want.packed)) and bool(torch.equal(op.scales, want.scales))
    ok = B.all_true(ok)
    del full, want
    B.barrier()

    def step(i: int):
        qlayers[i % 2].forward(A_ops[i % R])

    ms, _ = B.timed(step, args.steps, 3, 60.0)
    ave.check_device_status(dev)
    flops = 2.0 * M * n_local * K
    link_bytes = M * n_local * (0.5 + 1.0 / 16.0) * (world - 1)
    t_flop = flops / (fp4_peak * 1e12)
    t_link = link_bytes / (NVLINK_GBS_PER_DIR * 1e9)
    return {"what": "GEMM with quantising epilogue + peer stores of the packed bytes and scale bytes (the next layer's NVFP4 "
                    "operand is gathered instead of the bf16 matrix) + device barrier",
            "parity_gathered_operand_equals_quantise_of_gathered_bf16": ok,
            "step_ms": round(ms, 4), "whole_job_tflops": round(world * flops / (ms * 1e-3) / 1e12, 1),
            "nvlink_bytes_in_per_gpu": int(link_bytes), "nvlink_ingress_gbs": round(link_bytes / (ms * 1e-3) / 1e9, 1),
            "target_ms": round(max(t_flop, t_link) * 1e3, 4), "frac": round(max(t_flop, t_link) * 1e3 / ms, 4),
            "bound": "nvlink" if t_link > t_flop else "tensor", "bf16_gather_step_ms": round(head["step_ms"], 4)}


def ksharded_block(B: Bench, fp4_peak: float, args) -> dict:
    """The other split of a linear layer: K-sharded (row-parallel) GEMM + reduce-scatter, M = N = 8192 and K = 8192 per
    rank.  The fused form (fp32 partial tiles stored by the epilogue straight into the owner's staging buffer, then a slab
    sum) is checked, bit for bit, against the same arithmetic done on this GPU alone with every rank's regenerated
    operands, and against local partials + NCCL reduce-scatter; then both forms are timed."""
    torch, ave = B.torch, B.ave
    from avelang_b200 import fp4_gemm, sharded

    world, rank, dev = B.world, B.rank, B.dev
    rows = M // world

    def operands(r):
        return B.operand(M, K, 300_000 + r)[0], B.operand(N, K, 400_000 + r, std=0.02)[0]

    A, W = operands(rank)
    fused = sharded.RowShardedFp4Linear(W, fused=True)
    got = fused.forward(A).clone()
    B.barrier()
    nccl = sharded.RowShardedFp4Linear(W, fused=False)
    got_nccl = nccl.forward(A).clone()
    B.barrier()
    # this rank's rows computed alone: every rank's partial of them, summed in rank order by the same kernels
    staging = torch.empty((world, rows, N), dtype=torch.float32, device=dev)
    scratch = torch.empty((world, rows, N), dtype=torch.float32, device=dev)
    for p in range(world):
        Ap, Wp = (A, W) if p == rank else operands(p)
        fp4_gemm.gemm_partials_transposed_b(Ap, Wp, [scratch[j].data_ptr() for j in range(world)], first_owner=(p + 1) % world)
        staging[p].copy_(scratch[rank])
    want = fp4_gemm.reduce_partials(staging)
    torch.cuda.synchronize(dev)
    ok = B.all_true(bool(torch.equal(got, want)))
    # NCCL sums the fp32 partials in its own order (ring / tree), so beyond two ranks its bf16 result may differ from the
    # rank-order sum in the last place: compared within the GEMM tolerance (relative Frobenius 1e-3), bit equality reported
    diff = (got_nccl.float() - got.float())
    rel = float(torch.linalg.norm(diff) / torch.linalg.norm(got.float()))
    rel = B.max_over_ranks(rel)
    bit_equal_nccl = B.all_true(bool(torch.equal(got_nccl, got)))
    del staging, scratch, want, got_nccl, diff
    B.barrier()
    steps = 10
    fused_ms, _ = B.timed(lambda i: fused.forward(A), steps, 3, 0.0)
    nccl_ms, _ = B.timed(lambda i: nccl.forward(A), steps, 3, 0.0)
    ave.check_device_status(dev)
    link_bytes = 4.0 * M * N * (world - 1) / world
    floor_ms = max(2.0 * M * N * K / (fp4_peak * 1e12), link_bytes / (NVLINK_GBS_PER_DIR * 1e9)) * 1e3
    return {"workload": f"row_parallel_8192x8192x8192_per_rank_nvfp4_x{world}",
            "parity_fused_equals_single_gpu_recomputation": ok,
            "nccl_reduce_scatter_form_rel_fro_vs_fused": round(rel, 8), "nccl_form_within_1e-3": rel <= 1e-3,
            "nccl_form_bit_equal": bit_equal_nccl,
            "fused_ms_per_step": round(fused_ms, 4), "nccl_ms_per_step": round(nccl_ms, 4),
            "fused_tflops_whole_box": round(2.0 * M * N * K * world / (fused_ms * 1e-3) / 1e12, 1),
            "nvlink_bytes_out_per_gpu": int(link_bytes), "floor_ms": round(floor_ms, 4), "frac_of_floor": round(floor_ms / fused_ms, 4)}


def c3_block(B: Bench, fp4_peak: float, args) -> dict:
    """Config 3: M = 8192, N = 57344 split over the ranks, K = 8192 (strong scaling), same kernels as the headline."""
    world = B.world
    n_local = C3_N // world
    steps = 8 if world == 1 else 10
    blk = sharded_block(B, n_local, 2, steps, 3, 60.0, "c3")
    flops_gpu = 2.0 * M * n_local * K
    res = {"workload": f"c3_prefill_8192x57344x8192_nvfp4_n_sharded_x{world}", "n_per_gpu": n_local, "scaling": "strong",
           "gemm_only_ms": round(blk["gemm_ms"], 4), "gemm_only_tflops_per_gpu": round(flops_gpu / (blk["gemm_ms"] * 1e-3) / 1e12, 1),
           "step_ms": round(blk["step_ms"], 4), "whole_box_tflops": round(world * flops_gpu / (blk["step_ms"] * 1e-3) / 1e12, 1),
           "per_gpu_tflops": round(flops_gpu / (blk["step_ms"] * 1e-3) / 1e12, 1),
           "frac_of_nominal_9000_per_gpu_gemm_only": round(flops_gpu / (blk["gemm_ms"] * 1e-3) / 1e12 / NOMINAL_FP4_TFLOPS, 4)}
    if world > 1:
        res["fused_step"] = nvlink_roofline(world, n_local, fp4_peak, blk["step_ms"], blk["gemm_ms"], blk["ag_ms"], blk["fused"])
        res["parity"] = blk["parity"]
    del blk
    B.torch.cuda.empty_cache()
    return res


def _timed_simple(torch, dev, fn, steps, warm=5):
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) / steps


def decode_bench(ave, torch, dev, peaks) -> dict:
    """Decode shape M=16, N=28672, K=8192: weights pre-quantised, activations (0.1 % outlier channels)
    quantised on the fly.  Three weight sets are rotated (3 x 132 MB > L2).  Reports the GEMM kernel's
    HBM GB/s on its 133 111 808 algorithmic bytes, the quantise + GEMM chain next to it (config 2 as
    written), and the time of an isolated launch (nothing queued behind or before it to overlap with)."""
    from avelang_b200 import inputs

    m, n, k = 16, 28672, 8192
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    Ws = []
    for _ in range(3):
        w = (torch.randn((n, k), generator=gen, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        Ws.append(ave.quantize_nvfp4(w))
        del w
    x = inputs.outlier_activations_bf16(m, k, seed=0).to(dev)
    X = ave.quantize_nvfp4(x)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    algo_bytes = m * k // 2 + n * k // 2 + (m + n) * k // 16 + 2 * m * n
    chain_bytes = algo_bytes + 2 * m * k + m * k // 2 + m * k // 16

    # plain launches are host-bound at this size, so replay a captured graph of 12 GEMMs (4 rounds x 3 weight sets)
    ROUNDS = 4

    def three():
        for _ in range(ROUNDS):
            for W in Ws:
                # weights are resident and never rewritten: the decode kernel may overlap its start-up with the previous launch
                ave.gemm_nvfp4_transposed_b(X, W, out=out, static_weights=True)

    Xq = ave.quantize_nvfp4(x)    # preallocated quantised activations, rewritten by every chain step

    def chain():
        for _ in range(ROUNDS):
            for W in Ws:
                q = ave.quantize_nvfp4(x, out=Xq)
                ave.gemm_nvfp4_transposed_b(q, W, out=out, static_weights=True)

    variants = [("gemm", three), ("chain", chain)]
    fused_fn = getattr(ave, "linear_nvfp4_decode", None)
    if fused_fn is not None:
        def fused():
            for _ in range(ROUNDS):
                for W in Ws:
                    fused_fn(x, W, out=out, static_weights=True)
        variants.append(("one_call", fused))

    graphs = {}
    for name, fn in variants:
        fn()
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream(dev)
        with torch.cuda.graph(g, stream=s):
            fn()
        torch.cuda.synchronize(dev)
        graphs[name] = g
    # the variants are timed in turn, six rounds of 10 replays each, best round per variant: a transient of the board
    # (clock or memory-clock dip after the compute-bound blocks before this one) then hits all of them alike
    res = {name: float("inf") for name in graphs}
    for _ in range(6):
        for name, g in graphs.items():
            res[name] = min(res[name], _timed_simple(torch, dev, lambda i: g.replay(), 10) / (3.0 * ROUNDS))

    # single launch, nothing to overlap with: the events and the launch are queued behind a 256 MB memset (which also
    # flushes L2, TLBs included), so that the host's launch latency is not inside the interval
    flush = torch.empty((256 << 20,), dtype=torch.uint8, device=dev)
    iso = []
    for i in range(9):
        torch.cuda.synchronize(dev)
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ave.gemm_nvfp4_transposed_b(X, Ws[i % 3], out=out)
        e1.record()
        torch.cuda.synchronize(dev)
        iso.append(e0.elapsed_time(e1))
    del flush
    iso_ms = statistics.median(iso[2:])

    ave.check_device_status(dev)
    gbs = algo_bytes / (res["gemm"] * 1e-3) / 1e9
    d = {"workload": "c2_decode_16x28672x8192_nvfp4", "gemm_us": round(res["gemm"] * 1e3, 2), "gbs": round(gbs, 1),
         "algorithmic_bytes": algo_bytes, "frac_of_measured_hbm": round(gbs / peaks["hbm"], 4),
         "frac_of_nominal_8000": round(gbs / NOMINAL_HBM_GBS, 4),
         "isolated_launch_us": round(iso_ms * 1e3, 2),
         "isolated_launch_how": "one launch between two events, queued behind a 256 MB memset (cold L2 and TLBs, no neighbour to overlap with); median of 7",
         "quantise_plus_gemm_us": round(res["chain"] * 1e3, 2),
         "quantise_plus_gemm_gbs": round(chain_bytes / (res["chain"] * 1e-3) / 1e9, 1),
         "quantise_plus_gemm_frac_of_measured_hbm": round(chain_bytes / (res["chain"] * 1e-3) / 1e9 / peaks["hbm"], 4),
         "timing": "CUDA graph of 12 launches (4 rounds over 3 weight sets, programmatic dependent launch between them), 10 replays per round, best of 6 rounds",
         "traffic": NCU_TRAFFIC["decode"][0], "traffic_source": NCU_TRAFFIC["decode"][1]}
    if "one_call" in res:
        fg = chain_bytes / (res["one_call"] * 1e-3) / 1e9
        d.update({"linear_decode_one_call_us": round(res["one_call"] * 1e3, 2), "linear_decode_one_call_gbs": round(fg, 1),
                  "linear_decode_one_call_frac_of_measured_hbm": round(fg / peaks["hbm"], 4),
                  "linear_decode_one_call_frac_of_nominal_8000": round(fg / NOMINAL_HBM_GBS, 4)})
    return d


def quantise_bench(ave, torch, dev, peaks) -> dict:
    """bf16 -> NVFP4 / MXFP4 at 8192 x 8192 (C1's activations) with preallocated outputs: static tensor scale
    (one kernel), dynamic tensor scale (amax + quantise) and MXFP4.  Three inputs are rotated (3 x 134 MB > L2)."""
    rows = k = 8192
    gen = torch.Generator(device=dev)
    gen.manual_seed(11)
    xs = [torch.randn((rows, k), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16) for _ in range(3)]
    q_nv = ave.quantize_nvfp4(xs[0])
    q_mx = ave.quantize_mxfp4(xs[0])
    gs = q_nv.global_scale.clone()
    b_nv = 2 * rows * k + rows * k // 2 + rows * k // 16
    b_mx = 2 * rows * k + rows * k // 2 + rows * k // 32
    steps = 30
    t_static = min(_timed_simple(torch, dev, lambda i: ave.quantize_nvfp4(xs[i % 3], global_scale=gs, out=q_nv), steps) for _ in range(3))
    t_dyn = min(_timed_simple(torch, dev, lambda i: ave.quantize_nvfp4(xs[i % 3], out=q_nv), steps) for _ in range(3))
    t_mx = min(_timed_simple(torch, dev, lambda i: ave.quantize_mxfp4(xs[i % 3], out=q_mx), steps) for _ in range(3))
    ave.check_device_status(dev)

    def blk(t_ms, nbytes):
        g = nbytes / (t_ms * 1e-3) / 1e9
        return {"us": round(t_ms * 1e3, 2), "gbs": round(g, 1), "algorithmic_bytes": nbytes,
                "frac_of_measured_hbm": round(g / peaks["hbm"], 4), "frac_of_nominal_8000": round(g / NOMINAL_HBM_GBS, 4)}

    return {"workload": "quantise_8192x8192_bf16", "bound": "hbm", "peak_gbs": peaks["hbm"], "peak_source": peaks["source"],
            "nvfp4_static_scale": blk(t_static, b_nv),
            "nvfp4_dynamic_scale_amax_plus_quantise": blk(t_dyn, b_nv + 2 * rows * k),
            "mxfp4": blk(t_mx, b_mx),
            "timing": "30 back-to-back calls with preallocated outputs over 3 rotated inputs, best of 3"}


def c4_bench(B: Bench, fp4_peak: float) -> dict:
    """Config 4: MXFP4 16384^3, activations Student-t (3 degrees of freedom), weights N(0, 0.02)."""
    torch, ave, dev = B.torch, B.ave, B.dev
    n = 16384
    gen = torch.Generator(device=dev)
    gen.manual_seed(4)
    ops = []
    for _ in range(2):
        z = torch.randn((n, n), generator=gen, device=dev, dtype=torch.float32)
        s = torch.zeros((n, n), device=dev, dtype=torch.float32)
        for _ in range(3):
            t = torch.randn((n, n), generator=gen, device=dev, dtype=torch.float32)
            s.addcmul_(t, t)
        a = (z / torch.sqrt(s / 3.0)).to(torch.bfloat16)
        del z, s, t
        w = (torch.randn((n, n), generator=gen, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        ops.append((ave.quantize_mxfp4(a), ave.quantize_mxfp4(w)))
        del a, w
    out = torch.empty((n, n), dtype=torch.bfloat16, device=dev)
    ms = min(_timed_simple(torch, dev, lambda i: ave.gemm_mxfp4_transposed_b(ops[i % 2][0], ops[i % 2][1], out=out), 20, warm=4)
             for _ in range(2))
    ave.check_device_status(dev)
    tf = 2.0 * n * n * n / (ms * 1e-3) / 1e12
    del ops, out
    torch.cuda.empty_cache()
    return {"workload": "c4_mxfp4_16384", "ms": round(ms, 4), "tflops": round(tf, 1), "frac_of_4x_measured_bf16": round(tf / fp4_peak, 4),
            "frac_of_nominal_9000": round(tf / NOMINAL_FP4_TFLOPS, 4),
            "algorithmic_bytes": n * n // 2 * 2 + 2 * n * n // 32 + 2 * n * n,
            "timing": "20 back-to-back launches over 2 rotated operand sets (2 x 285 MB + 512 MB output > L2), best of 2"}


def library_context(B: Bench) -> dict:
    """Context, outside every timed path above: the vendor library's NVFP4 GEMM (torch._scaled_mm) on the same
    bytes, same board, same loop as this kernel, timed back to back with it."""
    torch, ave, dev = B.torch, B.ave, B.dev
    if not hasattr(torch, "float4_e2m1fn_x2") or not hasattr(torch, "_scaled_mm"):
        return {"unavailable": "this torch has no NVFP4 _scaled_mm"}
    sets = [(B.operand(M, K, act_seed(10 + i))[0], B.operand(N, K, weight_seed(0, 10 + i))[0]) for i in range(3)]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    f4, f8 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
    views = [(a.packed.view(f4), b.packed.view(f4).t(), a.scales.view(f8), b.scales.view(f8)) for a, b in sets]

    def lib(i):
        va, vb, sa, sb = views[i % 3]
        torch._scaled_mm(va, vb, scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16, out=out)

    def ours(i):
        ave.gemm_nvfp4_transposed_b(sets[i % 3][0], sets[i % 3][1], out=out)

    try:
        lib(0)
        torch.cuda.synchronize(dev)
    except Exception as exc:
        return {"unavailable": repr(exc)[:200]}
    t_lib, t_ours = [], []
    for _ in range(3):
        t_ours.append(_timed_simple(torch, dev, ours, 200, warm=20))
        t_lib.append(_timed_simple(torch, dev, lib, 200, warm=20))
    fl = 2.0 * M * N * K
    return {"what": "torch._scaled_mm (vendor library NVFP4 GEMM, no tensor scale) vs this kernel: 8192^3, 3 operand sets rotated, "
                    "200 back-to-back launches each, alternating, best of 3",
            "library_us": round(min(t_lib) * 1e3, 2), "library_tflops": round(fl / (min(t_lib) * 1e-3) / 1e12, 1),
            "ours_us": round(min(t_ours) * 1e3, 2), "ours_tflops": round(fl / (min(t_ours) * 1e-3) / 1e12, 1),
            "ours_over_library": round(min(t_lib) / min(t_ours), 4)}


# ----------------------------------------------------------------------------- CPU oracle
def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


def claim_host_threads() -> int:
    """Make the CPU legs use every host core this process may run on.  torch.distributed.run exports
    OMP_NUM_THREADS=1 to its workers, which would otherwise hold the oracle and torch to one thread."""
    n = host_threads()
    for var in ("OMP_NUM_THREADS", "MKL_NUM_THREADS", "OPENBLAS_NUM_THREADS"):
        os.environ[var] = str(n)
    import torch

    torch.set_num_threads(n)
    from oracle import fp4_oracle as O

    O.build()
    O.set_num_threads(n)
    return n


def cpu_oracle_step(O, torch, a_bits, qb, n_rows, phases=None):
    """The oracle path on the host: quantise the activation rows, dequantise both operands,
    fp32 matmul (the reference's expression on CPU tensors), round to bf16."""
    t0 = time.perf_counter()
    qa = O.c_quantize(a_bits[:n_rows], O.NVFP4)
    t1 = time.perf_counter()
    a_hat = O.c_dequantize(*qa, O.NVFP4)
    b_hat = O.c_dequantize(*qb, O.NVFP4)
    t2 = time.perf_counter()
    d32 = torch.from_numpy(a_hat) @ torch.from_numpy(b_hat).T
    d = d32.to(torch.bfloat16)
    t3 = time.perf_counter()
    if phases is not None:
        phases.append((t1 - t0, t2 - t1, t3 - t2))
    return d


def cpu_baseline(full: bool = True, sample_rows: int = 512) -> dict:
    """CPU legs reported beside the GPU numbers: config 1 in full on the torch path (quantise / dequantise / fp32
    matmul + bf16 round, phases split), config 0 on both the torch path and the C oracle's own GEMM, and the C
    oracle GEMM on a 1024^3 sub-problem."""
    import numpy as np
    import torch

    cores = claim_host_threads()
    from oracle import fp4_oracle as O

    rng = np.random.default_rng(0)
    rows = M if full else sample_rows
    a_bits = O.f32_to_bf16_bits(rng.standard_normal((rows, K), dtype=np.float32))
    b_bits = O.f32_to_bf16_bits(rng.standard_normal((N, K), dtype=np.float32))
    qb = O.c_quantize(b_bits, O.NVFP4)          # weights are pre-quantised, as on the GPU arm
    t0 = time.perf_counter()
    cpu_oracle_step(O, torch, a_bits, qb, rows)  # warm-up, and the size check: fall back to a sample if a pass is slow
    if time.perf_counter() - t0 > 8.0 and rows > sample_rows:
        rows = sample_rows
    phases = []
    for _ in range(3):
        cpu_oracle_step(O, torch, a_bits, qb, rows, phases)
    tot = sorted(sum(p) for p in phases)[1]
    ph = [statistics.median(p[i] for p in phases) for i in range(3)]
    flops = 2.0 * rows * N * K
    res = {"value": round(flops / tot / 1e12, 5), "unit": "TFLOP/s", "cores": cores, "kind": "port",
           "sample": (f"config 1, {'all' if rows == M else rows} of {M} rows of A against the full 8192x8192 B: quantise A, dequantise A and B, "
                      f"fp32 matmul (torch CPU), bf16 round; median of 3 passes, {tot:.2f} s per pass"),
           "seconds": round(tot, 3),
           "phases_s": {"quantise_a": round(ph[0], 4), "dequantise_a_b": round(ph[1], 4), "matmul_f32_plus_bf16_round": round(ph[2], 4)},
           "omp_threads": O.num_threads(), "torch_threads": int(torch.get_num_threads())}

    # config 0 (128 x 256 x 512), both implementations, and their agreement
    a0 = O.f32_to_bf16_bits(rng.standard_normal((128, 512), dtype=np.float32))
    b0 = O.f32_to_bf16_bits(rng.standard_normal((256, 512), dtype=np.float32))

    def c0_torch():
        qa_, qb_ = O.c_quantize(a0, O.NVFP4), O.c_quantize(b0, O.NVFP4)
        d32 = torch.from_numpy(O.c_dequantize(*qa_, O.NVFP4)) @ torch.from_numpy(O.c_dequantize(*qb_, O.NVFP4)).T
        return d32.to(torch.bfloat16)

    def c0_c():
        qa_, qb_ = O.c_quantize(a0, O.NVFP4), O.c_quantize(b0, O.NVFP4)
        return O.c_gemm_fp4(qa_, qb_, O.NVFP4, want_f32=False)[1]

    def med(fn, n=5):
        fn()
        ts = []
        for _ in range(n):
            t = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t)
        return statistics.median(ts)

    t_t, t_c = med(c0_torch), med(c0_c)
    dt = c0_torch().view(torch.int16).numpy().view(np.uint16)
    dc = c0_c()
    f0 = 2.0 * 128 * 256 * 512
    res["c0_128x256x512"] = {"torch_path_ms": round(t_t * 1e3, 3), "torch_path_gflops": round(f0 / t_t / 1e9, 2),
                             "c_oracle_ms": round(t_c * 1e3, 3), "c_oracle_gflops": round(f0 / t_c / 1e9, 2),
                             "bf16_results_differing": int((dt != dc).sum()), "elements": int(dc.size)}
    s = 1024
    qa1 = O.c_quantize(a_bits[:s, :s].copy(), O.NVFP4)
    qb1 = O.c_quantize(b_bits[:s, :s].copy(), O.NVFP4)
    t_g = med(lambda: O.c_gemm_fp4(qa1, qb1, O.NVFP4, want_f32=False), n=3)
    res["c_oracle_gemm_1024"] = {"ms": round(t_g * 1e3, 2), "gflops": round(2.0 * s ** 3 / t_g / 1e9, 2),
                                 "what": "the C oracle's own GEMM (dequantise + fp64-accumulated product, OpenMP) on a 1024^3 sub-problem"}
    return res


def run_reference(args) -> dict:
    """The reference arm: the oracle's CPU path on the host cores (the reference project has no FP4
    implementation and cannot be built here, so the oracle port is the reference for this path).
    One step = config 1 in full (all 8192 rows); rows are halved only if a full pass would not fit the time budget."""
    _, rank, _ = dist_env()
    if rank != 0:
        return {}
    cores = claim_host_threads()
    import numpy as np
    import torch

    from oracle import fp4_oracle as O

    rows = M
    rng = np.random.default_rng(0)
    a_bits = O.f32_to_bf16_bits(rng.standard_normal((rows, K), dtype=np.float32))
    b_bits = O.f32_to_bf16_bits(rng.standard_normal((N, K), dtype=np.float32))
    qb = O.c_quantize(b_bits, O.NVFP4)
    # size the sample so that steps + warm-up stay within ~3 minutes
    t0 = time.perf_counter()
    cpu_oracle_step(O, torch, a_bits, qb, rows)
    t_one = time.perf_counter() - t0
    budget = 150.0
    total = args.steps + args.warmup
    while rows > 8 and t_one * total > budget:
        rows //= 2
        t0 = time.perf_counter()
        cpu_oracle_step(O, torch, a_bits, qb, rows)
        t_one = time.perf_counter() - t0
    for _ in range(args.warmup):
        cpu_oracle_step(O, torch, a_bits, qb, rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_oracle_step(O, torch, a_bits, qb, rows)
    dt = (time.perf_counter() - t0) / args.steps
    value = 2.0 * rows * N * K / dt / 1e12
    sample = (f"each step = {'all' if rows == M else rows} of {M} rows of A against the full 8192x8192 B (one GPU's share of the workload): "
              f"quantise A rows, dequantise A and B, fp32 matmul (torch CPU), bf16 round; {cores} host threads")
    return {
        "impl": "reference", "metric": METRIC, "value": round(value, 5), "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": "strong" if args.workload == "c3" else "weak", "vs_baseline": None,
        "dtype": "fp32 (dequantised E2M1 x scale)", "data": "synthetic",
        "config": make_config(args.gpus, args.workload),
        "cpu_baseline": {"value": round(value, 5), "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample,
                         "omp_threads": O.num_threads(), "torch_threads": int(torch.get_num_threads()), "rows_per_step": rows},
        "e2e": {"value": round(value, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=512, help="rows of A in the CPU baseline when a sample is used")
    ap.add_argument("--cpu-sample", action="store_true", help="CPU baseline on --cpu-rows rows instead of config 1 in full")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-decode", action="store_true")
    ap.add_argument("--skip-quantise", action="store_true")
    ap.add_argument("--skip-c3", action="store_true")
    ap.add_argument("--skip-c4", action="store_true")
    ap.add_argument("--skip-context", action="store_true")
    ap.add_argument("--skip-fp4-gather", action="store_true")
    ap.add_argument("--skip-ksharded", action="store_true")
    ap.add_argument("--bind-cpus", action="store_true",
                    help="N > 1: bind every rank to the CPUs NVML names as local to its GPU before it allocates pinned buffers "
                         "(measured both ways on this pool: 652 vs 635 TFLOP/s end to end at N = 2, 531 vs 624 at N = 4; off by default)")
    ap.add_argument("--min-timed-ms", type=float, default=MIN_TIMED_MS,
                    help="the K steps are repeated until the timed region is this long (0: time the K steps once, e.g. under a profiler)")
    ap.add_argument("--workload", default="c1", choices=["c1", "c3"],
                    help="headline workload. c1: 8192^3 per GPU (weak scaling); c3: 8192 x 57344 x 8192 with N split over the GPUs")
    ap.add_argument("--nccl-allgather", action="store_true", help="N > 1: exchange with NCCL after the GEMM instead of the fused epilogue")
    args = ap.parse_args()
    res = run_reference(args) if args.impl == "reference" else run_ours(args)
    if res:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
