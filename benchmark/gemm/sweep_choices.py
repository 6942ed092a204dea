#!/usr/bin/env python3
"""Measure the design choices of the FP4 kernels one knob at a time and print them as tables.

    python benchmark/gemm/sweep_choices.py [--ncu] [--only tiles,stages,decode] [--out FILE]

Each row is one run of benchmark/gemm/bench_fp4_gemm.py in a process of its own (the tuning knobs are
environment variables the library reads once): CUDA-event time over a replayed graph, and with --ncu
one more short run of the same configuration under

    ncu --metrics gpu__time_duration.sum,sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active,
        dram__bytes_read.sum,dram__bytes_write.sum,sm__cycles_elapsed.avg.per_second
        --clock-control none -k regex:<kernel> -s <warm-up launches> -c 2

(preceded by the same command line without ncu, which must exit 0).  The decisions covered:

  tiles    tile shape / CTA pairing of the compute-bound kernel, at 8192^3 and at config 3's per-GPU shape on
           8 GPUs (8192 x 7168 x 8192)
  stages   shared-memory pipeline depth of the 256x256 CTA-pair tile (AVE_FP4_GEMM_STAGES)
  decode   load-burst size (AVE_FP4_SKINNY_BURST) and stream-K split on/off (AVE_FP4_SKINNY_STREAMK) of the
           decode kernel at 16 x 28672 x 8192

The reference has one fixed tile (128x128x64, python/avelang_kernels/amdgpu_gemm.py:34-41) and no such sweep;
this is the counterpart of its benchmark driver (benchmark/gemm/bench_amdgpu_gemm.py) for choosing ours.
"""
import argparse
import csv
import io
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BENCH = os.path.join(HERE, "bench_fp4_gemm.py")
METRICS = ("gpu__time_duration.sum,sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active,"
           "dram__bytes_read.sum,dram__bytes_write.sum,sm__cycles_elapsed.avg.per_second")
VARIANTS = {1: "1-CTA 128x128", 2: "1-CTA 128x256", 3: "2-CTA 256x256", 4: "2-CTA 256x128", 5: "2-CTA 256x192"}


def run(cmd, env):
    e = dict(os.environ)
    e.update(env)
    p = subprocess.run(cmd, env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    return p.returncode, p.stdout


def timed(shape, extra, env):
    m, n, k = shape
    rc, out = run([sys.executable, BENCH, "--m", str(m), "--n", str(n), "--k", str(k), "--warmup", "3", "--repeat", "3",
                   "--iters", "20", "--rotate", "3", *extra], env)
    mt = re.search(r"time_ms=([0-9.]+) tflops=([0-9.]+) bandwidth_gbs=([0-9.]+)", out)
    if rc != 0 or not mt:
        return None
    return float(mt.group(1)), float(mt.group(2)), float(mt.group(3))


def counters(shape, extra, env, kernel_regex):
    """Two launches of the configuration under ncu (after the same command line has run plain)."""
    m, n, k = shape
    cmd = [sys.executable, BENCH, "--m", str(m), "--n", str(n), "--k", str(k), "--warmup", "1", "--repeat", "1", "--iters", "2",
           "--rotate", "1", "--no-graph", *extra]
    rc, out = run(cmd, env)
    if rc != 0:
        return {"error": "plain run failed: " + out[-200:]}
    rc, out = run(["ncu", "--metrics", METRICS, "--clock-control", "none", "-k", f"regex:{kernel_regex}", "-s", "1", "-c", "2",
                   "--csv", *cmd], env)
    rows = [r for r in csv.reader(io.StringIO(out)) if len(r) > 8 and r[0].isdigit()]
    if not rows:
        return {"error": "no ncu rows (closed or failed): " + out[-200:].replace("\n", " ")}
    res = {}
    for r in rows:
        name, val = r[-3], r[-1].replace(",", "")
        try:
            res.setdefault(name, []).append(float(val))
        except ValueError:
            pass
    return {k: sum(v) / len(v) for k, v in res.items()}


def fmt_counters(c, flops=None, algo_bytes=None):
    if c is None:
        return "", "", ""
    if "error" in c:
        return c["error"][:60], "", ""
    us = c.get("gpu__time_duration.sum", 0.0) / 1e3
    tens = c.get("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active")
    dram = (c.get("dram__bytes_read.sum", 0.0) + c.get("dram__bytes_write.sum", 0.0)) / 1e6
    ghz = c.get("sm__cycles_elapsed.avg.per_second", 0.0)
    ghz = ghz / 1e9 if ghz > 1e6 else ghz          # reported in Hz or in cycles per nanosecond
    a = f"{us:.1f} us @ {ghz:.2f} GHz"
    b = f"{tens:.1f} %" if tens is not None else ""
    d = f"{dram:.1f} MB"
    if algo_bytes:
        d += f" ({dram * 1e6 / algo_bytes:.2f}x algorithmic)"
    return a, b, d


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ncu", action="store_true", help="also capture counters with ncu (two launches per row)")
    ap.add_argument("--only", default="tiles,stages,decode")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    which = set(args.only.split(","))
    lines = []

    def emit(s=""):
        print(s, flush=True)
        lines.append(s)

    if "tiles" in which:
        for shape in ((8192, 8192, 8192), (8192, 7168, 8192)):
            m, n, k = shape
            algo = m * k // 2 + n * k // 2 + (m + n) * k // 16 + 2 * m * n
            emit(f"### Tile shape, NVFP4 {m} x {n} x {k} (3 operand sets rotated)")
            emit("| variant | tiles | waves on 148 SMs | graph-replay time | TFLOP/s | ncu launch | tensor pipe active | DRAM traffic |")
            emit("|---|---|---|---|---|---|---|---|")
            for v, name in VARIANTS.items():
                cm = 256 if v >= 3 else 128
                bn = {1: 128, 2: 256, 3: 256, 4: 128, 5: 192}[v]
                tiles = -(-m // cm) * -(-n // bn)
                slots = 74 if v >= 3 else 148
                t = timed(shape, ["--variant", str(v)], {})
                c = counters(shape, ["--variant", str(v)], {}, "gemm_fp4_kernel") if args.ncu else None
                a, b, d = fmt_counters(c, algo_bytes=algo)
                emit(f"| {name} | {tiles} | {tiles / slots:.2f} | " + (f"{t[0] * 1e3:.1f} us | {t[1]:.0f}" if t else "failed | ") + f" | {a} | {b} | {d} |")
            emit()

    if "stages" in which:
        shape = (8192, 8192, 8192)
        emit("### Pipeline depth of the 2-CTA 256x256 tile, NVFP4 8192^3 (38 KB per stage and CTA; 5 stages + 32 KB epilogue staging = 223 KB)")
        emit("| stages | graph-replay time | TFLOP/s | ncu launch | tensor pipe active | DRAM traffic |")
        emit("|---|---|---|---|---|---|")
        for st in (3, 4, 5):
            env = {"AVE_FP4_GEMM_STAGES": str(st)} if st != 5 else {}
            t = timed(shape, ["--variant", "3"], env)
            c = counters(shape, ["--variant", "3"], env, "gemm_fp4_kernel") if args.ncu else None
            a, b, d = fmt_counters(c)
            emit(f"| {st} | " + (f"{t[0] * 1e3:.1f} us | {t[1]:.0f}" if t else "failed | ") + f" | {a} | {b} | {d} |")
        emit()

    if "decode" in which:
        shape = (16, 28672, 8192)
        m, n, k = shape
        algo = m * k // 2 + n * k // 2 + (m + n) * k // 16 + 2 * m * n
        extra = ["--a-kind", "outlier", "--b-kind", "weight"]
        emit(f"### Decode kernel, NVFP4 {m} x {n} x {k}: load burst and stream-K split ({algo} algorithmic bytes)")
        emit("| burst (K blocks per load burst) | stream-K split of the T mod G tiles | graph-replay time | GB/s | ncu launch | DRAM traffic |")
        emit("|---|---|---|---|---|---|")
        for burst, sk in ((1, 1), (2, 1), (4, 1), (8, 1), (4, 0)):
            env = {"AVE_FP4_SKINNY_BURST": str(burst)}
            if not sk:
                env["AVE_FP4_SKINNY_STREAMK"] = "0"
            t = timed(shape, extra, env)
            c = counters(shape, extra, env, "gemm_fp4_skinny_kernel") if args.ncu else None
            a, _, d = fmt_counters(c, algo_bytes=algo)
            emit(f"| {burst} | {'yes' if sk else 'no (whole tiles, tile t on CTA t mod 148)'} | " +
                 (f"{t[0] * 1e3:.2f} us | {t[2]:.0f}" if t else "failed | ") + f" | {a} | {d} |")
        emit()

    if args.out:
        with open(args.out, "w") as f:
            f.write("\n".join(lines) + "\n")


if __name__ == "__main__":
    main()
