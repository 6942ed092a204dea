"""CPU tier: the benchmark's contract pieces that need no GPU -- both arms print the same `config`, the reference arm
uses every host thread even when the launcher exports OMP_NUM_THREADS=1, and ranks other than 0 stay silent."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_config_object_depends_only_on_world_and_workload():
    a, b = bench.make_config(4, "c1"), bench.make_config(4, "c1")
    assert a == b and a["world"] == 4 and a["n_per_gpu"] == 8192
    c3 = bench.make_config(8, "c3")
    assert c3["n_per_gpu"] == 57344 // 8 and "c3" in c3["workload"]
    assert bench.make_config(1, "c1")["workload"] == "c1_square_nvfp4_8192"


def test_nvlink_roofline_arithmetic():
    r = bench.nvlink_roofline(8, 8192, 6480.0, 1.448, 0.204, 1.543, True)
    assert r["bound"] == "nvlink" and r["nvlink_bytes_in_per_gpu"] == 2 * 8192 * 8192 * 7
    assert abs(r["target_ms"] - 2 * 8192 * 8192 * 7 / 770e9 * 1e3) < 1e-3
    assert abs(r["frac"] - r["target_ms"] / 1.448) < 1e-3


def _run_reference(rank: str):
    env = dict(os.environ, OMP_NUM_THREADS="1", RANK=rank, WORLD_SIZE="2", LOCAL_RANK=rank)
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                           "--warmup", "0"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900)


def test_reference_arm_uses_all_host_threads_and_the_same_config():
    p = _run_reference("0")
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 2
    assert line["config"] == bench.make_config(2, "c1")
    threads = bench.host_threads()
    assert line["cpu_baseline"]["cores"] == threads
    assert line["cpu_baseline"]["omp_threads"] == threads          # not the launcher's OMP_NUM_THREADS=1
    assert line["cpu_baseline"]["kind"] == "port" and line["value"] > 0
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["value"] == line["value"]


def test_reference_arm_is_silent_on_other_ranks():
    p = _run_reference("1")
    assert p.returncode == 0 and p.stdout.strip() == ""
