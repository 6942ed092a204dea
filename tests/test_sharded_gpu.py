"""GPU tier, needs >= 2 GPUs (skipped otherwise): N-sharded GEMM with the NCCL all-gather and with the
all-gather fused into the GEMM epilogue (peer stores over NVLink) give the same bits, equal to the
unsharded GEMM; and the form that gathers the quantised output gives the quantise kernel's bytes."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["AVE_ROOT"])
import avelang_b200 as ave
from avelang_b200 import inputs, sharded
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local); dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
m, n, k = 384, 1024 * world, 1024
a = inputs.normal_bf16(m, k, 0).to(dev)
w = inputs.normal_bf16(n, k, 1, std=0.02).to(dev)
A = ave.quantize_nvfp4(a)
Wfull = ave.quantize_nvfp4(w, sf_layout=ave.SF_ROW_MAJOR)
full = ave.gemm_nvfp4_transposed_b(A, Wfull)
# every shard is quantised with the tensor scale of the whole weight
shard = ave.quantize_nvfp4(sharded.shard_rows(w, world, rank).contiguous(), global_scale=Wfull.global_scale)
ok = True
for fused in (False, True):
    layer = sharded.ShardedFp4Linear(shard, fused=fused)
    for _ in range(2):
        g = layer.forward(A)
        torch.cuda.synchronize(); dist.barrier()
        logical = sharded.columns_view(g).reshape(m, n)
        ok = ok and bool(torch.equal(logical, full))
        dist.barrier()
# the same layer gathering its output as the next layer's FP4 operand (quantising epilogue + peer stores)
gs_out = torch.tensor([float(full.float().abs().max()) / 2688.0], dtype=torch.float32, device=dev)
want = ave.quantize_nvfp4(full, global_scale=gs_out)
qlayer = sharded.ShardedFp4LinearQuantizedOut(shard, out_global_scale=gs_out)
for _ in range(2):
    op = qlayer.forward(A)
    torch.cuda.synchronize(); dist.barrier()
    ok = ok and bool(torch.equal(op.packed, want.packed)) and bool(torch.equal(op.scales, want.scales))
    dist.barrier()
ave.check_device_status(dev)
print(f"rank {rank} ok={ok}", flush=True)
dist.destroy_process_group()
sys.exit(0 if ok else 1)
"""


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_sharded_fused_equals_nccl_equals_unsharded(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, AVE_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), str(script)]
    proc = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:]
    assert "rank 0 ok=True" in proc.stdout and "rank 1 ok=True" in proc.stdout
