"""GPU tier: the N-sharded GEMM whose epilogue quantises its tile and stores it into every rank's copy of the next
layer's FP4 operand (`ave_fp4_gemm_allgather_quantized`, through the C ABI).

Parity bar (bytes): every rank's gathered operand equals, bit for bit, the quantise kernel applied to the bf16
result of the unsharded GEMM -- packed nibbles and tiled scale bytes.  The ranks are emulated on one GPU here (one
call per rank, the "peers" are the other ranks' buffers in the same memory; no kernel waits for another); the real
two-process form is in test_sharded_gpu.py."""
import pytest
import torch

import avelang_b200 as ave
from avelang_b200 import fp4_gemm, inputs

pytestmark = pytest.mark.gpu


def _gathered_buffers(world, m, n_total, fmt, gs, dev):
    ops = []
    for _ in range(world):
        packed = torch.full((m, n_total // 2), 0xEE, dtype=torch.uint8, device=dev)
        scales = torch.full((fp4_gemm.sf_bytes(m, n_total, fmt, ave.SF_TILED),), 0xEE, dtype=torch.uint8, device=dev)
        ops.append(ave.Fp4Operand(packed, scales, gs, fmt, m, n_total, ave.SF_TILED))
    return ops


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
@pytest.mark.parametrize("world,m,n_local,k,act", [(2, 384, 256, 1024, None), (4, 300, 320, 512, "silu"), (8, 256, 64, 768, "relu")])
def test_emulated_ranks_gather_the_quantise_kernels_bytes(cuda_device, fmt, world, m, n_local, k, act):
    dev = cuda_device
    quant = ave.quantize_nvfp4 if fmt == ave.NVFP4 else ave.quantize_mxfp4
    gemm = ave.gemm_nvfp4_transposed_b if fmt == ave.NVFP4 else ave.gemm_mxfp4_transposed_b
    n_total = world * n_local
    A = quant(inputs.normal_bf16(m, k, 0).to(dev))
    w = inputs.normal_bf16(n_total, k, 1, std=0.05).to(dev)
    Wfull = quant(w)
    bias = inputs.normal_bf16(1, n_total, 2).reshape(n_total).to(dev) if act else None
    d = gemm(A, Wfull, bias=bias, activation=act)                     # unsharded bf16 result
    gs = torch.tensor([float(d.float().abs().max()) / 2688.0], dtype=torch.float32, device=dev) if fmt == ave.NVFP4 else None
    want = quant(d, global_scale=gs) if fmt == ave.NVFP4 else quant(d)     # tiled scales, padding zero
    bufs = _gathered_buffers(world, m, n_total, fmt, gs, dev)
    for r in range(world):
        shard = w[r * n_local:(r + 1) * n_local].contiguous()
        Wr = quant(shard, global_scale=Wfull.global_scale) if fmt == ave.NVFP4 else quant(shard)
        peers = [p for p in range(world) if p != r]
        fp4_gemm.gemm_allgather_quantized_transposed_b(
            A, Wr, bufs[r], r * n_local, [bufs[p].packed.data_ptr() for p in peers], [bufs[p].scales.data_ptr() for p in peers],
            bias=None if bias is None else bias[r * n_local:(r + 1) * n_local].contiguous(), activation=act)
    ave.check_device_status(dev)
    for r in range(world):
        assert torch.equal(bufs[r].packed, want.packed), f"rank {r}: packed bytes differ"
        assert torch.equal(bufs[r].scales, want.scales), f"rank {r}: scale bytes differ"
    # and the gathered operand feeds the next layer's GEMM like the two-kernel result does
    W2 = quant(inputs.normal_bf16(128, n_total, 3, std=0.05).to(dev))
    assert torch.equal(gemm(bufs[0], W2), gemm(want, W2))


def test_rejects_shapes_it_cannot_place(cuda_device):
    dev = cuda_device
    A = ave.quantize_mxfp4(inputs.normal_bf16(128, 256, 0).to(dev))
    W = ave.quantize_mxfp4(inputs.normal_bf16(96, 256, 1).to(dev))       # 96 columns: not whole 64-column groups
    buf = _gathered_buffers(1, 128, 192, ave.MXFP4, None, dev)[0]
    with pytest.raises(ValueError, match="multiples of 64"):
        fp4_gemm.gemm_allgather_quantized_transposed_b(A, W, buf, 0, [], [])
