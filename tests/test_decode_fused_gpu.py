"""GPU tier: the one-call decode linear layer on unquantised activations (`ave_fp4_linear_decode`, through the C ABI):
activation quantise into the caller's scratch, then the decode GEMM chained behind it.

Parity bar: the activation bytes it leaves in its scratch are the oracle's (bit for bit), the result is bit-identical
to the two operators called one after the other, and within 1e-3 relative Frobenius error of the CPU oracle chain
(quantise -> dequantise -> fp32 matmul -> bf16)."""
import numpy as np
import pytest
import torch

import avelang_b200 as ave
from avelang_b200 import _lib, fp4_gemm, inputs

pytestmark = pytest.mark.gpu

SHAPES = [(16, 4096, 8192), (9, 1160, 2080), (32, 520, 2048), (1, 128, 256), (16, 28672, 1024), (16, 20480, 2048),
          (24, 256, 12288), (16, 19072, 512)]


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _fns(fmt):
    if fmt == ave.NVFP4:
        return ave.quantize_nvfp4, ave.gemm_nvfp4_transposed_b, ave.linear_nvfp4_decode
    return ave.quantize_mxfp4, ave.gemm_mxfp4_transposed_b, ave.linear_mxfp4_decode


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_fused_equals_two_kernel_chain_bit_for_bit(cuda_device, fmt, m, n, k):
    dev = cuda_device
    quant, gemm, linear = _fns(fmt)
    x = inputs.outlier_activations_bf16(m, k, seed=m + n).to(dev)
    W = quant(inputs.normal_bf16(n, k, seed=k + 1, std=0.02).to(dev))
    want = gemm(quant(x), W, variant=ave.GEMM_SKINNY)
    for i in range(3):        # the scratch (counters, header) must come back to zero after every call
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
        res = linear(x, W, out=got, static_weights=(i == 2))
        ave.check_device_status(dev)
        assert res is got
        assert torch.equal(got, want), f"call {i}: {(got != want).sum().item()} of {got.numel()} elements differ"


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
@pytest.mark.parametrize("m,k", [(16, 8192), (5, 2080), (32, 1024)])
def test_fused_leaves_the_quantise_kernels_bytes_in_scratch(cuda_device, oracle, fmt, m, k):
    """The packed nibbles and scale bytes (and, through them, the tensor scale) the call leaves in its scratch are
    the oracle's bytes."""
    dev = cuda_device
    n = 384
    quant, _, linear = _fns(fmt)
    xs = inputs.outlier_activations_bf16(m, k, seed=3)
    x = xs.to(dev)
    W = quant(inputs.normal_bf16(n, k, seed=4, std=0.02).to(dev))
    linear(x, W)
    ave.check_device_status(dev)
    L = _lib.ensure_init(dev.index or 0)
    up = lambda v: (v + 255) // 256 * 256
    mp = 16 if m <= 16 else 32
    ws = fp4_gemm._decode_workspaces[dev.index or 0]
    assert ws[0:12].view(torch.int32).tolist() == [0, 0, 0]       # header words left zero for the next launch
    packed_off = up(L.ave_fp4_workspace_bytes(m, n, k, fmt, ave.GEMM_SKINNY, dev.index or 0))
    packed = ws[packed_off: packed_off + mp * (k // 2)].view(mp, k // 2).cpu().numpy()
    sf_off = packed_off + up(mp * (k // 2))
    blk = 16 if fmt == ave.NVFP4 else 32
    sf = ws[sf_off: sf_off + ((k // blk + 3) // 4) * 512].cpu().numpy()
    q = oracle.c_quantize(_bits(xs), fmt)
    assert np.array_equal(packed[:m], q[0])
    # scale bytes of rows < MP, read back through the 128x4 tile formula
    r, c = np.meshgrid(np.arange(mp), np.arange(k // blk), indexing="ij")
    k_atoms = (k // blk + 3) // 4
    got_sf = sf[(c // 4) * 512 + (r % 32) * 16 + (r // 32) * 4 + (c % 4)] if k_atoms == 1 else \
        sf[((r // 128) * k_atoms + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (c % 4)]
    assert np.array_equal(got_sf[:m], q[1])
    assert not got_sf[m:].any()
    ref = quant(x)
    assert np.array_equal(packed[:m], ref.packed.cpu().numpy())


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
def test_fused_matches_oracle_chain(cuda_device, oracle, fmt):
    dev = cuda_device
    m, n, k = 16, 1024, 4096
    _, _, linear = _fns(fmt)
    quant = _fns(fmt)[0]
    xs = inputs.outlier_activations_bf16(m, k, seed=0)
    ws = inputs.normal_bf16(n, k, seed=1, std=0.02)
    qx, qw = oracle.c_quantize(_bits(xs), fmt), oracle.c_quantize(_bits(ws), fmt)
    _, dbf = oracle.c_gemm_fp4(qx, qw, fmt, want_f32=False)
    exp = oracle.bf16_bits_to_f32(dbf)
    got = linear(xs.to(dev), quant(ws.to(dev))).float().cpu().numpy()
    ave.check_device_status(dev)
    rel = float(np.linalg.norm(got - exp) / np.linalg.norm(exp))
    assert rel <= 1e-3, f"rel_fro {rel:.3e} max_abs {np.abs(got - exp).max():.4g}"


def test_fused_bias_activation_and_tile_major_weights(cuda_device):
    dev = cuda_device
    m, n, k = 12, 1536, 4096
    x = inputs.outlier_activations_bf16(m, k, seed=8).to(dev)
    W = ave.quantize_nvfp4(inputs.normal_bf16(n, k, seed=9, std=0.02).to(dev))
    bias = inputs.normal_bf16(1, n, seed=10).reshape(n).to(dev)
    want = ave.gemm_nvfp4_transposed_b(ave.quantize_nvfp4(x), W, variant=ave.GEMM_SKINNY, bias=bias, activation="silu")
    got = ave.linear_nvfp4_decode(x, W, bias=bias, activation="silu")
    assert torch.equal(got, want)
    got_t = ave.linear_nvfp4_decode(x, ave.pack_weight_tiles(W))
    assert torch.equal(got_t, ave.gemm_nvfp4_transposed_b(ave.quantize_nvfp4(x), W, variant=ave.GEMM_SKINNY))
    ave.check_device_status(dev)


def test_fused_in_a_graph_of_dependent_launches(cuda_device):
    """Twelve launches back to back with programmatic dependent launch between them, captured and replayed: every
    launch finds the header words zero again and gives the same bits."""
    dev = cuda_device
    m, n, k = 16, 28672, 8192
    x = inputs.outlier_activations_bf16(m, k, seed=0).to(dev)
    Ws = [ave.quantize_nvfp4(inputs.normal_bf16(n, k, seed=20 + i, std=0.02).to(dev)) for i in range(2)]
    wants = [ave.gemm_nvfp4_transposed_b(ave.quantize_nvfp4(x), W, variant=ave.GEMM_SKINNY) for W in Ws]
    outs = [torch.empty((m, n), dtype=torch.bfloat16, device=dev) for _ in range(12)]
    ave.linear_nvfp4_decode(x, Ws[0], out=outs[0])       # workspace allocated outside the capture
    torch.cuda.synchronize(dev)
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream(dev)
    with torch.cuda.graph(g, stream=s):
        for i in range(12):
            ave.linear_nvfp4_decode(x, Ws[i % 2], out=outs[i], static_weights=True)
    for _ in range(3):
        for o in outs:
            o.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize(dev)
        ave.check_device_status(dev)
        for i, o in enumerate(outs):
            assert torch.equal(o, wants[i % 2]), i


def test_fused_more_than_32_rows_takes_the_two_kernel_route(cuda_device):
    dev = cuda_device
    m, n, k = 48, 512, 1024
    x = inputs.normal_bf16(m, k, seed=1).to(dev)
    W = ave.quantize_mxfp4(inputs.normal_bf16(n, k, seed=2, std=0.02).to(dev))
    assert torch.equal(ave.linear_mxfp4_decode(x, W), ave.gemm_mxfp4_transposed_b(ave.quantize_mxfp4(x), W))
    L = _lib.ensure_init(dev.index or 0)
    rc = L.ave_fp4_linear_decode(None, k, None, None, None, None, m, n, k, n, 1, 0, None, 0, None, None)
    assert rc == -1 and b"M <= 32" in L.ave_fp4_last_error()
