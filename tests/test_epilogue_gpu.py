"""GPU tier: the fused bias + activation epilogue of the FP4 GEMM against the CPU oracle.

The oracle applies act(d + bias) in double to its fp32 GEMM result and rounds to bf16 once; the
kernel does the same in fp32.  Tolerance: relative Frobenius error <= 1e-3 (max-abs in the message).
"""
import numpy as np
import pytest
import torch

import avelang_b200 as ave
from avelang_b200 import inputs
from test_gemm_gpu import _bits, _check, _gemm, _to_dev

pytestmark = pytest.mark.gpu

ACTS = {"none": 0, "relu": 1, "gelu": 2, "gelu_tanh": 3, "silu": 4}


def _case(oracle, dev, fmt, m, n, k, variant, act, with_bias, seed=0):
    a = inputs.make_operand_bf16("normal", m, k, seed)
    b = inputs.make_operand_bf16("weight", n, k, seed + 1)
    qa, qb = oracle.c_quantize(_bits(a), fmt), oracle.c_quantize(_bits(b), fmt)
    d32, _ = oracle.c_gemm_fp4(qa, qb, fmt)
    # bias on the scale of the product so that it matters, in bf16 like the kernel reads it
    bias = (inputs.normal_bf16(1, n, seed + 2).float() * float(np.abs(d32).mean())).to(torch.bfloat16).reshape(n) if with_bias else None
    _, ybf = oracle.c_bias_act(d32, None if bias is None else _bits(bias), ACTS[act])
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
    res = _gemm(_to_dev(qa, fmt, dev), _to_dev(qb, fmt, dev), fmt, out=out, variant=variant,
                bias=None if bias is None else bias.to(dev), activation=None if act == "none" else act)
    ave.check_device_status(dev)
    assert res is out
    return _check(out, ybf, oracle, f"fmt={fmt} {m}x{n}x{k} variant={variant} act={act} bias={with_bias}")


@pytest.mark.parametrize("act", ["relu", "gelu", "gelu_tanh", "silu"])
@pytest.mark.parametrize("variant", [ave.GEMM_2CTA_N256, ave.GEMM_1CTA_N128, ave.GEMM_2CTA_N192])
def test_bias_activation_tiled(cuda_device, oracle, variant, act):
    _case(oracle, cuda_device, ave.NVFP4, 256, 512, 1024, variant, act, True)


@pytest.mark.parametrize("variant", [ave.GEMM_1CTA_N256, ave.GEMM_2CTA_N128, ave.GEMM_2CTA_N256])
@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
def test_bias_only_and_activation_only(cuda_device, oracle, fmt, variant):
    _case(oracle, cuda_device, fmt, 384, 640, 768, variant, "none", True)
    _case(oracle, cuda_device, fmt, 384, 640, 768, variant, "silu", False)


@pytest.mark.parametrize("m,n,k", [(100, 136, 96), (257, 1000, 320)])
def test_ragged_with_epilogue(cuda_device, oracle, m, n, k):
    """The bias read is clipped at N like the stores."""
    for variant in (ave.GEMM_2CTA_N256, ave.GEMM_2CTA_N192, ave.GEMM_1CTA_N128):
        _case(oracle, cuda_device, ave.NVFP4, m, n, k, variant, "gelu", True)


@pytest.mark.parametrize("m,n,k", [(16, 1024, 8192), (8, 384, 1024), (32, 520, 2048), (64, 256, 512)])
@pytest.mark.parametrize("act", ["none", "relu", "silu"])
def test_decode_kernel_with_epilogue(cuda_device, oracle, m, n, k, act):
    """Decode kernel: the bias runs along the weight rows (the tensor core's M axis after the operand swap);
    both the whole-tile and the stream-K partial-sum write-outs apply it."""
    _case(oracle, cuda_device, ave.NVFP4, m, n, k, ave.GEMM_SKINNY, act, True)


def test_argument_errors(cuda_device, oracle):
    a = ave.quantize_nvfp4(inputs.normal_bf16(128, 256, 0).to(cuda_device))
    b = ave.quantize_nvfp4(inputs.normal_bf16(256, 256, 1).to(cuda_device))
    with pytest.raises(ValueError):
        ave.gemm_nvfp4_transposed_b(a, b, activation="tanh")
    with pytest.raises(ValueError):
        ave.gemm_nvfp4_transposed_b(a, b, bias=torch.zeros(255, dtype=torch.bfloat16, device=cuda_device))
    with pytest.raises(ValueError):
        ave.gemm_nvfp4_transposed_b(a, b, bias=torch.zeros(256, dtype=torch.float32, device=cuda_device))


# ------------------------------------------------------------------ quantising epilogue
def _operands(dev, fmt, m, n, k, seed=0):
    quant = ave.quantize_nvfp4 if fmt == ave.NVFP4 else ave.quantize_mxfp4
    A = quant(inputs.make_operand_bf16("normal", m, k, seed).to(dev))
    B = quant(inputs.make_operand_bf16("weight", n, k, seed + 1).to(dev))
    bias = (inputs.normal_bf16(1, n, seed + 2).float() * 0.5).to(torch.bfloat16).reshape(n).to(dev)
    return A, B, bias


@pytest.mark.parametrize("sf_layout", [ave.SF_TILED, ave.SF_ROW_MAJOR])
@pytest.mark.parametrize("variant", [ave.GEMM_AUTO, ave.GEMM_2CTA_N256, ave.GEMM_1CTA_N128, ave.GEMM_2CTA_N192,
                                     ave.GEMM_1CTA_N256, ave.GEMM_2CTA_N128])
@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
@pytest.mark.parametrize("m,n,k", [(384, 640, 768), (100, 224, 96), (16, 512, 1024)])
def test_quantised_result_equals_gemm_then_quantise(cuda_device, fmt, variant, sf_layout, m, n, k):
    """The quantising epilogue must give, byte for byte, what the quantise kernel gives on the bf16 result of the
    same GEMM (bit-exact bar for nibbles and scale bytes), including the zero padding of the tiled scale layout."""
    A, B, bias = _operands(cuda_device, fmt, m, n, k)
    tiled_variant = variant if (variant != ave.GEMM_AUTO or m > 64) else ave.GEMM_1CTA_N128
    ref = _gemm(A, B, fmt, variant=tiled_variant, bias=bias, activation="silu")
    gs = (ref.float().abs().max() / 2688.0).reshape(1) if fmt == ave.NVFP4 else None
    q, d = ave.gemm_quantized_out_transposed_b(A, B, gs, bias=bias, activation="silu", sf_layout=sf_layout,
                                               out_bf16=True, variant=variant)
    ave.check_device_status(cuda_device)
    assert torch.equal(d, ref)
    q2 = ave.quantize_nvfp4(ref, global_scale=gs, sf_layout=sf_layout) if fmt == ave.NVFP4 else ave.quantize_mxfp4(ref, sf_layout=sf_layout)
    assert torch.equal(q.packed, q2.packed), f"{(q.packed != q2.packed).sum().item()} packed bytes differ"
    assert torch.equal(q.scales, q2.scales), f"{(q.scales != q2.scales).sum().item()} scale bytes differ"
    # quantised result only: the bf16 matrix is never written
    q3 = ave.gemm_quantized_out_transposed_b(A, B, gs, bias=bias, activation="silu", sf_layout=sf_layout, variant=variant)
    assert torch.equal(q3.packed, q2.packed) and torch.equal(q3.scales, q2.scales)


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
def test_quantised_result_against_oracle_chain(cuda_device, oracle, fmt):
    """Against the CPU oracle chain GEMM -> act(x + bias) -> bf16 -> quantise.  The accumulation order differs
    (fp32 in tensor memory vs fp64), so a bf16 value can land on the other side of a rounding boundary: the
    bytes agree except for a small fraction, and the dequantised results agree closely."""
    m, n, k = 256, 512, 1024
    a = inputs.make_operand_bf16("normal", m, k, 0)
    b = inputs.make_operand_bf16("weight", n, k, 1)
    qa, qb = oracle.c_quantize(_bits(a), fmt), oracle.c_quantize(_bits(b), fmt)
    d32, _ = oracle.c_gemm_fp4(qa, qb, fmt)
    bias = (inputs.normal_bf16(1, n, 2).float() * 0.5).to(torch.bfloat16).reshape(n)
    y32, ybf = oracle.c_bias_act(d32, _bits(bias), ACTS["gelu"])
    gs = float(np.abs(oracle.bf16_bits_to_f32(ybf)).max() / 2688.0) if fmt == ave.NVFP4 else None
    exp_packed, exp_sf, exp_gs = oracle.c_quantize(ybf, fmt, gs)
    gs_t = torch.tensor([np.float32(exp_gs)], dtype=torch.float32, device=cuda_device) if fmt == ave.NVFP4 else None
    q = ave.gemm_quantized_out_transposed_b(_to_dev(qa, fmt, cuda_device), _to_dev(qb, fmt, cuda_device), gs_t,
                                            bias=bias.to(cuda_device), activation="gelu", sf_layout=ave.SF_ROW_MAJOR)
    ave.check_device_status(cuda_device)
    got_packed, got_sf = q.packed.cpu().numpy(), q.scales.cpu().numpy()
    assert (got_sf != exp_sf).mean() < 2e-3
    assert (got_packed != exp_packed).mean() < 5e-3
    deq_got = oracle.c_dequantize(got_packed, got_sf, exp_gs, fmt)
    deq_exp = oracle.c_dequantize(exp_packed, exp_sf, exp_gs, fmt)
    rel = float(np.linalg.norm(deq_got - deq_exp) / np.linalg.norm(deq_exp))
    assert rel < 2e-2, rel


def test_quantised_result_feeds_next_gemm(cuda_device):
    """Two-layer chain: the quantised result of layer 1 is the A operand of layer 2 and gives the same bf16 output
    as the unfused sequence GEMM -> quantise -> GEMM."""
    m, h, n, k = 256, 512, 384, 768
    A, W1, bias = _operands(cuda_device, ave.NVFP4, m, h, k)
    W2 = ave.quantize_nvfp4(inputs.make_operand_bf16("weight", n, h, 7).to(cuda_device))
    mid = ave.gemm_nvfp4_transposed_b(A, W1, bias=bias, activation="relu")
    gs = (mid.float().abs().max() / 2688.0).reshape(1)
    expect = ave.gemm_nvfp4_transposed_b(ave.quantize_nvfp4(mid, global_scale=gs), W2)
    q = ave.gemm_quantized_out_transposed_b(A, W1, gs, bias=bias, activation="relu")
    got = ave.gemm_nvfp4_transposed_b(q, W2)
    ave.check_device_status(cuda_device)
    assert torch.equal(got, expect)


def test_quantised_result_argument_errors(cuda_device):
    A, B, _ = _operands(cuda_device, ave.NVFP4, 128, 264, 256)   # N = 264 is not a multiple of 16
    gs = torch.ones(1, dtype=torch.float32, device=cuda_device)
    with pytest.raises(ValueError):
        ave.gemm_quantized_out_transposed_b(A, B, gs)
    A, B, _ = _operands(cuda_device, ave.NVFP4, 128, 256, 256)
    with pytest.raises(ValueError):
        ave.gemm_quantized_out_transposed_b(A, B, None)
    with pytest.raises(ValueError):
        ave.gemm_quantized_out_transposed_b(A, B, gs, variant=ave.GEMM_SKINNY)


def test_epilogues_inside_cuda_graph(cuda_device):
    """The fused-epilogue entry points are capturable like the plain operator (the reference benchmark captures its
    operator call the same way, benchmark/gemm/bench_amdgpu_gemm.py:37-41): no allocation, sync or host read inside."""
    A, B, bias = _operands(cuda_device, ave.NVFP4, 256, 512, 1024)
    out = torch.empty((256, 512), dtype=torch.bfloat16, device=cuda_device)
    ref = ave.gemm_nvfp4_transposed_b(A, B, bias=bias, activation="gelu")
    gs = (ref.float().abs().max() / 2688.0).reshape(1)
    qref = ave.quantize_nvfp4(ref, global_scale=gs)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    with torch.cuda.graph(graph, stream=stream):
        ave.gemm_nvfp4_transposed_b(A, B, out=out, bias=bias, activation="gelu")
        q = ave.gemm_quantized_out_transposed_b(A, B, gs, bias=bias, activation="gelu")
    out.zero_()
    q.packed.zero_()
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    ave.check_device_status(cuda_device)
    assert torch.equal(out, ref)
    assert torch.equal(q.packed, qref.packed) and torch.equal(q.scales, qref.scales)


def test_epilogue_golden_fixture(cuda_device, oracle):
    """The kernels against the committed fused-epilogue fixture on the C0 operands (tests/golden/c0_epilogue.npz)."""
    import os

    from conftest import GOLDEN

    z = np.load(os.path.join(GOLDEN, "c0_nvfp4.npz"))
    e = np.load(os.path.join(GOLDEN, "c0_epilogue.npz"))
    A = _to_dev((z["a_packed"], z["a_scales"], float(z["a_gs"])), ave.NVFP4, cuda_device)
    B = _to_dev((z["b_packed"], z["b_scales"], float(z["b_gs"])), ave.NVFP4, cuda_device)
    bias = torch.from_numpy(e["bias"].astype(np.int16)).view(torch.bfloat16).to(cuda_device)
    for name, act, use_bias in (("bias_gelu", "gelu", True), ("bias_silu", "silu", True), ("relu", "relu", False),
                                ("bias_gelu_tanh", "gelu_tanh", True)):
        for variant in (ave.GEMM_2CTA_N256, ave.GEMM_1CTA_N128, ave.GEMM_2CTA_N192):
            out = ave.gemm_nvfp4_transposed_b(A, B, variant=variant, bias=bias if use_bias else None, activation=act)
            _check(out, e["d_" + name], oracle, f"golden {name} variant {variant}")
    gs = torch.tensor([float(e["q_gs"])], dtype=torch.float32, device=cuda_device)
    q = ave.gemm_quantized_out_transposed_b(A, B, gs, bias=bias, activation="gelu", sf_layout=ave.SF_ROW_MAJOR)
    ave.check_device_status(cuda_device)
    assert (q.packed.cpu().numpy() != e["q_packed"]).mean() < 5e-3
    assert (q.scales.cpu().numpy() != e["q_scales"]).mean() < 2e-3
