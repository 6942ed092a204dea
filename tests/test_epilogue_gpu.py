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
    _case(oracle, cuda_device, ave.NVFP4, m, n, k, ave.GEMM_AUTO, act, True)


def test_argument_errors(cuda_device, oracle):
    a = ave.quantize_nvfp4(inputs.normal_bf16(128, 256, 0).to(cuda_device))
    b = ave.quantize_nvfp4(inputs.normal_bf16(256, 256, 1).to(cuda_device))
    with pytest.raises(ValueError):
        ave.gemm_nvfp4_transposed_b(a, b, activation="tanh")
    with pytest.raises(ValueError):
        ave.gemm_nvfp4_transposed_b(a, b, bias=torch.zeros(255, dtype=torch.bfloat16, device=cuda_device))
    with pytest.raises(ValueError):
        ave.gemm_nvfp4_transposed_b(a, b, bias=torch.zeros(256, dtype=torch.float32, device=cuda_device))
