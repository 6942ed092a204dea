"""GPU tier: the reference operator ``gemm_pipeline_transposed_b`` (bf16) on B200, tested the way the
reference tests it (test/examples/gemm/amdgpu/test_amdgpu_gemm.py:15-38: seed 0, randn bf16 operands,
oracle ``(A.float() @ B.float().T).to(bfloat16)`` compared on the CPU, rtol = atol = 1e-1), with the
oracle evaluated on CPU tensors and a much tighter bound stated next to the reference's own."""
import numpy as np
import pytest
import torch

import avelang_b200 as ave
from avelang_b200.bf16_gemm import gemm_pipeline_transposed_b

pytestmark = pytest.mark.gpu


def _oracle(A, B):
    return (A.float() @ B.float().T).to(dtype=torch.bfloat16, device="cpu")


@pytest.mark.parametrize("variant", [ave.GEMM_AUTO, ave.GEMM_1CTA_N128])
@pytest.mark.parametrize("m,n,k", [(1024, 1024, 1024), (128, 256, 512), (384, 640, 320), (100, 136, 72), (1, 8, 8)])
def test_gemm_pipeline_transposed_b(cuda_device, m, n, k, variant):
    torch.manual_seed(0)
    A = torch.randn((m, k), dtype=torch.bfloat16)
    B = torch.randn((n, k), dtype=torch.bfloat16)
    expected = _oracle(A, B)
    actual = gemm_pipeline_transposed_b(A.to(cuda_device), B.to(cuda_device), variant=variant).cpu()
    ave.check_device_status(cuda_device)
    # the reference's own tolerance ...
    assert torch.allclose(actual, expected, rtol=1e-1, atol=1e-1), f"max abs diff {torch.max(torch.abs(actual - expected))}"
    # ... and the bound this implementation actually meets: fp32 accumulation, one bf16 rounding
    rel = (torch.linalg.norm(actual.float() - expected.float()) / torch.linalg.norm(expected.float())).item()
    assert rel <= 1e-3, rel
    assert (actual != expected).float().mean().item() < 0.02


def test_out_and_validation(cuda_device):
    A = torch.randn((256, 128), dtype=torch.bfloat16, device=cuda_device)
    B = torch.randn((128, 128), dtype=torch.bfloat16, device=cuda_device)
    out = torch.empty((256, 128), dtype=torch.bfloat16, device=cuda_device)
    assert gemm_pipeline_transposed_b(A, B, out=out) is out
    with pytest.raises(ValueError, match="A must have dtype torch.bfloat16"):
        gemm_pipeline_transposed_b(A.float(), B)
    with pytest.raises(ValueError, match="B must have dtype torch.bfloat16"):
        gemm_pipeline_transposed_b(A, B.half())
    with pytest.raises(ValueError, match="out must have shape"):
        gemm_pipeline_transposed_b(A, B, out=torch.empty((256, 256), dtype=torch.bfloat16, device=cuda_device))
    with pytest.raises(ValueError, match="out must have dtype"):
        gemm_pipeline_transposed_b(A, B, out=torch.empty((256, 128), dtype=torch.float16, device=cuda_device))
    with pytest.raises(ValueError, match="out must be on device"):
        gemm_pipeline_transposed_b(A, B, out=torch.empty((256, 128), dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="K must be"):
        gemm_pipeline_transposed_b(A[:, :4].contiguous(), B[:, :4].contiguous())
    # no rows on either side: an empty result, nothing launched
    assert tuple(gemm_pipeline_transposed_b(A[:0], B).shape) == (0, 128)
    assert tuple(gemm_pipeline_transposed_b(A, B[:0]).shape) == (256, 0)


def test_large_8192_against_row_sample(cuda_device):
    torch.manual_seed(0)
    A = torch.randn((8192, 8192), dtype=torch.bfloat16, device=cuda_device)
    B = torch.randn((8192, 8192), dtype=torch.bfloat16, device=cuda_device)
    D = gemm_pipeline_transposed_b(A, B)
    ave.check_device_status(cuda_device)
    rows = torch.tensor([0, 127, 128, 4097, 8191], device=cuda_device)
    expected = _oracle(A[rows].cpu(), B.cpu())
    actual = D[rows].cpu()
    rel = (torch.linalg.norm(actual.float() - expected.float()) / torch.linalg.norm(expected.float())).item()
    assert rel <= 1e-3, rel
    assert torch.equal(gemm_pipeline_transposed_b(A[2048:2304], B), D[2048:2304])
