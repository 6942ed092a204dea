"""GPU tier: failure detection without any fault.  Every device-side wait in this library is bounded and
ends in a status word the host reads; the self-test kernel makes one such wait run out (a barrier that
nothing arrives on, 2 ms limit) and the host must see the code, after which the device is still usable.
Also: guard bands around the output stay untouched for ragged shapes."""
import ctypes

import numpy as np
import pytest
import torch

import avelang_b200 as ave
from avelang_b200 import _lib, inputs

pytestmark = pytest.mark.gpu


def test_bounded_wait_reports_status_and_context_survives(cuda_device):
    dev = cuda_device
    L = _lib.ensure_init(dev.index or 0)
    ave.check_device_status(dev)                       # clean to start with
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    assert L.ave_fp4_selftest_wait_timeout(2000, stream) == 0
    with pytest.raises(RuntimeError, match="status 104"):
        ave.check_device_status(dev)
    ave.check_device_status(dev)                       # the word was cleared by the failed check
    assert L.ave_fp4_selftest_wait_timeout(0, stream) < 0      # argument error, nothing launched
    # the context is intact: a normal GEMM still runs and checks clean
    A = ave.quantize_nvfp4(inputs.normal_bf16(128, 256, 0).to(dev))
    B = ave.quantize_nvfp4(inputs.normal_bf16(128, 256, 1).to(dev))
    d = ave.gemm_nvfp4_transposed_b(A, B)
    ave.check_device_status(dev)
    assert torch.isfinite(d.float()).all()


@pytest.mark.parametrize("m,n,k,variant", [(100, 136, 96, ave.GEMM_2CTA_N256), (130, 200, 288, ave.GEMM_2CTA_N192),
                                           (257, 264, 2080, ave.GEMM_1CTA_N128), (9, 136, 544, ave.GEMM_SKINNY)])
def test_output_guard_bands_untouched(cuda_device, m, n, k, variant):
    dev = cuda_device
    A = ave.quantize_nvfp4(inputs.normal_bf16(m, k, 0).to(dev))
    B = ave.quantize_nvfp4(inputs.normal_bf16(n, k, 1).to(dev))
    pad = 16
    canary = 12345.0
    buf = torch.full((m + 2 * pad, n + 2 * pad), canary, dtype=torch.bfloat16, device=dev)
    out = buf[pad:pad + m, pad:pad + n]
    ave.gemm_nvfp4_transposed_b(A, B, out=out, variant=variant)
    ave.check_device_status(dev)
    ref = ave.gemm_nvfp4_transposed_b(A, B, variant=variant)
    assert torch.equal(out, ref)
    mask = torch.ones_like(buf, dtype=torch.bool)
    mask[pad:pad + m, pad:pad + n] = False
    assert bool((buf[mask] == canary).all())
