"""GPU tier: the quantise kernels (through the C ABI) against the CPU oracle, bit for bit.

Pattern follows the reference's bit-exact packed-conversion test
(test/primitives/jit/test_amdgpu_packed_f8_conversion.py:34-36,55-64): integer results
are compared with exact equality.
"""
import os

import numpy as np
import pytest
import torch

import avelang_b200 as ave
from avelang_b200 import inputs
from conftest import GOLDEN

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _q(x, fmt, layout, gs=None):
    if fmt == ave.NVFP4:
        return ave.quantize_nvfp4(x, global_scale=gs, sf_layout=layout)
    return ave.quantize_mxfp4(x, sf_layout=layout)


CASES = [
    ("normal", 128, 512), ("normal", 16, 8192), ("outlier", 16, 8192), ("weight", 300, 1024),
    ("student_t3", 257, 2080), ("normal", 1, 32), ("normal", 3, 96), ("normal", 1000, 4096), ("normal", 129, 1056),
]


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
@pytest.mark.parametrize("kind,rows,k", CASES)
def test_quantize_bit_exact(cuda_device, oracle, fmt, kind, rows, k):
    x = inputs.make_operand_bf16(kind, rows, k, seed=3)
    if rows >= 8:
        x[1] = 0            # all-zero row
        x[2, :32] = 0       # zero block
        x[3, 0] = -0.0      # negative zero keeps its sign
    ep, es, eg = oracle.c_quantize(_bits(x), fmt)
    xd = x.to(cuda_device)
    q = _q(xd, fmt, ave.SF_ROW_MAJOR)
    qt = _q(xd, fmt, ave.SF_TILED)
    ave.check_device_status(cuda_device)
    assert np.array_equal(q.packed.cpu().numpy(), ep)
    assert np.array_equal(q.scales.cpu().numpy(), es)
    if fmt == ave.NVFP4:
        assert np.float32(q.global_scale.item()) == np.float32(eg)
    assert np.array_equal(qt.packed.cpu().numpy(), ep)
    assert np.array_equal(qt.scales.cpu().numpy(), oracle.np_sf_to_tiled(es))
    assert np.array_equal(ave.to_tiled(q).scales.cpu().numpy(), oracle.np_sf_to_tiled(es))


def test_quantize_static_scale_and_strided_rows(cuda_device, oracle):
    x = inputs.normal_bf16(64, 512, seed=5)
    gs = torch.tensor([0.0123], dtype=torch.float32, device=cuda_device)
    q = ave.quantize_nvfp4(x.to(cuda_device), global_scale=gs, sf_layout=ave.SF_ROW_MAJOR)
    ep, es, _ = oracle.c_quantize(_bits(x), oracle.NVFP4, global_scale=0.0123)
    assert np.array_equal(q.packed.cpu().numpy(), ep) and np.array_equal(q.scales.cpu().numpy(), es)
    # a K-contiguous view with a larger row stride
    wide = inputs.normal_bf16(32, 1024, seed=6).to(cuda_device)
    view = wide[:, 256:768]
    q2 = ave.quantize_mxfp4(view, sf_layout=ave.SF_ROW_MAJOR)
    ep2, es2, _ = oracle.c_quantize(_bits(wide.cpu()[:, 256:768]), oracle.MXFP4)
    assert np.array_equal(q2.packed.cpu().numpy(), ep2) and np.array_equal(q2.scales.cpu().numpy(), es2)


def test_quantize_all_zero_tensor(cuda_device, oracle):
    x = torch.zeros((16, 64), dtype=torch.bfloat16)
    for fmt in (ave.NVFP4, ave.MXFP4):
        q = _q(x.to(cuda_device), fmt, ave.SF_ROW_MAJOR)
        ep, es, eg = oracle.c_quantize(_bits(x), fmt)
        assert np.array_equal(q.packed.cpu().numpy(), ep) and np.array_equal(q.scales.cpu().numpy(), es)
        if fmt == ave.NVFP4:
            assert q.global_scale.item() == 1.0 == eg


def test_quantize_empty(cuda_device):
    x = torch.zeros((0, 64), dtype=torch.bfloat16, device=cuda_device)
    q = ave.quantize_mxfp4(x)
    assert q.packed.shape == (0, 32)


def test_quantize_matches_golden_fixture(cuda_device):
    z = np.load(os.path.join(GOLDEN, "small_cases.npz"))
    names = sorted({k.split("__")[0] for k in z.files})
    for name in names:
        g = {k.split("__")[1]: z[k] for k in z.files if k.startswith(name + "__")}
        fmt = int(g["fmt"])
        for side in ("a", "b"):
            x = torch.from_numpy(g[side].view(np.int16)).view(torch.bfloat16).to(cuda_device)
            q = _q(x, fmt, ave.SF_ROW_MAJOR)
            assert np.array_equal(q.packed.cpu().numpy(), g[side + "_packed"]), name
            assert np.array_equal(q.scales.cpu().numpy(), g[side + "_scales"]), name
            if fmt == ave.NVFP4:
                assert np.float32(q.global_scale.item()) == g[side + "_gs"], name


def test_quantize_full_size_properties(cuda_device, oracle):
    """8192 x 8192 (the square config's operand): idempotence of the scale bytes under
    re-quantising the dequantised values is not guaranteed by the format, so the
    size-independent checks are: a row sample equals the oracle exactly, and the whole
    output equals quantising the two halves separately with the same tensor scale."""
    x = inputs.normal_bf16(8192, 8192, seed=0).to(cuda_device)
    q = ave.quantize_nvfp4(x, sf_layout=ave.SF_ROW_MAJOR)
    gs = q.global_scale
    top = ave.quantize_nvfp4(x[:4096], global_scale=gs, sf_layout=ave.SF_ROW_MAJOR)
    bot = ave.quantize_nvfp4(x[4096:], global_scale=gs, sf_layout=ave.SF_ROW_MAJOR)
    assert torch.equal(q.packed[:4096], top.packed) and torch.equal(q.packed[4096:], bot.packed)
    assert torch.equal(q.scales[:4096], top.scales) and torch.equal(q.scales[4096:], bot.scales)
    rows = torch.tensor([0, 1, 127, 128, 4095, 4096, 8191])
    xs = x[rows.to(cuda_device)].cpu()
    ep, es, _ = oracle.c_quantize(_bits(xs), oracle.NVFP4, global_scale=float(gs.item()))
    assert np.array_equal(q.packed[rows.to(cuda_device)].cpu().numpy(), ep)
    assert np.array_equal(q.scales[rows.to(cuda_device)].cpu().numpy(), es)
    amax = x.float().abs().max().item()
    assert np.float32(gs.item()) == np.float32(np.float32(amax) / np.float32(2688.0))


def test_quantize_full_8192_bit_exact(cuda_device, oracle):
    """Every byte of the 8192 x 8192 quantise (67 M elements) against the C oracle, both formats."""
    x = inputs.normal_bf16(8192, 8192, seed=0)
    xd = x.to(cuda_device)
    for fmt in (ave.NVFP4, ave.MXFP4):
        q = _q(xd, fmt, ave.SF_ROW_MAJOR)
        ep, es, eg = oracle.c_quantize(_bits(x), fmt)
        assert np.array_equal(q.scales.cpu().numpy(), es)
        assert np.array_equal(q.packed.cpu().numpy(), ep)


@pytest.mark.parametrize("gs", [1.0, 0.0123, 5.9604645e-08 * 1.9999999, 1e-36, 3e-39, 1e30, 1.1754942e-38])
def test_quantize_static_scales_fuzz(cuda_device, oracle, gs):
    """Static tensor scales, including one whose significand is all ones, tiny, subnormal and huge ones,
    on rows spanning 60 orders of magnitude: the division shortcuts must agree with IEEE division."""
    rng = np.random.default_rng(1)
    base = rng.standard_normal((512, 1024)).astype(np.float32)
    row_scale = np.float32(10.0) ** rng.uniform(-30, 30, size=(512, 1)).astype(np.float32)
    with np.errstate(over="ignore"):
        base *= row_scale * np.float32(gs if gs > 1e-30 else 1e-30)
    base = np.clip(base, -3e38, 3e38)   # NaN / Inf inputs are outside the contract
    x = torch.from_numpy(base).to(torch.bfloat16)
    x[0] = 0
    g = torch.tensor([gs], dtype=torch.float32, device=cuda_device)
    q = ave.quantize_nvfp4(x.to(cuda_device), global_scale=g, sf_layout=ave.SF_ROW_MAJOR)
    ep, es, _ = oracle.c_quantize(_bits(x), oracle.NVFP4, global_scale=float(np.float32(gs)))
    assert np.array_equal(q.scales.cpu().numpy(), es)
    assert np.array_equal(q.packed.cpu().numpy(), ep)


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
def test_quantize_signed_zeros_and_tiny_values(cuda_device, oracle, fmt):
    """Zeros of both signs, bf16 subnormals and values far below the block scale, scattered through blocks whose
    scale is not zero: the nibble keeps the sign of x even when the magnitude rounds to zero."""
    g = torch.Generator().manual_seed(11)
    x = torch.randn((64, 1024), generator=g)
    pick = torch.rand((64, 1024), generator=g)
    x[pick < 0.10] = 0.0
    x[(pick >= 0.10) & (pick < 0.20)] = -0.0
    x[(pick >= 0.20) & (pick < 0.25)] = 1e-39          # bf16 subnormal
    x[(pick >= 0.25) & (pick < 0.30)] = -1e-39
    x[(pick >= 0.30) & (pick < 0.35)] *= 1e-6
    x = x.to(torch.bfloat16)
    assert (x.view(torch.int16) == -32768).any()        # -0 survived the cast
    ep, es, eg = oracle.c_quantize(_bits(x), fmt)
    q = _q(x.to(cuda_device), fmt, ave.SF_ROW_MAJOR)
    ave.check_device_status(cuda_device)
    assert np.array_equal(q.packed.cpu().numpy(), ep)
    assert np.array_equal(q.scales.cpu().numpy(), es)
