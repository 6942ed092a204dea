"""GPU tier, collected last: the decode GEMM entry point that allocates nothing.

`ave_fp4_gemm_decode_noalloc` is for hosts that cannot call cudaMalloc (a plugin inside another
runtime's memory pool, a serving loop that must not stall on an allocation): its stream-K
scratch is a fixed array inside the library.  The test calls it through the C ABI twice in a
row and compares with the ordinary entry point (caller-provided workspace), which runs the same
kernel, so the results must be identical bit for bit.
"""
import ctypes

import pytest
import torch

import avelang_b200 as ave
from avelang_b200 import _lib, inputs

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _call_noalloc(L, X, W, out, fmt, dev):
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    return L.ave_fp4_gemm_decode_noalloc(_p(X.packed), _p(X.scales), _p(X.global_scale), _p(W.packed), _p(W.scales),
                                         _p(W.global_scale), _p(out), X.rows, W.rows, X.k, out.stride(0), fmt, stream)


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
def test_noalloc_matches_workspace_entry_point_twice(cuda_device, fmt):
    dev = cuda_device
    L = _lib.ensure_init(dev.index or 0)
    quant = ave.quantize_nvfp4 if fmt == ave.NVFP4 else ave.quantize_mxfp4
    gemm = ave.gemm_nvfp4_transposed_b if fmt == ave.NVFP4 else ave.gemm_mxfp4_transposed_b
    # two different problems back to back: the second call meets whatever the first left in the array
    for m, n, k, seed in ((16, 4096, 8192, 0), (9, 1160, 2080, 3)):
        X = quant(inputs.outlier_activations_bf16(m, k, seed).to(dev))
        W = quant(inputs.normal_bf16(n, k, seed + 1, std=0.02).to(dev))
        want = gemm(X, W, variant=ave.GEMM_SKINNY)
        for _ in range(2):
            got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
            rc = _call_noalloc(L, X, W, got, fmt, dev)
            assert rc == 0, L.ave_fp4_last_error().decode()
            ave.check_device_status(dev)
            assert torch.equal(got, want)


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
def test_noalloc_matches_oracle_many_tiles_short_k(cuda_device, oracle, fmt):
    """Checked against the CPU oracle directly (not only against the sibling entry point), on shapes whose
    stream-K phase has fewer units than there are CTAs, twice in a row on the shared array."""
    import numpy as np

    dev = cuda_device
    L = _lib.ensure_init(dev.index or 0)

    def bits(t):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)

    for m, n, k in ((16, 20480, 2048), (8, 19072, 512)):
        x = inputs.outlier_activations_bf16(m, k, 11)
        w = inputs.normal_bf16(n, k, 12, std=0.02)
        qx, qw = oracle.c_quantize(bits(x), fmt), oracle.c_quantize(bits(w), fmt)
        _, dbf = oracle.c_gemm_fp4(qx, qw, fmt, want_f32=False)
        exp = oracle.bf16_bits_to_f32(dbf)

        def dev_op(q):
            gs = torch.tensor([q[2]], dtype=torch.float32, device=dev) if fmt == ave.NVFP4 else None
            return ave.to_tiled(ave.make_operand(torch.from_numpy(q[0]).to(dev), torch.from_numpy(q[1]).to(dev), gs, fmt))

        X, W = dev_op(qx), dev_op(qw)
        first = None
        for _ in range(2):
            got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
            rc = _call_noalloc(L, X, W, got, fmt, dev)
            assert rc == 0, L.ave_fp4_last_error().decode()
            ave.check_device_status(dev)
            g = got.float().cpu().numpy()
            assert np.isfinite(g).all()
            rel = float(np.linalg.norm(g - exp) / np.linalg.norm(exp))
            assert rel <= 1e-3, f"{m}x{n}x{k} fmt {fmt}: rel_fro {rel:.3e}, max_abs {np.abs(g - exp).max():.4g}"
            first = got if first is None else first
            assert torch.equal(got, first)


def test_noalloc_rejects_shapes_beyond_its_scratch(cuda_device):
    dev = cuda_device
    L = _lib.ensure_init(dev.index or 0)
    X = ave.quantize_nvfp4(inputs.normal_bf16(32, 256, 0).to(dev))
    W = ave.quantize_nvfp4(inputs.normal_bf16(128, 256, 1).to(dev))
    out = torch.empty((32, 128), dtype=torch.bfloat16, device=dev)
    rc = _call_noalloc(L, X, W, out, ave.NVFP4, dev)
    assert rc < 0
    assert b"M <= 16" in L.ave_fp4_last_error()
