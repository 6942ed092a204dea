"""CPU tier: the C-ABI library builds, loads and exports what include/ave_fp4.h declares;
host-side argument validation of the operators (no GPU compute calls here)."""
import ctypes
import os
import re

import pytest
import torch

import avelang_b200 as ave
from avelang_b200 import _lib, build, fp4_gemm

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "ave_fp4.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ave_(?:fp4|bf16)_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    declared = _declared_functions()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ave_fp4.h but not exported"
    assert sorted(_lib.EXPORTS) == declared


def test_sf_bytes_is_pure_host_arithmetic(lib):
    assert lib.ave_fp4_sf_bytes(128, 512, 0, 0) == 128 * 32
    assert lib.ave_fp4_sf_bytes(128, 512, 0, 1) == 8 * 512
    assert lib.ave_fp4_sf_bytes(16, 8192, 0, 1) == 128 * 512
    assert lib.ave_fp4_sf_bytes(130, 96, 1, 1) == 2 * 1 * 512
    for rows, k, fmt in ((1, 32, 0), (300, 1024, 1), (8192, 8192, 0)):
        for layout in (0, 1):
            assert lib.ave_fp4_sf_bytes(rows, k, fmt, layout) == fp4_gemm.sf_bytes(rows, k, fmt, layout)


def test_calls_before_init_fail_loudly(lib):
    # no GPU here: there is no current device state, so the call must refuse (never fall back)
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; this checks the no-device path")
    rc = lib.ave_fp4_gemm(None, None, None, None, None, None, None, 128, 128, 128, 128, 0, 0, None, 0, None)
    assert rc != 0
    assert len(lib.ave_fp4_last_error()) > 0
    assert lib.ave_fp4_workspace_bytes(16, 256, 512, 0, 0, 0) < 0


def test_missing_library_raises(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(build, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or library fallback"):
        _lib.load()


def test_quantize_rejects_bad_arguments():
    x = torch.zeros((4, 64), dtype=torch.float32)
    with pytest.raises(ValueError, match="torch.bfloat16"):
        ave.quantize_nvfp4(x)
    with pytest.raises(ValueError, match="CUDA tensor"):
        ave.quantize_nvfp4(x.to(torch.bfloat16))
    with pytest.raises(ValueError, match="2-D"):
        ave.quantize_mxfp4(torch.zeros((64,), dtype=torch.bfloat16))


def _fake_operand(rows, k, fmt, device="cpu"):
    packed = torch.zeros((rows, k // 2), dtype=torch.uint8, device=device)
    blk = 16 if fmt == ave.NVFP4 else 32
    scales = torch.zeros((rows, k // blk), dtype=torch.uint8, device=device)
    gs = torch.ones((1,), dtype=torch.float32, device=device) if fmt == ave.NVFP4 else None
    return ave.make_operand(packed, scales, gs, fmt)


def test_gemm_rejects_bad_arguments():
    A = _fake_operand(128, 256, ave.NVFP4)
    B = _fake_operand(64, 256, ave.NVFP4)
    with pytest.raises(ValueError, match="must be an MXFP4 operand"):
        ave.gemm_mxfp4_transposed_b(A, B)
    with pytest.raises(ValueError, match="share K"):
        ave.gemm_nvfp4_transposed_b(A, _fake_operand(64, 512, ave.NVFP4))
    with pytest.raises(ValueError, match="multiple of 8"):
        ave.gemm_nvfp4_transposed_b(A, _fake_operand(60, 256, ave.NVFP4))
    with pytest.raises(ValueError, match="CUDA tensor"):
        ave.gemm_nvfp4_transposed_b(A, B)
    with pytest.raises(ValueError, match="scales must be uint8"):
        ave.make_operand(torch.zeros((4, 32), dtype=torch.uint8), torch.zeros((4, 3), dtype=torch.uint8), None, ave.MXFP4)


def test_inputs_are_deterministic():
    from avelang_b200 import inputs

    a = inputs.normal_bf16(8, 64, seed=3)
    assert torch.equal(a, inputs.normal_bf16(8, 64, seed=3))
    assert not torch.equal(a, inputs.normal_bf16(8, 64, seed=4))
    x = inputs.outlier_activations_bf16(16, 8192, seed=0)
    big = (x.float().abs().mean(dim=0) > 10).sum().item()
    assert big == 8  # round(0.001 * 8192) outlier channels, the same columns for every row
    t = inputs.student_t3_bf16(64, 256, seed=1)
    assert torch.isfinite(t.float()).all() and t.float().abs().max() > 4
    w = inputs.make_operand_bf16("weight", 64, 256, seed=2)
    assert 0.015 < w.float().std().item() < 0.025


def test_make_operand_accepts_torch_fp4_fp8_views():
    if not hasattr(torch, "float4_e2m1fn_x2") or not hasattr(torch, "float8_e8m0fnu"):
        pytest.skip("this torch has no fp4 / e8m0 view dtypes")
    packed = torch.arange(4 * 32, dtype=torch.uint8).reshape(4, 32)
    sc_nv = torch.full((4, 4), 0x38, dtype=torch.uint8)
    op = ave.make_operand(packed.view(torch.float4_e2m1fn_x2), sc_nv.view(torch.float8_e4m3fn), torch.ones(1), ave.NVFP4)
    assert op.packed.dtype == torch.uint8 and op.scales.dtype == torch.uint8 and op.shape == (4, 64)
    assert torch.equal(op.packed, packed)
    sc_mx = torch.full((4, 2), 127, dtype=torch.uint8)
    op = ave.make_operand(packed.view(torch.float4_e2m1fn_x2), sc_mx.view(torch.float8_e8m0fnu), None, ave.MXFP4)
    assert op.scales.dtype == torch.uint8 and op.k == 64


def test_gemm_rejects_n_not_multiple_of_8_before_any_launch(lib):
    """The write-out moves 8-column (16-byte) chunks, so a C-ABI caller with N % 8 != 0 must get a negative
    return code instead of up to 7 columns written past N (the Python operators reject it earlier still)."""
    dummy = ctypes.c_void_p(4096)   # never dereferenced: the argument check comes first
    for entry in ("ave_fp4_gemm", "ave_fp4_gemm_epilogue"):
        args = [dummy, dummy, None, dummy, dummy, None, dummy, 128, 132, 256, 136, 1, 0, None, 0, None]
        if entry == "ave_fp4_gemm_epilogue":
            args.append(None)
        rc = getattr(lib, entry)(*args)
        assert rc == -1, rc
        assert b"N must be a multiple of 8" in lib.ave_fp4_last_error()
    peers = (ctypes.c_void_p * 1)(4096)
    rc = lib.ave_fp4_gemm_allgather(dummy, dummy, None, dummy, dummy, None, dummy, peers, 1, 128, 132, 256, 136, 1, 0, None)
    assert rc == -1 and b"N must be a multiple of 8" in lib.ave_fp4_last_error()


def test_operators_are_importable_under_the_reference_package_name():
    """`python/avelang_kernels/` mirrors the reference's package layout (python/avelang_kernels/amdgpu_gemm.py)."""
    import importlib
    import sys

    sys.path.insert(0, os.path.join(ROOT, "python"))
    try:
        nv = importlib.import_module("avelang_kernels.nvfp4_gemm")
        amd = importlib.import_module("avelang_kernels.amdgpu_gemm")
    finally:
        sys.path.remove(os.path.join(ROOT, "python"))
    assert nv.gemm_nvfp4_transposed_b is ave.gemm_nvfp4_transposed_b
    assert nv.quantize_mxfp4 is ave.quantize_mxfp4 and nv.linear_nvfp4_decode is ave.linear_nvfp4_decode
    from avelang_b200 import bf16_gemm

    assert amd.gemm_pipeline_transposed_b is bf16_gemm.gemm_pipeline_transposed_b
    with pytest.raises(ValueError, match="torch.bfloat16"):
        amd.gemm_pipeline_transposed_b(torch.zeros((128, 64)), torch.zeros((128, 64), dtype=torch.bfloat16))


def test_native_module_builds_loads_and_forwards_to_the_c_abi(lib):
    """python/src/avefp4_shim.cc: the pybind11 form of the binding (the reference keeps its native module in
    python/src as well).  No GPU here: host arithmetic must agree with the C ABI and a launch must fail loudly."""
    import importlib
    import sys

    build.build_shim()
    sys.path.insert(0, os.path.join(ROOT, "python"))
    try:
        S = importlib.import_module("avelang_kernels._avefp4_shim")
    finally:
        sys.path.remove(os.path.join(ROOT, "python"))
    for name in ("init", "gemm", "quantize", "quantize_nvfp4_dynamic", "linear_decode", "bf16_gemm", "check", "sf_bytes",
                 "workspace_bytes", "linear_decode_workspace_bytes", "last_error", "sm_count"):
        assert hasattr(S, name), name
    for rows, k, fmt, layout in ((128, 512, 0, 1), (130, 96, 1, 1), (16, 8192, 0, 0)):
        assert S.sf_bytes(rows, k, fmt, layout) == lib.ave_fp4_sf_bytes(rows, k, fmt, layout)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="ave-lang Error"):
            S.gemm(4096, 4096, 0, 4096, 4096, 0, 4096, 128, 128, 128, 128, 0)
