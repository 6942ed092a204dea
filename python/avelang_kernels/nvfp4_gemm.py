"""Block-scaled FP4 GEMM operators for sm_100a under the reference's ``avelang_kernels`` package name.

Same convention as ``gemm_pipeline_transposed_b`` (python/avelang_kernels/amdgpu_gemm.py:458-494): A is (M, K), B is
(N, K), both K-contiguous, ``A @ B.T`` with fp32 accumulation and bf16 output, ``ValueError`` before any launch,
``out=`` written in place, asynchronous on torch's current stream.
"""
from avelang_b200.fp4_gemm import (  # noqa: F401
    MXFP4,
    NVFP4,
    SF_ROW_MAJOR,
    SF_TILED,
    Fp4Operand,
    check_device_status,
    gemm_mxfp4_transposed_b,
    gemm_nvfp4_transposed_b,
    gemm_quantized_out_transposed_b,
    linear_mxfp4_decode,
    linear_nvfp4_decode,
    make_operand,
    pack_weight_tiles,
    quantize_mxfp4,
    quantize_nvfp4,
    to_tiled,
)

__all__ = [
    "Fp4Operand", "quantize_nvfp4", "quantize_mxfp4", "gemm_nvfp4_transposed_b", "gemm_mxfp4_transposed_b",
    "gemm_quantized_out_transposed_b", "linear_nvfp4_decode", "linear_mxfp4_decode", "make_operand", "pack_weight_tiles",
    "to_tiled", "check_device_status", "NVFP4", "MXFP4", "SF_ROW_MAJOR", "SF_TILED",
]
