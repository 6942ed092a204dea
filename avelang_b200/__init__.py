"""B200-native block-scaled FP4 GEMM + activation quantise behind the avelang operator convention."""
from .fp4_gemm import (  # noqa: F401
    GEMM_1CTA_N128,
    GEMM_1CTA_N256,
    GEMM_2CTA_N128,
    GEMM_2CTA_N192,
    GEMM_2CTA_N256,
    GEMM_AUTO,
    GEMM_SKINNY,
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
    "gemm_quantized_out_transposed_b", "linear_nvfp4_decode", "linear_mxfp4_decode", "make_operand", "pack_weight_tiles", "to_tiled", "check_device_status", "NVFP4", "MXFP4", "SF_ROW_MAJOR", "SF_TILED",
    "GEMM_AUTO", "GEMM_1CTA_N128", "GEMM_1CTA_N256", "GEMM_2CTA_N256", "GEMM_2CTA_N128", "GEMM_2CTA_N192", "GEMM_SKINNY",
]
