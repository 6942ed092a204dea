"""``gemm_pipeline_transposed_b`` under the module name the reference ships it in
(python/avelang_kernels/amdgpu_gemm.py:458-494), served on B200 by the dense bf16 mode of the tcgen05 kernel.
Callers of the reference operator keep their import line."""
from avelang_b200.bf16_gemm import gemm_pipeline_transposed_b  # noqa: F401

__all__ = ["gemm_pipeline_transposed_b"]
