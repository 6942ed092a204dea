"""Operator entry points under the reference's package name.

causalflow-ai/avelang ships its library kernels as ``avelang_kernels.<module>`` (one module today:
python/avelang_kernels/amdgpu_gemm.py).  With this directory's parent (``python/``) on ``sys.path`` the same import
paths resolve to the B200 implementation:

    from avelang_kernels.nvfp4_gemm import quantize_nvfp4, gemm_nvfp4_transposed_b
    from avelang_kernels.amdgpu_gemm import gemm_pipeline_transposed_b      # bf16, same signature as the reference

    from avelang_kernels.native import gemm_fp4_transposed_b                # the same operator through the pybind11 module

The first two modules re-export ``avelang_b200`` (ctypes binding); ``native`` goes through ``_avefp4_shim``, the pybind11
module built from python/src/avefp4_shim.cc.  All compute is in ``libavefp4.so`` behind the C ABI of include/ave_fp4.h.
"""
import os
import sys

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:       # the repository root holds the avelang_b200 package
    sys.path.insert(0, _ROOT)
