"""ctypes binding of libavefp4.so (the C ABI in include/ave_fp4.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
Error convention mirrors the reference backend, which turns driver errors into
``RuntimeError("ave-lang Error [CUDA]: ...")`` (python/avelang/backends/nvidia/driver.py:68-81).
"""
from __future__ import annotations

import ctypes
import os
import threading

from . import build as _build

class Epilogue(ctypes.Structure):
    """struct ave_fp4_epilogue of include/ave_fp4.h."""
    _fields_ = [("bias_bf16", ctypes.c_void_p), ("activation", ctypes.c_int32), ("quantize_out", ctypes.c_int32),
                ("q_packed", ctypes.c_void_p), ("q_scales", ctypes.c_void_p), ("q_global_scale", ctypes.c_void_p),
                ("q_sf_layout", ctypes.c_int32), ("reserved", ctypes.c_int32)]


_lock = threading.Lock()
_lib = None
_inited: set[int] = set()

# every symbol include/ave_fp4.h declares
EXPORTS = (
    "ave_fp4_init", "ave_fp4_last_error", "ave_fp4_sf_bytes", "ave_fp4_workspace_bytes", "ave_fp4_amax",
    "ave_fp4_quantize", "ave_fp4_sf_to_tiled", "ave_fp4_gemm", "ave_fp4_check", "ave_fp4_sm_count", "ave_fp4_set_trace",
    "ave_fp4_weight_tiles_bytes", "ave_fp4_pack_weight_tiles", "ave_fp4_gemm_decode_noalloc", "ave_fp4_gemm_allgather", "ave_fp4_quantize_nvfp4_dynamic", "ave_bf16_gemm", "ave_fp4_selftest_wait_timeout",
    "ave_fp4_gemm_epilogue", "ave_fp4_gemm_partials", "ave_fp4_reduce_partials",
    "ave_fp4_linear_decode", "ave_fp4_linear_decode_workspace_bytes", "ave_fp4_gemm_allgather_quantized",
)


def load() -> ctypes.CDLL:
    """Load the shared library (without touching any GPU)."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.LIB_PATH
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m avelang_b200.build` (needs nvcc). "
                "This package has no CPU or library fallback.")
        L = ctypes.CDLL(path)
        i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        L.ave_fp4_init.restype = i32
        L.ave_fp4_init.argtypes = [i32]
        L.ave_fp4_last_error.restype = ctypes.c_char_p
        L.ave_fp4_last_error.argtypes = []
        L.ave_fp4_sf_bytes.restype = i64
        L.ave_fp4_sf_bytes.argtypes = [i64, i64, i32, i32]
        L.ave_fp4_workspace_bytes.restype = i64
        L.ave_fp4_workspace_bytes.argtypes = [i64, i64, i64, i32, i32, i32]
        L.ave_fp4_amax.restype = i32
        L.ave_fp4_amax.argtypes = [vp, i64, i64, i64, vp, vp]
        L.ave_fp4_quantize.restype = i32
        L.ave_fp4_quantize.argtypes = [vp, i64, i64, i64, i32, vp, vp, vp, vp, i32, vp]
        L.ave_fp4_sf_to_tiled.restype = i32
        L.ave_fp4_sf_to_tiled.argtypes = [vp, i64, i64, vp, vp]
        L.ave_fp4_gemm.restype = i32
        L.ave_fp4_gemm.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp, i64, vp]
        L.ave_fp4_gemm_epilogue.restype = i32
        L.ave_fp4_gemm_epilogue.argtypes = L.ave_fp4_gemm.argtypes + [ctypes.POINTER(Epilogue)]
        L.ave_fp4_gemm_partials.restype = i32
        L.ave_fp4_gemm_partials.argtypes = [vp, vp, vp, vp, vp, vp, ctypes.POINTER(vp), i32, i32, i64, i64, i64, i32, vp]
        L.ave_fp4_reduce_partials.restype = i32
        L.ave_fp4_reduce_partials.argtypes = [vp, i32, i64, i64, vp, i64, ctypes.POINTER(Epilogue), vp]
        L.ave_fp4_check.restype = i32
        L.ave_fp4_check.argtypes = [vp]
        L.ave_fp4_sm_count.restype = i32
        L.ave_fp4_sm_count.argtypes = []
        L.ave_fp4_weight_tiles_bytes.restype = i64
        L.ave_fp4_weight_tiles_bytes.argtypes = [i64, i64]
        L.ave_fp4_pack_weight_tiles.restype = i32
        L.ave_fp4_pack_weight_tiles.argtypes = [vp, i64, i64, vp, vp]
        L.ave_fp4_gemm_decode_noalloc.restype = i32
        L.ave_fp4_gemm_decode_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, vp]
        L.ave_fp4_gemm_allgather.restype = i32
        L.ave_fp4_gemm_allgather.argtypes = [vp, vp, vp, vp, vp, vp, vp, ctypes.POINTER(vp), i32, i64, i64, i64, i64, i32, i32, vp]
        L.ave_fp4_quantize_nvfp4_dynamic.restype = i32
        L.ave_fp4_quantize_nvfp4_dynamic.argtypes = [vp, i64, i64, i64, vp, vp, vp, i32, vp, vp]
        L.ave_bf16_gemm.restype = i32
        L.ave_bf16_gemm.argtypes = [vp, vp, vp, i64, i64, i64, i64, i32, vp]
        L.ave_fp4_selftest_wait_timeout.restype = i32
        L.ave_fp4_selftest_wait_timeout.argtypes = [i64, vp]
        L.ave_fp4_linear_decode_workspace_bytes.restype = i64
        L.ave_fp4_linear_decode_workspace_bytes.argtypes = [i64, i64, i64, i32, i32]
        L.ave_fp4_linear_decode.restype = i32
        L.ave_fp4_linear_decode.argtypes = [vp, i64, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp, i64, vp, ctypes.POINTER(Epilogue)]
        L.ave_fp4_gemm_allgather_quantized.restype = i32
        L.ave_fp4_gemm_allgather_quantized.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, ctypes.POINTER(Epilogue), i64, i64,
                                                       ctypes.POINTER(vp), ctypes.POINTER(vp), i32, vp]
        L.ave_fp4_set_trace.restype = i32
        L.ave_fp4_set_trace.argtypes = [vp, i64]
        _lib = L
        return L


def check(rc: int) -> None:
    """Raise for a non-zero return code of the C ABI."""
    if rc != 0:
        msg = load().ave_fp4_last_error().decode("utf-8", "replace")
        if not msg.startswith("ave-lang Error"):
            msg = "ave-lang Error [CUDA]: " + msg
        raise RuntimeError(f"{msg} (code {rc})")


def ensure_init(device_index: int) -> ctypes.CDLL:
    L = load()
    if device_index not in _inited:
        check(L.ave_fp4_init(device_index))
        _inited.add(device_index)
    return L
