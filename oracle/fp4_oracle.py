"""CPU oracle for the block-scaled FP4 path -- TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this module; the shipped package never does.

PARITY UNPINNED: the reference project has no FP4 code or golden vectors.  The
GEMM half restates the reference's oracle expression
``(A.float() @ B.float().T).to(torch.bfloat16)``
(test/examples/gemm/amdgpu/test_amdgpu_gemm.py:27) on CPU tensors; the quantise /
dequantise half restates the public OCP-MX / NVFP4 formats (see fp4_oracle.c).

Two independent statements of the same arithmetic live here:

* ``c_*``  -- ctypes bindings of ``libfp4_oracle.so`` (plain C, OpenMP);
* ``np_*`` -- a vectorised numpy restatement written separately from the C one,
  used to cross-check it (and, for the GEMM, torch's CPU fp32 matmul).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfp4_oracle.so")

NVFP4 = 0
MXFP4 = 1

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def build(force: bool = False) -> str:
    """Compile the C oracle next to its source (gcc only; seconds)."""
    src = os.path.join(_HERE, "fp4_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libfp4_oracle.so"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, f32, vp, i32 = ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_int
        L.ave_oracle_amax_bf16.restype = f32
        L.ave_oracle_amax_bf16.argtypes = [vp, ctypes.c_size_t]
        L.ave_oracle_global_scale.restype = f32
        L.ave_oracle_global_scale.argtypes = [f32]
        L.ave_oracle_quantize_nvfp4.restype = None
        L.ave_oracle_quantize_nvfp4.argtypes = [vp, i64, i64, i64, f32, vp, vp]
        L.ave_oracle_quantize_mxfp4.restype = None
        L.ave_oracle_quantize_mxfp4.argtypes = [vp, i64, i64, i64, vp, vp]
        L.ave_oracle_dequantize.restype = None
        L.ave_oracle_dequantize.argtypes = [vp, vp, f32, i32, i64, i64, vp]
        L.ave_oracle_gemm_f32.restype = None
        L.ave_oracle_gemm_f32.argtypes = [vp, vp, i64, i64, i64, vp, vp]
        L.ave_oracle_gemm_fp4.restype = i32
        L.ave_oracle_gemm_fp4.argtypes = [vp, vp, f32, vp, vp, f32, i32, i64, i64, i64, vp, vp]
        L.ave_oracle_sf_to_tiled.restype = None
        L.ave_oracle_sf_to_tiled.argtypes = [vp, i64, i64, vp]
        L.ave_oracle_e2m1_code.restype = ctypes.c_uint8
        L.ave_oracle_e2m1_code.argtypes = [f32]
        L.ave_oracle_e4m3_code.restype = ctypes.c_uint8
        L.ave_oracle_e4m3_code.argtypes = [f32]
        L.ave_oracle_e4m3_decode.restype = f32
        L.ave_oracle_e4m3_decode.argtypes = [ctypes.c_uint8]
        L.ave_oracle_f32_to_bf16.restype = ctypes.c_uint16
        L.ave_oracle_f32_to_bf16.argtypes = [f32]
        L.ave_oracle_num_threads.restype = i32
        L.ave_oracle_num_threads.argtypes = []
        L.ave_oracle_set_num_threads.restype = None
        L.ave_oracle_set_num_threads.argtypes = [i32]
        L.ave_oracle_bias_act.restype = None
        L.ave_oracle_bias_act.argtypes = [vp, i64, i64, vp, i32, vp, vp]
        _lib = L
    return _lib


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    assert a.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(a.ctypes.data)


# --------------------------------------------------------------------------- C
def c_amax(x_bf16_bits: np.ndarray) -> float:
    x = np.ascontiguousarray(x_bf16_bits, dtype=np.uint16)
    return float(lib().ave_oracle_amax_bf16(_ptr(x), x.size))


def c_global_scale(amax: float) -> float:
    return float(lib().ave_oracle_global_scale(np.float32(amax)))


def c_quantize(x_bf16_bits: np.ndarray, fmt: int, global_scale: float | None = None):
    """(rows,k) uint16 bf16 bit patterns -> (packed (rows,k/2) u8, scales (rows,k/blk) u8, gs)."""
    x = np.ascontiguousarray(x_bf16_bits, dtype=np.uint16)
    rows, k = x.shape
    blk = 16 if fmt == NVFP4 else 32
    assert k % blk == 0
    packed = np.empty((rows, k // 2), dtype=np.uint8)
    scales = np.empty((rows, k // blk), dtype=np.uint8)
    if fmt == NVFP4:
        gs = c_global_scale(c_amax(x)) if global_scale is None else float(np.float32(global_scale))
        lib().ave_oracle_quantize_nvfp4(_ptr(x), rows, k, k, np.float32(gs), _ptr(packed), _ptr(scales))
    else:
        gs = 1.0
        lib().ave_oracle_quantize_mxfp4(_ptr(x), rows, k, k, _ptr(packed), _ptr(scales))
    return packed, scales, gs


def c_dequantize(packed: np.ndarray, scales: np.ndarray, gs: float, fmt: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    rows, k2 = packed.shape
    out = np.empty((rows, k2 * 2), dtype=np.float32)
    lib().ave_oracle_dequantize(_ptr(packed), _ptr(scales), np.float32(gs), fmt, rows, k2 * 2, _ptr(out))
    return out


def c_gemm_fp4(a, b, fmt: int, want_f32: bool = True):
    """a, b = (packed, scales, gs) triples; returns (d32 (m,n) f32 | None, dbf16 bits (m,n) u16)."""
    ap, asf, ags = a
    bp, bsf, bgs = b
    ap = np.ascontiguousarray(ap, dtype=np.uint8)
    bp = np.ascontiguousarray(bp, dtype=np.uint8)
    asf = np.ascontiguousarray(asf, dtype=np.uint8)
    bsf = np.ascontiguousarray(bsf, dtype=np.uint8)
    m, k = ap.shape[0], ap.shape[1] * 2
    n = bp.shape[0]
    d32 = np.empty((m, n), dtype=np.float32) if want_f32 else None
    dbf = np.empty((m, n), dtype=np.uint16)
    rc = lib().ave_oracle_gemm_fp4(_ptr(ap), _ptr(asf), np.float32(ags), _ptr(bp), _ptr(bsf), np.float32(bgs),
                                   fmt, m, n, k, _ptr(d32) if want_f32 else None, _ptr(dbf))
    if rc != 0:
        raise MemoryError("oracle temporaries")
    return d32, dbf


ACT_NONE, ACT_RELU, ACT_GELU, ACT_GELU_TANH, ACT_SILU = 0, 1, 2, 3, 4


def c_bias_act(d32: np.ndarray, bias_bf16_bits: np.ndarray | None, act: int):
    """Fused-epilogue restatement on the fp32 GEMM result: returns (y f32, y bf16 bits)."""
    d32 = np.ascontiguousarray(d32, dtype=np.float32)
    m, n = d32.shape
    bias = None if bias_bf16_bits is None else np.ascontiguousarray(bias_bf16_bits, dtype=np.uint16)
    if bias is not None and bias.shape != (n,):
        raise ValueError("bias must have n entries")
    y32 = np.empty_like(d32)
    ybf = np.empty((m, n), dtype=np.uint16)
    lib().ave_oracle_bias_act(_ptr(d32), m, n, None if bias is None else _ptr(bias), act, _ptr(y32), _ptr(ybf))
    return y32, ybf


def np_bias_act(d32: np.ndarray, bias_bf16_bits: np.ndarray | None, act: int):
    """Independent numpy restatement of c_bias_act (double arithmetic, math.erf per element for GELU)."""
    import math

    x = d32.astype(np.float64)
    if bias_bf16_bits is not None:
        x = x + bf16_bits_to_f32(bias_bf16_bits).astype(np.float64)[None, :]
    if act == ACT_RELU:
        y = np.maximum(x, 0.0)
    elif act == ACT_GELU:
        y = 0.5 * x * (1.0 + np.vectorize(math.erf)(x / math.sqrt(2.0)))
    elif act == ACT_GELU_TANH:
        y = 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))
    elif act == ACT_SILU:
        y = x / (1.0 + np.exp(-x))
    else:
        y = x
    y32 = y.astype(np.float32)
    return y32, f32_to_bf16_bits(y32)


def c_sf_to_tiled(scales: np.ndarray) -> np.ndarray:
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    rows, ncol = scales.shape
    out = np.empty((((rows + 127) // 128) * ((ncol + 3) // 4) * 512,), dtype=np.uint8)
    lib().ave_oracle_sf_to_tiled(_ptr(scales), rows, ncol, _ptr(out))
    return out


def num_threads() -> int:
    return int(lib().ave_oracle_num_threads())


def set_num_threads(n: int) -> None:
    """OpenMP threads used by the C oracle's loops from now on (a timing leg states its thread count)."""
    lib().ave_oracle_set_num_threads(int(n))


# ----------------------------------------------------------------------- numpy
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def np_e2m1_code(ay: np.ndarray) -> np.ndarray:
    """|y| -> magnitude code 0..7: nearest, ties to even mantissa, saturating at 6."""
    ay = np.asarray(ay, dtype=np.float32)
    # boundaries between codes; a tie belongs to the code whose mantissa bit is 0
    code = np.zeros(ay.shape, dtype=np.uint8)
    code += (ay > np.float32(0.25))
    code += (ay >= np.float32(0.75))
    code += (ay > np.float32(1.25))
    code += (ay >= np.float32(1.75))
    code += (ay > np.float32(2.5))
    code += (ay >= np.float32(3.5))
    code += (ay > np.float32(5.0))
    return code


def np_e4m3_decode(c: np.ndarray) -> np.ndarray:
    c = np.asarray(c, dtype=np.uint8)
    e = ((c >> 3) & 0xF).astype(np.int32)
    m = (c & 7).astype(np.float32)
    sub = np.ldexp(m, -9)
    nor = np.ldexp(np.float32(8.0) + m, e - 10)
    return np.where(e == 0, sub, nor).astype(np.float32)


_E4M3_TABLE = None


def np_e4m3_code(u: np.ndarray) -> np.ndarray:
    """u >= 0 -> nearest E4M3 code (ties to even code), saturating at 448 (0x7E).

    Written as a search over the 127 finite non-negative E4M3 values, which is a
    different method from the bit manipulation in the C oracle.
    """
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        _E4M3_TABLE = np_e4m3_decode(np.arange(0x7F, dtype=np.uint8)).astype(np.float64)
    t = _E4M3_TABLE
    u64 = np.minimum(np.asarray(u, dtype=np.float32).astype(np.float64), 448.0)
    hi = np.clip(np.searchsorted(t, u64, side="left"), 0, 0x7E)
    lo = np.clip(hi - 1, 0, 0x7E)
    dlo = u64 - t[lo]
    dhi = t[hi] - u64
    pick_hi = (dhi < dlo) | ((dhi == dlo) & (hi % 2 == 0))
    return np.where(pick_hi, hi, lo).astype(np.uint8)


def np_quantize(x_bf16_bits: np.ndarray, fmt: int, global_scale: float | None = None):
    x = bf16_bits_to_f32(np.asarray(x_bf16_bits, dtype=np.uint16))
    rows, k = x.shape
    blk = 16 if fmt == NVFP4 else 32
    xb = x.reshape(rows, k // blk, blk)
    a = np.abs(xb).max(axis=2)
    if fmt == NVFP4:
        if global_scale is None:
            T = np.float32(np.abs(x).max()) if x.size else np.float32(0)
            gs = np.float32(1.0) if T == 0 else np.float32(T / np.float32(2688.0))
        else:
            gs = np.float32(global_scale)
        t = (a / np.float32(6.0)).astype(np.float32)
        u = np.minimum((t / gs).astype(np.float32), np.float32(448.0))
        codes = np_e4m3_code(u)
        d = (np_e4m3_decode(codes) * gs).astype(np.float32)
    else:
        gs = np.float32(1.0)
        E = ((a.view(np.uint32) >> 23) & 0xFF).astype(np.int32)
        codes = np.where(a == 0, 127, np.clip(E - 2, 0, 254)).astype(np.uint8)
        d = np.ldexp(np.float32(1.0), codes.astype(np.int32) - 127).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        y = np.abs(xb / d[:, :, None]).astype(np.float32)
    mag = np_e2m1_code(y)
    mag = np.where(d[:, :, None] == 0, 0, mag).astype(np.uint8)
    sign = (np.signbit(xb).astype(np.uint8) << 3)
    nib = (sign | mag).reshape(rows, k)
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    return packed, codes, float(gs)


def np_dequantize(packed: np.ndarray, scales: np.ndarray, gs: float, fmt: int) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint8)
    rows, k2 = packed.shape
    nib = np.empty((rows, k2 * 2), dtype=np.uint8)
    nib[:, 0::2] = packed & 0xF
    nib[:, 1::2] = packed >> 4
    mag = E2M1_VALUES[nib & 7]
    blk = 16 if fmt == NVFP4 else 32
    if fmt == NVFP4:
        s = np.repeat(np_e4m3_decode(scales), blk, axis=1)
        v = ((mag * s).astype(np.float32) * np.float32(gs)).astype(np.float32)
    else:
        s = np.repeat(np.ldexp(np.float32(1.0), np.asarray(scales).astype(np.int32) - 127).astype(np.float32), blk, axis=1)
        v = (mag * s).astype(np.float32)
    return np.where(nib & 8, -v, v).astype(np.float32)


def np_sf_to_tiled(scales: np.ndarray) -> np.ndarray:
    scales = np.asarray(scales, dtype=np.uint8)
    rows, ncol = scales.shape
    rb, cb = (rows + 127) // 128, (ncol + 3) // 4
    pad = np.zeros((rb * 128, cb * 4), dtype=np.uint8)
    pad[:rows, :ncol] = scales
    # (rb, 4 groups of 32 rows, 32, cb, 4) -> (rb, cb, 32, 4 groups, 4)
    t = pad.reshape(rb, 4, 32, cb, 4).transpose(0, 3, 2, 1, 4)
    return np.ascontiguousarray(t).reshape(-1)


def torch_gemm_oracle(a_hat: np.ndarray, b_hat: np.ndarray):
    """The reference's own oracle expression on CPU tensors; returns (f32, bf16 bits)."""
    import torch

    A = torch.from_numpy(np.ascontiguousarray(a_hat))
    B = torch.from_numpy(np.ascontiguousarray(b_hat))
    d32 = A.float() @ B.float().T
    dbf = d32.to(torch.bfloat16)
    return d32.numpy(), dbf.view(torch.int16).numpy().view(np.uint16)
