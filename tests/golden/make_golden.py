"""Generates the committed golden fixtures from the CPU oracle.

Run from the repository root:  python tests/golden/make_golden.py

The reference project holds no FP4 vectors, so these are produced by the C oracle
(oracle/fp4_oracle.c) and cross-checked, at generation time, against the separate numpy
restatement and ml_dtypes element casts; the script refuses to write if they disagree.

Files written next to this script:
  known_answers.json   element / scale rounding at every threshold and tie, saturation, subnormals
  small_cases.npz      tiny end-to-end cases with stored inputs (one-hot, outlier channel, heavy tail, zeros)
  c0_nvfp4.npz         the 128x256x512 NVFP4 case with seed-0 inputs: quantised operands and bf16 result
  c0_epilogue.npz      the same case through the fused epilogues: bias, act(x + bias) as bf16, and the result quantised to NVFP4
"""
import hashlib
import json
import os
import sys

import ml_dtypes
import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from avelang_b200 import inputs  # noqa: E402
from oracle import fp4_oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def bits_of(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def known_answers() -> dict:
    L = O.lib()
    e2m1_in = [0.0, 0.1, 0.25, 0.2500001, 0.5, 0.7499999, 0.75, 1.0, 1.25, 1.2500001, 1.5, 1.7499999, 1.75, 2.0, 2.5,
               2.5000002, 3.0, 3.4999998, 3.5, 4.0, 5.0, 5.0000005, 6.0, 7.0, 8.0, 1e9]
    e2m1_in = [float(np.float32(v)) for v in e2m1_in]
    e2m1_out = [int(L.ave_oracle_e2m1_code(np.float32(v))) for v in e2m1_in]
    ml = (np.array(e2m1_in, dtype=np.float32).astype(ml_dtypes.float4_e2m1fn).view(np.uint8) & 7).tolist()
    assert ml == e2m1_out, "E2M1 rounding disagrees with ml_dtypes"
    assert O.np_e2m1_code(np.array(e2m1_in, dtype=np.float32)).tolist() == e2m1_out

    table = O.np_e4m3_decode(np.arange(0x7F, dtype=np.uint8)).astype(np.float64)
    mids = ((table[:-1] + table[1:]) / 2).astype(np.float32)
    e4m3_in = np.concatenate([
        table.astype(np.float32), mids, np.nextafter(mids, np.float32(0)), np.nextafter(mids, np.float32(1e9)),
        np.array([448.0, 449.0, 464.0, 465.0, 1000.0, 3e38, 2.0 ** -9, 2.0 ** -10, 2.0 ** -10 * 1.0001, 2.0 ** -11, 1e-30],
                 dtype=np.float32)]).astype(np.float32)
    e4m3_out = np.array([L.ave_oracle_e4m3_code(np.float32(v)) for v in e4m3_in], dtype=np.uint8)
    assert np.array_equal(e4m3_out, O.np_e4m3_code(e4m3_in)), "E4M3 rounding: C and numpy disagree"
    ml8 = np.minimum(e4m3_in, np.float32(448)).astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    assert np.array_equal(e4m3_out, ml8), "E4M3 rounding disagrees with ml_dtypes (after clamping to 448)"

    # E8M0 shared exponent (floor rule): block amax -> code
    e8_in = [0.0, 1.0, 1.5, 1.9999999, 2.0, 3.0, 4.0, 5.9, 6.0, 7.9, 8.0, 0.02, 1e-38, 1e-40, 2.0 ** -126, 2.0 ** -125,
             3e38, 448.0]
    e8_out = []
    for v in e8_in:
        row = np.zeros((1, 32), dtype=np.float32)
        row[0, 5] = v
        _, sc, _ = O.c_quantize(O.f32_to_bf16_bits(row), O.MXFP4)
        e8_out.append(int(sc[0, 0]))
    return {
        "e2m1": {"abs_value": e2m1_in, "code": e2m1_out},
        "e4m3": {"value_f32_bits": e4m3_in.view(np.uint32).tolist(), "code": e4m3_out.tolist()},
        "e8m0_block_amax": {"amax": [float(np.float32(v)) for v in e8_in], "code": e8_out},
    }


def small_cases() -> dict:
    out = {}
    rng = np.random.default_rng(7)

    def add(name, a_f32, b_f32, fmt):
        a = O.f32_to_bf16_bits(a_f32.astype(np.float32))
        b = O.f32_to_bf16_bits(b_f32.astype(np.float32))
        qa, qb = O.c_quantize(a, fmt), O.c_quantize(b, fmt)
        na, nb = O.np_quantize(a, fmt), O.np_quantize(b, fmt)
        for x, y in ((qa, na), (qb, nb)):
            assert np.array_equal(x[0], y[0]) and np.array_equal(x[1], y[1]) and np.float32(x[2]) == np.float32(y[2]), name
        d32, dbf = O.c_gemm_fp4(qa, qb, fmt)
        t32, _ = O.torch_gemm_oracle(O.np_dequantize(*qa, fmt), O.np_dequantize(*qb, fmt))
        den = np.linalg.norm(t32) or 1.0
        assert np.linalg.norm(d32 - t32) / den < 1e-5, name
        pre = f"{name}__"
        out.update({pre + "a": a, pre + "b": b, pre + "a_packed": qa[0], pre + "a_scales": qa[1],
                    pre + "a_gs": np.float32(qa[2]), pre + "b_packed": qb[0], pre + "b_scales": qb[1],
                    pre + "b_gs": np.float32(qb[2]), pre + "d_bf16": dbf, pre + "fmt": np.int32(fmt)})

    for fmt, tag in ((O.NVFP4, "nvfp4"), (O.MXFP4, "mxfp4")):
        m, n, k = 32, 64, 128
        # one-hot rows/columns: pins nibble order and scale placement
        a = np.zeros((m, k)); b = np.zeros((n, k))
        for i in range(m):
            a[i, (i * 5) % k] = 1.0 + (i % 4)
        for j in range(n):
            b[j, (j * 3) % k] = -0.5 * (1 + j % 5)
        add(f"onehot_{tag}", a, b, fmt)
        # gaussian
        add(f"gauss_{tag}", rng.standard_normal((m, k)), rng.standard_normal((n, k)) * 0.02, fmt)
        # outlier channels: a few K columns scaled x50
        a = rng.standard_normal((16, 256)); a[:, [3, 77, 200]] *= 50.0
        add(f"outlier_{tag}", a, rng.standard_normal((32, 256)) * 0.02, fmt)
        # heavy tail (Student-t 3) to exercise saturation and the scale range
        a = rng.standard_t(3, size=(16, 256))
        add(f"heavytail_{tag}", a, rng.standard_normal((32, 256)) * 0.02, fmt)
        # zero blocks, an all-zero row, negative zero, tiny and huge magnitudes
        a = rng.standard_normal((16, 128)); a[2] = 0; a[3, 32:64] = 0; a[4, 0] = -0.0; a[5] *= 1e-20; a[6] *= 1e10
        add(f"edge_{tag}", a, rng.standard_normal((16, 128)), fmt)
    return out


def c0_case() -> dict:
    m, n, k = 128, 256, 512
    A = inputs.normal_bf16(m, k, seed=0)
    B = inputs.normal_bf16(n, k, seed=1)
    a, b = bits_of(A), bits_of(B)
    qa, qb = O.c_quantize(a, O.NVFP4), O.c_quantize(b, O.NVFP4)
    na, nb = O.np_quantize(a, O.NVFP4), O.np_quantize(b, O.NVFP4)
    assert np.array_equal(qa[0], na[0]) and np.array_equal(qa[1], na[1]) and np.array_equal(qb[0], nb[0]) and np.array_equal(qb[1], nb[1])
    d32, dbf = O.c_gemm_fp4(qa, qb, O.NVFP4)
    t32, tbf = O.torch_gemm_oracle(O.c_dequantize(*qa, O.NVFP4), O.c_dequantize(*qb, O.NVFP4))
    assert np.linalg.norm(d32 - t32) / np.linalg.norm(t32) < 1e-5
    return {
        "a_sha256": hashlib.sha256(a.tobytes()).hexdigest(), "b_sha256": hashlib.sha256(b.tobytes()).hexdigest(),
        "a_packed": qa[0], "a_scales": qa[1], "a_gs": np.float32(qa[2]),
        "b_packed": qb[0], "b_scales": qb[1], "b_gs": np.float32(qb[2]), "d_bf16": dbf,
    }


def epilogue_case(c0: dict) -> dict:
    """Fused-epilogue expectations on the C0 operands: the C restatement, cross-checked against the numpy one."""
    qa = (c0["a_packed"], c0["a_scales"], float(c0["a_gs"]))
    qb = (c0["b_packed"], c0["b_scales"], float(c0["b_gs"]))
    d32, _ = O.c_gemm_fp4(qa, qb, O.NVFP4)
    n = d32.shape[1]
    bias = bits_of((inputs.normal_bf16(1, n, seed=2).float() * float(np.abs(d32).mean())).to(torch.bfloat16).reshape(n))
    out = {"bias": bias}
    for name, act, use_bias in (("bias_gelu", O.ACT_GELU, True), ("bias_silu", O.ACT_SILU, True), ("relu", O.ACT_RELU, False),
                                ("bias_gelu_tanh", O.ACT_GELU_TANH, True)):
        y32, ybf = O.c_bias_act(d32, bias if use_bias else None, act)
        n32, nbf = O.np_bias_act(d32, bias if use_bias else None, act)
        assert np.allclose(y32, n32, rtol=3e-7, atol=1e-9), name
        assert ((ybf != nbf) & (np.abs(y32) > 1e-6)).mean() < 1e-3, name
        out["d_" + name] = ybf
    # the quantising epilogue: bias + gelu, bf16, then NVFP4 with a static tensor scale (amax / 2688 of that result)
    ybf = out["d_bias_gelu"]
    gs = O.c_global_scale(O.c_amax(ybf))
    qp, qs, qg = O.c_quantize(ybf, O.NVFP4, gs)
    np_p, np_s, _ = O.np_quantize(ybf, O.NVFP4, gs)
    assert np.array_equal(qp, np_p) and np.array_equal(qs, np_s)
    out.update({"q_gs": np.float32(qg), "q_packed": qp, "q_scales": qs})
    return out


def main() -> None:
    with open(os.path.join(HERE, "known_answers.json"), "w") as f:
        json.dump(known_answers(), f, indent=1)
    np.savez_compressed(os.path.join(HERE, "small_cases.npz"), **small_cases())
    c0 = c0_case()
    np.savez_compressed(os.path.join(HERE, "c0_nvfp4.npz"), **c0)
    np.savez_compressed(os.path.join(HERE, "c0_epilogue.npz"), **epilogue_case(c0))
    for fn in ("known_answers.json", "small_cases.npz", "c0_nvfp4.npz", "c0_epilogue.npz"):
        print(fn, os.path.getsize(os.path.join(HERE, fn)), "bytes")


if __name__ == "__main__":
    main()
