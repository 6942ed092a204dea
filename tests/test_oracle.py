"""CPU tier: the oracle against its committed golden vectors and independent restatements.

The reference pins only the GEMM half of the oracle -- ``(A.float() @ B.float().T).to(bf16)``
(test/examples/gemm/amdgpu/test_amdgpu_gemm.py:27); it has no FP4 vectors, so the
fixtures under tests/golden come from the C oracle, cross-checked here against a
separately written numpy version, ml_dtypes element casts and torch's CPU matmul.
"""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from avelang_b200 import inputs
from conftest import GOLDEN


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


@pytest.fixture(scope="module")
def known():
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        return json.load(f)


def test_e2m1_known_answers(oracle, known):
    vals = np.array(known["e2m1"]["abs_value"], dtype=np.float32)
    want = known["e2m1"]["code"]
    assert [int(oracle.lib().ave_oracle_e2m1_code(np.float32(v))) for v in vals] == want
    assert oracle.np_e2m1_code(vals).tolist() == want
    # ties go to the code with an even mantissa bit; saturation at 6
    table = dict(zip(vals.tolist(), want))
    assert table[0.25] == 0 and table[0.75] == 2 and table[1.25] == 2 and table[1.75] == 4
    assert table[2.5] == 4 and table[3.5] == 6 and table[5.0] == 6 and table[8.0] == 7 and table[1e9] == 7


def test_e4m3_known_answers(oracle, known):
    vals = np.array(known["e4m3"]["value_f32_bits"], dtype=np.uint32).view(np.float32)
    want = np.array(known["e4m3"]["code"], dtype=np.uint8)
    got_c = np.array([oracle.lib().ave_oracle_e4m3_code(np.float32(v)) for v in vals], dtype=np.uint8)
    assert np.array_equal(got_c, want)
    assert np.array_equal(oracle.np_e4m3_code(vals), want)
    assert want.max() == 0x7E  # saturates at 448, never the NaN code 0x7F
    # decode(encode(x)) is the identity on representable values
    codes = np.arange(0x7F, dtype=np.uint8)
    dec = oracle.np_e4m3_decode(codes)
    assert np.array_equal(oracle.np_e4m3_code(dec), codes)
    assert [oracle.lib().ave_oracle_e4m3_decode(int(c)) for c in codes] == dec.tolist()


def test_e4m3_matches_ml_dtypes(oracle):
    import ml_dtypes

    rng = np.random.default_rng(11)
    u = np.concatenate([rng.random(20000) * 448, rng.random(20000) * 0.05, rng.random(5000) * 2.0 ** -8]).astype(np.float32)
    assert np.array_equal(oracle.np_e4m3_code(u), u.astype(ml_dtypes.float8_e4m3fn).view(np.uint8))


def test_e2m1_matches_ml_dtypes(oracle):
    import ml_dtypes

    rng = np.random.default_rng(12)
    y = (rng.random(50000) * 8).astype(np.float32)
    assert np.array_equal(oracle.np_e2m1_code(y), y.astype(ml_dtypes.float4_e2m1fn).view(np.uint8) & 7)


def test_e8m0_known_answers(oracle, known):
    for amax, code in zip(known["e8m0_block_amax"]["amax"], known["e8m0_block_amax"]["code"]):
        row = np.zeros((1, 32), dtype=np.float32)
        row[0, 5] = amax
        bits = oracle.f32_to_bf16_bits(row)
        assert int(oracle.c_quantize(bits, oracle.MXFP4)[1][0, 0]) == code
        assert int(oracle.np_quantize(bits, oracle.MXFP4)[1][0, 0]) == code
    table = dict(zip(known["e8m0_block_amax"]["amax"], known["e8m0_block_amax"]["code"]))
    assert table[0.0] == 127 and table[1.0] == 125 and table[4.0] == 127 and table[6.0] == 127 and table[8.0] == 128


def test_small_cases_golden(oracle):
    z = np.load(os.path.join(GOLDEN, "small_cases.npz"))
    names = sorted({k.split("__")[0] for k in z.files})
    assert len(names) == 10
    for name in names:
        g = {k.split("__")[1]: z[k] for k in z.files if k.startswith(name + "__")}
        fmt = int(g["fmt"])
        for side in ("a", "b"):
            for q in (oracle.c_quantize(g[side], fmt), oracle.np_quantize(g[side], fmt)):
                assert np.array_equal(q[0], g[side + "_packed"]), name
                assert np.array_equal(q[1], g[side + "_scales"]), name
                assert np.float32(q[2]) == g[side + "_gs"], name
        a = (g["a_packed"], g["a_scales"], float(g["a_gs"]))
        b = (g["b_packed"], g["b_scales"], float(g["b_gs"]))
        _, dbf = oracle.c_gemm_fp4(a, b, fmt)
        assert np.array_equal(dbf, g["d_bf16"]), name
        # the reference's own expression on CPU tensors agrees up to bf16 rounding of near-ties
        t32, tbf = oracle.torch_gemm_oracle(oracle.np_dequantize(*a, fmt), oracle.np_dequantize(*b, fmt))
        exp = oracle.bf16_bits_to_f32(g["d_bf16"])
        got = oracle.bf16_bits_to_f32(tbf)
        den = np.linalg.norm(exp) or 1.0
        assert np.linalg.norm(got - exp) / den < 1e-3, name


def test_onehot_pins_nibble_order_and_scale_position(oracle):
    z = np.load(os.path.join(GOLDEN, "small_cases.npz"))
    packed, scales = z["onehot_nvfp4__a_packed"], z["onehot_nvfp4__a_scales"]
    for i in range(packed.shape[0]):
        col = (i * 5) % 128
        byte = packed[i, col // 2]
        nib = (byte >> 4) if (col & 1) else (byte & 0xF)
        assert nib == 7, (i, col, hex(byte))            # the block maximum always encodes as 6.0
        other = (byte & 0xF) if (col & 1) else (byte >> 4)
        assert other == 0
        assert np.count_nonzero(packed[i]) == 1
        assert np.count_nonzero(scales[i]) == 1 and scales[i, col // 16] != 0


def test_c0_golden(oracle):
    z = np.load(os.path.join(GOLDEN, "c0_nvfp4.npz"))
    A = inputs.normal_bf16(128, 512, seed=0)
    B = inputs.normal_bf16(256, 512, seed=1)
    a, b = _bits(A), _bits(B)
    if hashlib.sha256(a.tobytes()).hexdigest() != str(z["a_sha256"]):
        pytest.skip("torch's CPU generator produced different seed-0 inputs than when the fixture was made")
    qa, qb = oracle.c_quantize(a, oracle.NVFP4), oracle.c_quantize(b, oracle.NVFP4)
    assert np.array_equal(qa[0], z["a_packed"]) and np.array_equal(qa[1], z["a_scales"]) and np.float32(qa[2]) == z["a_gs"]
    assert np.array_equal(qb[0], z["b_packed"]) and np.array_equal(qb[1], z["b_scales"]) and np.float32(qb[2]) == z["b_gs"]
    # block holding the tensor maximum gets the largest scale code, 448
    assert qa[1].max() == 0x7E and qb[1].max() == 0x7E
    _, dbf = oracle.c_gemm_fp4(qa, qb, oracle.NVFP4)
    assert np.array_equal(dbf, z["d_bf16"])


def test_c_and_numpy_agree_on_random_inputs(oracle):
    rng = np.random.default_rng(5)
    for fmt in (oracle.NVFP4, oracle.MXFP4):
        for scale in (1.0, 0.02, 1e-30, 1e20):
            x = (rng.standard_normal((48, 256)) * scale).astype(np.float32)
            x[1] = 0
            x[2, 64:96] = 0
            bits = oracle.f32_to_bf16_bits(x)
            c, n = oracle.c_quantize(bits, fmt), oracle.np_quantize(bits, fmt)
            assert np.array_equal(c[0], n[0]) and np.array_equal(c[1], n[1]) and np.float32(c[2]) == np.float32(n[2])
            d1, d2 = oracle.c_dequantize(*c, fmt), oracle.np_dequantize(*c, fmt)
            assert np.array_equal(d1.view(np.uint32), d2.view(np.uint32))


def test_static_global_scale(oracle):
    rng = np.random.default_rng(6)
    bits = oracle.f32_to_bf16_bits(rng.standard_normal((8, 64)).astype(np.float32))
    c = oracle.c_quantize(bits, oracle.NVFP4, global_scale=0.0123)
    n = oracle.np_quantize(bits, oracle.NVFP4, global_scale=0.0123)
    assert np.array_equal(c[0], n[0]) and np.array_equal(c[1], n[1])


def test_quantisation_error_is_small(oracle):
    x = inputs.normal_bf16(64, 512, seed=2)
    xf = x.float().numpy()
    for fmt, bound in ((oracle.NVFP4, 0.11), (oracle.MXFP4, 0.14)):
        q = oracle.c_quantize(_bits(x), fmt)
        xh = oracle.c_dequantize(*q, fmt)
        assert np.linalg.norm(xh - xf) / np.linalg.norm(xf) < bound


def test_gemm_matches_reference_expression(oracle):
    # (A.float() @ B.float().T).to(bf16) on CPU tensors vs the C oracle (fp64 accumulate)
    rng = np.random.default_rng(8)
    a = rng.standard_normal((40, 192)).astype(np.float32)
    b = rng.standard_normal((24, 192)).astype(np.float32)
    d32 = np.empty((40, 24), dtype=np.float32)
    dbf = np.empty((40, 24), dtype=np.uint16)
    oracle.lib().ave_oracle_gemm_f32(a.ctypes.data, b.ctypes.data, 40, 24, 192, d32.ctypes.data, dbf.ctypes.data)
    t32, tbf = oracle.torch_gemm_oracle(a, b)
    assert np.allclose(d32, t32, rtol=1e-5, atol=1e-5)
    assert np.array_equal(dbf, oracle.f32_to_bf16_bits(d32))
    assert np.mean(dbf != tbf) < 0.01


def test_tiled_scale_layout(oracle):
    rng = np.random.default_rng(9)
    for rows, cols in ((1, 1), (16, 512), (128, 4), (130, 6), (300, 33)):
        sf = rng.integers(1, 255, (rows, cols), dtype=np.uint8)
        t1, t2 = oracle.c_sf_to_tiled(sf), oracle.np_sf_to_tiled(sf)
        assert np.array_equal(t1, t2)
        k_atoms = (cols + 3) // 4
        for r, c in ((0, 0), (rows - 1, cols - 1), (rows // 2, cols // 2)):
            off = ((r // 128) * k_atoms + c // 4) * 512 + ((r % 128) % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
            assert t1[off] == sf[r, c]
        assert np.count_nonzero(t1) == rows * cols  # padding is zero


def test_bf16_rounding_is_nearest_even(oracle):
    vals = np.array([1.0, 1.00390625, 1.005859375, 1.01171875, -2.5, 3.3895313e38, 1e-40], dtype=np.float32)
    want = torch.from_numpy(vals).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16_bits(vals), want)
    assert [oracle.lib().ave_oracle_f32_to_bf16(np.float32(v)) for v in vals] == want.tolist()


@pytest.mark.parametrize("act", [0, 1, 2, 3, 4])
def test_bias_act_c_matches_numpy(oracle, act):
    """The epilogue restatement: C (double libm) and numpy (math.erf / np.tanh / np.exp) agree to an fp32 ulp,
    and known values hold."""
    rng = np.random.default_rng(5)
    d = (rng.standard_normal((37, 72)) * 3).astype(np.float32)
    bias = oracle.f32_to_bf16_bits(rng.standard_normal(72).astype(np.float32))
    y_c, b_c = oracle.c_bias_act(d, bias, act)
    y_n, b_n = oracle.np_bias_act(d, bias, act)
    assert np.allclose(y_c, y_n, rtol=3e-7, atol=1e-9)
    # (1 + tanh(u)) cancels for very negative inputs, so results below 1e-6 may differ in their last digits
    assert ((b_c != b_n) & (np.abs(y_c) > 1e-6)).mean() < 1e-3
    one = np.array([[1.0, -1.0, 0.0]], dtype=np.float32)
    expected = {0: [1.0, -1.0, 0.0], 1: [1.0, 0.0, 0.0], 2: [0.8413447, -0.15865526, 0.0],
                3: [0.841192, -0.158808, 0.0], 4: [0.7310586, -0.26894143, 0.0]}[act]
    y, _ = oracle.c_bias_act(one, None, act)
    assert np.allclose(y[0], expected, rtol=1e-6, atol=1e-7)


def test_epilogue_golden_reproduced(oracle):
    """The committed fused-epilogue fixture (C0 operands): the oracle reproduces every expected array, and the
    numpy restatement of the quantise step agrees on the quantised result."""
    z = np.load(os.path.join(GOLDEN, "c0_nvfp4.npz"))
    e = np.load(os.path.join(GOLDEN, "c0_epilogue.npz"))
    qa = (z["a_packed"], z["a_scales"], float(z["a_gs"]))
    qb = (z["b_packed"], z["b_scales"], float(z["b_gs"]))
    d32, _ = oracle.c_gemm_fp4(qa, qb, oracle.NVFP4)
    for name, act, use_bias in (("bias_gelu", 2, True), ("bias_silu", 4, True), ("relu", 1, False), ("bias_gelu_tanh", 3, True)):
        _, ybf = oracle.c_bias_act(d32, e["bias"] if use_bias else None, act)
        assert np.array_equal(ybf, e["d_" + name]), name
    qp, qs, qg = oracle.c_quantize(e["d_bias_gelu"], oracle.NVFP4, float(e["q_gs"]))
    assert np.array_equal(qp, e["q_packed"]) and np.array_equal(qs, e["q_scales"]) and np.float32(qg) == e["q_gs"]
    n_p, n_s, _ = oracle.np_quantize(e["d_bias_gelu"], oracle.NVFP4, float(e["q_gs"]))
    assert np.array_equal(n_p, e["q_packed"]) and np.array_equal(n_s, e["q_scales"])
