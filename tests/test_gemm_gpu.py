"""GPU tier: the FP4 GEMM kernels (through the C ABI) against the CPU oracle.

Tolerance (stated by the task): relative Frobenius error <= 1e-3 against the oracle's
bf16-rounded fp32 result computed from the same quantised operands; max-abs error is
reported in the assertion message.  The comparison idiom follows the reference test
(test/examples/gemm/amdgpu/test_amdgpu_gemm.py:23-38), which compares against
``(A.float() @ B.float().T).to(bf16)``.
"""
import os

import numpy as np
import pytest
import torch

import avelang_b200 as ave
from avelang_b200 import inputs
from conftest import GOLDEN

pytestmark = pytest.mark.gpu

REL_FRO_TOL = 1e-3
TILED_VARIANTS = [ave.GEMM_1CTA_N128, ave.GEMM_1CTA_N256, ave.GEMM_2CTA_N256, ave.GEMM_2CTA_N128, ave.GEMM_2CTA_N192]


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _to_dev(q, fmt, dev):
    packed, scales, gs = q
    g = torch.tensor([gs], dtype=torch.float32, device=dev) if fmt == ave.NVFP4 else None
    return ave.make_operand(torch.from_numpy(packed).to(dev), torch.from_numpy(scales).to(dev), g, fmt)


def _gemm(A, B, fmt, **kw):
    fn = ave.gemm_nvfp4_transposed_b if fmt == ave.NVFP4 else ave.gemm_mxfp4_transposed_b
    return fn(A, B, **kw)


def _check(got_bf16, exp_bits, oracle, what):
    got = got_bf16.float().cpu().numpy()
    exp = oracle.bf16_bits_to_f32(exp_bits)
    assert np.isfinite(got).all(), what
    den = np.linalg.norm(exp) or 1.0
    rel = float(np.linalg.norm(got - exp) / den)
    max_abs = float(np.abs(got - exp).max())
    assert rel <= REL_FRO_TOL, f"{what}: rel_fro={rel:.3e} max_abs={max_abs:.4g}"
    return rel, max_abs


def _run_case(oracle, dev, fmt, m, n, k, variant, a_kind="normal", b_kind="weight", seed=0):
    a = inputs.make_operand_bf16(a_kind, m, k, seed)
    b = inputs.make_operand_bf16(b_kind, n, k, seed + 1)
    qa, qb = oracle.c_quantize(_bits(a), fmt), oracle.c_quantize(_bits(b), fmt)
    _, dbf = oracle.c_gemm_fp4(qa, qb, fmt, want_f32=False)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
    res = _gemm(_to_dev(qa, fmt, dev), _to_dev(qb, fmt, dev), fmt, out=out, variant=variant)
    ave.check_device_status(dev)
    assert res is out
    return _check(out, dbf, oracle, f"fmt={fmt} {m}x{n}x{k} variant={variant}")


@pytest.mark.parametrize("variant", TILED_VARIANTS)
@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (256, 512, 1024), (384, 640, 768)])
def test_tiled_variants_match_oracle(cuda_device, oracle, fmt, variant, m, n, k):
    _run_case(oracle, cuda_device, fmt, m, n, k, variant)


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
@pytest.mark.parametrize("m,n,k", [(100, 136, 96), (1, 8, 32), (130, 264, 2080), (257, 1000, 320), (65, 128, 4096)])
def test_ragged_shapes(cuda_device, oracle, fmt, m, n, k):
    """M, N not multiples of the tile and K not a multiple of the 256-element stage: edges are
    zero-filled on load and clipped on store."""
    for variant in (ave.GEMM_1CTA_N128, ave.GEMM_2CTA_N256, ave.GEMM_2CTA_N192):
        _run_case(oracle, cuda_device, fmt, m, n, k, variant)


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
@pytest.mark.parametrize("m,n,k", [(16, 256, 512), (16, 1024, 8192), (8, 384, 1024), (1, 128, 256), (32, 520, 2048),
                                   (64, 1160, 1056), (16, 28672, 1024)])
def test_skinny_matches_oracle(cuda_device, oracle, fmt, m, n, k):
    _run_case(oracle, cuda_device, fmt, m, n, k, ave.GEMM_SKINNY, a_kind="outlier")
    _run_case(oracle, cuda_device, fmt, m, n, k, ave.GEMM_AUTO, a_kind="outlier")


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
@pytest.mark.parametrize("m,n,k", [(16, 20480, 2048), (16, 19200, 1024), (8, 19072, 512), (32, 19072, 256)])
def test_skinny_many_tiles_short_k(cuda_device, oracle, fmt, m, n, k):
    """More weight tiles than SMs and a short K: the stream-K phase has fewer (tile, K block) units than there are
    CTAs, so only some CTAs take part in it.  Every column must be written, and a second call must find the arrival
    counters back at zero (same bits again)."""
    a = inputs.make_operand_bf16("outlier", m, k, 5)
    b = inputs.make_operand_bf16("weight", n, k, 6)
    qa, qb = oracle.c_quantize(_bits(a), fmt), oracle.c_quantize(_bits(b), fmt)
    _, dbf = oracle.c_gemm_fp4(qa, qb, fmt, want_f32=False)
    A, B = _to_dev(qa, fmt, cuda_device), _to_dev(qb, fmt, cuda_device)
    outs = []
    for _ in range(2):
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=cuda_device)
        _gemm(A, B, fmt, out=out, variant=ave.GEMM_SKINNY)
        ave.check_device_status(cuda_device)
        _check(out, dbf, oracle, f"fmt={fmt} {m}x{n}x{k} skinny, many tiles")
        outs.append(out)
    assert torch.equal(outs[0], outs[1])


def test_skinny_scratch_is_shared_across_shapes(cuda_device, oracle):
    """One scratch buffer serves calls of different shapes one after the other: a small-N call that leaves stream-K
    partials behind must not disturb the arrival counters of a following large-N call (everything that has to be zero
    between calls sits in a shape-independent prefix of the scratch)."""
    for m, n, k in ((9, 1160, 2080), (16, 28672, 1024), (32, 520, 2048), (16, 20480, 2048), (1, 128, 256), (16, 28672, 1024)):
        _run_case(oracle, cuda_device, ave.NVFP4, m, n, k, ave.GEMM_SKINNY, a_kind="outlier", seed=m + n)


def test_skinny_is_deterministic_and_reusable(cuda_device, oracle):
    """Stream-K partials are added in a fixed order, and the scratch counters return to zero,
    so back-to-back calls give identical bits."""
    m, n, k = 16, 4096, 8192
    a = inputs.outlier_activations_bf16(m, k, 0).to(cuda_device)
    b = inputs.normal_bf16(n, k, 1, std=0.02).to(cuda_device)
    A, B = ave.quantize_nvfp4(a), ave.quantize_nvfp4(b)
    outs = [ave.gemm_nvfp4_transposed_b(A, B).clone() for _ in range(4)]
    ave.check_device_status(cuda_device)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


def test_c0_golden_end_to_end(cuda_device, oracle):
    """Quantise on the GPU, multiply on the GPU, compare with the committed 128x256x512 fixture."""
    z = np.load(os.path.join(GOLDEN, "c0_nvfp4.npz"))
    A = ave.quantize_nvfp4(inputs.normal_bf16(128, 512, seed=0).to(cuda_device), sf_layout=ave.SF_ROW_MAJOR)
    B = ave.quantize_nvfp4(inputs.normal_bf16(256, 512, seed=1).to(cuda_device), sf_layout=ave.SF_ROW_MAJOR)
    if not np.array_equal(A.packed.cpu().numpy(), z["a_packed"]):
        import hashlib
        a_bits = _bits(inputs.normal_bf16(128, 512, seed=0))
        if hashlib.sha256(a_bits.tobytes()).hexdigest() != str(z["a_sha256"]):
            pytest.skip("torch's CPU generator produced different seed-0 inputs than when the fixture was made")
    assert np.array_equal(A.packed.cpu().numpy(), z["a_packed"]) and np.array_equal(A.scales.cpu().numpy(), z["a_scales"])
    assert np.array_equal(B.packed.cpu().numpy(), z["b_packed"]) and np.array_equal(B.scales.cpu().numpy(), z["b_scales"])
    for variant in TILED_VARIANTS + [ave.GEMM_AUTO]:
        out = ave.gemm_nvfp4_transposed_b(A, B, variant=variant)
        _check(out, z["d_bf16"], oracle, f"c0 variant {variant}")


def test_small_golden_cases(cuda_device, oracle):
    z = np.load(os.path.join(GOLDEN, "small_cases.npz"))
    for name in sorted({k.split("__")[0] for k in z.files}):
        g = {k.split("__")[1]: z[k] for k in z.files if k.startswith(name + "__")}
        fmt = int(g["fmt"])
        A = _to_dev((g["a_packed"], g["a_scales"], float(g["a_gs"])), fmt, cuda_device)
        B = _to_dev((g["b_packed"], g["b_scales"], float(g["b_gs"])), fmt, cuda_device)
        for variant in (ave.GEMM_1CTA_N128, ave.GEMM_2CTA_N256, ave.GEMM_2CTA_N192, ave.GEMM_SKINNY):
            out = _gemm(A, B, fmt, variant=variant)
            ave.check_device_status(cuda_device)
            _check(out, g["d_bf16"], oracle, f"{name} variant {variant}")


def test_out_argument_and_row_stride(cuda_device, oracle):
    """`out=` semantics of the reference operator (python/avelang_kernels/amdgpu_gemm.py:478-486)
    plus writing into a column block of a wider row-major matrix (how N-sharded results are laid out)."""
    m, n, k = 256, 256, 512
    a = inputs.normal_bf16(m, k, 0)
    b = inputs.normal_bf16(n, k, 1)
    qa, qb = oracle.c_quantize(_bits(a), oracle.NVFP4), oracle.c_quantize(_bits(b), oracle.NVFP4)
    _, dbf = oracle.c_gemm_fp4(qa, qb, oracle.NVFP4, want_f32=False)
    A, B = _to_dev(qa, ave.NVFP4, cuda_device), _to_dev(qb, ave.NVFP4, cuda_device)
    wide = torch.zeros((m, 3 * n), dtype=torch.bfloat16, device=cuda_device)
    ave.gemm_nvfp4_transposed_b(A, B, out=wide[:, n:2 * n])
    _check(wide[:, n:2 * n], dbf, oracle, "column block")
    assert torch.count_nonzero(wide[:, :n]) == 0 and torch.count_nonzero(wide[:, 2 * n:]) == 0
    with pytest.raises(ValueError, match="out must have shape"):
        ave.gemm_nvfp4_transposed_b(A, B, out=torch.empty((m, n + 8), dtype=torch.bfloat16, device=cuda_device))
    with pytest.raises(ValueError, match="out must have dtype"):
        ave.gemm_nvfp4_transposed_b(A, B, out=torch.empty((m, n), dtype=torch.float16, device=cuda_device))


@pytest.mark.parametrize("fmt", [ave.NVFP4, ave.MXFP4])
def test_empty_operands(cuda_device, fmt):
    """No activation rows or no weight rows: an empty result of the right shape, nothing launched, `out` returned."""
    q = ave.quantize_nvfp4 if fmt == ave.NVFP4 else ave.quantize_mxfp4
    g = ave.gemm_nvfp4_transposed_b if fmt == ave.NVFP4 else ave.gemm_mxfp4_transposed_b
    k = 256
    full = q(torch.randn((64, k), device=cuda_device).to(torch.bfloat16))
    none = q(torch.zeros((0, k), dtype=torch.bfloat16, device=cuda_device))
    assert tuple(g(none, full).shape) == (0, 64)
    assert tuple(g(full, none).shape) == (64, 0)
    out = torch.empty((0, 64), dtype=torch.bfloat16, device=cuda_device)
    assert g(none, full, out=out) is out
    ave.check_device_status(cuda_device)


def test_global_scale_is_linear(cuda_device):
    """Scaling a tensor scale by a power of two scales the output exactly (size-independent property)."""
    m = n = k = 1024
    A = ave.quantize_nvfp4(inputs.normal_bf16(m, k, 0).to(cuda_device))
    B = ave.quantize_nvfp4(inputs.normal_bf16(n, k, 1).to(cuda_device))
    d1 = ave.gemm_nvfp4_transposed_b(A, B)
    A4 = ave.Fp4Operand(A.packed, A.scales, A.global_scale * 4.0, A.fmt, A.rows, A.k, A.sf_layout)
    d4 = ave.gemm_nvfp4_transposed_b(A4, B)
    assert torch.equal(d4.float(), d1.float() * 4.0)


def test_square_8192_full_size(cuda_device, oracle):
    """The square benchmark config at full size.  The oracle cannot do 1.1 Tflop in seconds, so
    the checks are: (1) a sample of rows against the oracle, (2) the full result equals the
    result of multiplying a row slab on its own (tiles do not depend on their neighbours),
    (3) all tiled variants agree bit for bit (same accumulation order along K)."""
    m = n = k = 8192
    a = inputs.normal_bf16(m, k, 0).to(cuda_device)
    b = inputs.normal_bf16(n, k, 1).to(cuda_device)
    A = ave.quantize_nvfp4(a, sf_layout=ave.SF_ROW_MAJOR)
    B = ave.quantize_nvfp4(b, sf_layout=ave.SF_ROW_MAJOR)
    d = ave.gemm_nvfp4_transposed_b(A, B)
    ave.check_device_status(cuda_device)
    rows = [0, 1, 127, 128, 255, 256, 4097, 8191] + list(range(5000, 5024))
    ridx = torch.tensor(rows, device=cuda_device)
    qa = (A.packed[ridx].cpu().numpy(), A.scales[ridx].cpu().numpy(), float(A.global_scale.item()))
    qb = (B.packed.cpu().numpy(), B.scales.cpu().numpy(), float(B.global_scale.item()))
    _, dbf = oracle.c_gemm_fp4(qa, qb, oracle.NVFP4, want_f32=False)
    _check(d[ridx], dbf, oracle, "8192^3 row sample")
    slab = ave.Fp4Operand(A.packed[2048:2560], A.scales[2048:2560].contiguous(), A.global_scale, A.fmt, 512, k, ave.SF_ROW_MAJOR)
    d_slab = ave.gemm_nvfp4_transposed_b(slab, B)
    assert torch.equal(d_slab, d[2048:2560])
    for variant in (ave.GEMM_1CTA_N128, ave.GEMM_2CTA_N128, ave.GEMM_2CTA_N192, ave.GEMM_2CTA_N256):
        assert torch.equal(ave.gemm_nvfp4_transposed_b(A, B, variant=variant), d)


def test_decode_28672_full_size(cuda_device, oracle):
    """The decode config at full size (16 x 28672 x 8192, outlier activations quantised on the
    GPU, N(0, 0.02) weights): whole result against the oracle (7.5 Gflop on the CPU)."""
    m, n, k = 16, 28672, 8192
    x = inputs.outlier_activations_bf16(m, k, 0).to(cuda_device)
    w = inputs.normal_bf16(n, k, 1, std=0.02).to(cuda_device)
    X = ave.quantize_nvfp4(x, sf_layout=ave.SF_ROW_MAJOR)
    W = ave.quantize_nvfp4(w, sf_layout=ave.SF_ROW_MAJOR)
    d = ave.gemm_nvfp4_transposed_b(X, W)
    ave.check_device_status(cuda_device)
    qx = (X.packed.cpu().numpy(), X.scales.cpu().numpy(), float(X.global_scale.item()))
    qw = (W.packed.cpu().numpy(), W.scales.cpu().numpy(), float(W.global_scale.item()))
    ex, es, eg = oracle.c_quantize(_bits(x.cpu()), oracle.NVFP4)
    assert np.array_equal(qx[0], ex) and np.array_equal(qx[1], es)
    _, dbf = oracle.c_gemm_fp4(qx, qw, oracle.NVFP4, want_f32=False)
    _check(d, dbf, oracle, "decode full size")


def test_mxfp4_heavy_tail_2048(cuda_device, oracle):
    """The MXFP4 config's distributions (Student-t activations, N(0, 0.02) weights) on a 2048^3
    sub-problem the oracle finishes in seconds."""
    _run_case(oracle, cuda_device, ave.MXFP4, 2048, 2048, 2048, ave.GEMM_AUTO, a_kind="student_t3", b_kind="weight")


def test_tile_major_weights_match_row_major(cuda_device, oracle):
    """Weights re-packed into 16 KB tiles for the decode path give the same bits as row-major weights,
    including ragged N and a K that is not a multiple of the 256-element tile."""
    for fmt, m, n, k in ((ave.NVFP4, 16, 4096, 8192), (ave.MXFP4, 7, 1160, 2080), (ave.NVFP4, 64, 136, 96)):
        quant = ave.quantize_nvfp4 if fmt == ave.NVFP4 else ave.quantize_mxfp4
        X = quant(inputs.outlier_activations_bf16(m, k, 0).to(cuda_device))
        W = quant(inputs.normal_bf16(n, k, 1, std=0.02).to(cuda_device))
        Wt = ave.pack_weight_tiles(W)
        assert Wt.tile_major and Wt.packed.numel() == ((n + 127) // 128) * ((k + 255) // 256) * 16384
        d0 = _gemm(X, W, fmt)
        d1 = _gemm(X, Wt, fmt)
        ave.check_device_status(cuda_device)
        assert torch.equal(d0, d1)
    big = ave.quantize_nvfp4(inputs.normal_bf16(128, 256, 2).to(cuda_device))
    with pytest.raises(ValueError, match="M <= 64"):
        ave.gemm_nvfp4_transposed_b(big, ave.pack_weight_tiles(big))


def test_static_weights_overlap_keeps_results(cuda_device, oracle):
    """With static_weights=True the decode kernel starts before its predecessor in the stream has
    finished.  Activations quantised by that predecessor, the shared scratch and the output must
    still be handled in order: a chain of quantise -> GEMM steps with fresh activations every step
    gives exactly the results of the fully serialised form."""
    m, n, k = 16, 8192, 4096
    W = ave.quantize_nvfp4(inputs.normal_bf16(n, k, 1, std=0.02).to(cuda_device))
    xs = [inputs.outlier_activations_bf16(m, k, 10 + i).to(cuda_device) for i in range(8)]
    want = [ave.gemm_nvfp4_transposed_b(ave.quantize_nvfp4(x), W).clone() for x in xs]
    torch.cuda.synchronize()
    outs = [torch.empty((m, n), dtype=torch.bfloat16, device=cuda_device) for _ in xs]
    for _ in range(3):
        for x, o in zip(xs, outs):
            ave.gemm_nvfp4_transposed_b(ave.quantize_nvfp4(x), W, out=o, static_weights=True)
        ave.check_device_status(cuda_device)
        for o, w in zip(outs, want):
            assert torch.equal(o, w)
    # and inside a captured graph, the way the benchmark replays it
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.graph(g, stream=s):
        for x, o in zip(xs, outs):
            ave.gemm_nvfp4_transposed_b(ave.quantize_nvfp4(x), W, out=o, static_weights=True)
    for o in outs:
        o.zero_()
    for _ in range(3):
        g.replay()
    ave.check_device_status(cuda_device)
    for o, w in zip(outs, want):
        assert torch.equal(o, w)


def test_mxfp4_16384_full_size(cuda_device, oracle):
    """The MXFP4 config at full size (16384^3, Student-t activations, N(0, 0.02) weights): a row sample
    against the oracle, quantise bytes of the sample bit-exact, and slab independence."""
    m = n = k = 16384
    a = inputs.student_t3_bf16(m, k, 0).to(cuda_device)
    b = inputs.normal_bf16(n, k, 1, std=0.02).to(cuda_device)
    A = ave.quantize_mxfp4(a, sf_layout=ave.SF_ROW_MAJOR)
    B = ave.quantize_mxfp4(b, sf_layout=ave.SF_ROW_MAJOR)
    d = ave.gemm_mxfp4_transposed_b(A, B)
    ave.check_device_status(cuda_device)
    rows = [0, 255, 256, 8191, 16383] + list(range(12000, 12011))
    ridx = torch.tensor(rows, device=cuda_device)
    ep, es, _ = oracle.c_quantize(_bits(a[ridx].cpu()), oracle.MXFP4)
    assert np.array_equal(A.packed[ridx].cpu().numpy(), ep) and np.array_equal(A.scales[ridx].cpu().numpy(), es)
    qa = (ep, es, 1.0)
    qb = (B.packed.cpu().numpy(), B.scales.cpu().numpy(), 1.0)
    _, dbf = oracle.c_gemm_fp4(qa, qb, oracle.MXFP4, want_f32=False)
    _check(d[ridx], dbf, oracle, "16384^3 mxfp4 row sample")
    slab = ave.Fp4Operand(A.packed[4096:4352], A.scales[4096:4352].contiguous(), None, A.fmt, 256, k, ave.SF_ROW_MAJOR)
    assert torch.equal(ave.gemm_mxfp4_transposed_b(slab, B), d[4096:4352])


def test_prefill_57344_full_size(cuda_device, oracle):
    """The prefill config on one GPU (8192 x 57344 x 8192): a row sample against the oracle and the
    N-shard property the multi-GPU path relies on -- each of 8 column shards computed on its own
    (with the whole-tensor scale) equals the matching columns of the unsharded result."""
    m, n, k = 8192, 57344, 8192
    a = inputs.normal_bf16(m, k, 0).to(cuda_device)
    A = ave.quantize_nvfp4(a, sf_layout=ave.SF_ROW_MAJOR)
    del a
    b = inputs.normal_bf16(n, k, 1).to(cuda_device)
    B = ave.quantize_nvfp4(b, sf_layout=ave.SF_ROW_MAJOR)
    del b
    d = ave.gemm_nvfp4_transposed_b(A, B)
    ave.check_device_status(cuda_device)
    ridx = torch.tensor([0, 129, 4095, 8191], device=cuda_device)
    qa = (A.packed[ridx].cpu().numpy(), A.scales[ridx].cpu().numpy(), float(A.global_scale.item()))
    qb = (B.packed.cpu().numpy(), B.scales.cpu().numpy(), float(B.global_scale.item()))
    _, dbf = oracle.c_gemm_fp4(qa, qb, oracle.NVFP4, want_f32=False)
    _check(d[ridx], dbf, oracle, "prefill row sample")
    per = n // 8
    for r in (0, 3, 7):
        shard = ave.Fp4Operand(B.packed[r * per:(r + 1) * per], B.scales[r * per:(r + 1) * per].contiguous(), B.global_scale,
                               B.fmt, per, k, ave.SF_ROW_MAJOR)
        assert torch.equal(ave.gemm_nvfp4_transposed_b(A, shard), d[:, r * per:(r + 1) * per])


def test_agrees_with_library_nvfp4_gemm(cuda_device):
    """Independent cross-check of the storage conventions (nibble order, 128x4 scale tiles): torch's
    `_scaled_mm` (the vendor library's NVFP4 GEMM) consumes the very same bytes.  It rounds to bf16 before
    the tensor scales are applied, so the two results differ by one extra bf16 rounding (~2e-3)."""
    if not hasattr(torch, "float4_e2m1fn_x2") or not hasattr(torch, "_scaled_mm"):
        pytest.skip("this torch has no NVFP4 _scaled_mm")
    m, n, k = 512, 768, 1024
    A = ave.quantize_nvfp4(inputs.normal_bf16(m, k, 0).to(cuda_device))
    B = ave.quantize_nvfp4(inputs.normal_bf16(n, k, 1).to(cuda_device))
    ours = ave.gemm_nvfp4_transposed_b(A, B).float()
    try:
        lib = torch._scaled_mm(A.packed.view(torch.float4_e2m1fn_x2), B.packed.view(torch.float4_e2m1fn_x2).t(),
                               scale_a=A.scales.view(torch.float8_e4m3fn), scale_b=B.scales.view(torch.float8_e4m3fn),
                               out_dtype=torch.bfloat16)
    except Exception as exc:  # library path not available for this build / shape
        pytest.skip(f"library NVFP4 GEMM unavailable: {exc!r}"[:200])
    ref = lib.float() * (A.global_scale * B.global_scale)
    rel = (torch.linalg.norm(ours - ref) / torch.linalg.norm(ref)).item()
    assert rel < 5e-3, rel


def test_native_module_gives_the_same_bits_as_ctypes(cuda_device):
    """The pybind11 module in python/src forwards to the same C ABI: tiled GEMM, decode GEMM (shared scratch) and a fused
    epilogue through it equal the ctypes operators bit for bit."""
    import importlib
    import sys

    from avelang_b200 import build

    build.build_shim()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "python"))
    try:
        native = importlib.import_module("avelang_kernels.native")
    finally:
        sys.path.remove(os.path.join(root, "python"))
    dev = cuda_device
    for fmt, quant, gemm in ((ave.NVFP4, ave.quantize_nvfp4, ave.gemm_nvfp4_transposed_b), (ave.MXFP4, ave.quantize_mxfp4, ave.gemm_mxfp4_transposed_b)):
        for m, n, k in ((256, 512, 1024), (16, 1160, 2080)):
            A = quant(inputs.normal_bf16(m, k, 0).to(dev))
            B = quant(inputs.normal_bf16(n, k, 1, std=0.02).to(dev))
            bias = inputs.normal_bf16(1, n, 2).reshape(n).to(dev)
            assert torch.equal(native.gemm_fp4_transposed_b(A, B), gemm(A, B))
            assert torch.equal(native.gemm_fp4_transposed_b(A, B, bias=bias, activation="gelu_tanh"), gemm(A, B, bias=bias, activation="gelu_tanh"))
    ave.check_device_status(dev)
    with pytest.raises(ValueError, match="share K"):
        native.gemm_fp4_transposed_b(A, ave.quantize_mxfp4(inputs.normal_bf16(64, 512, 3).to(dev)))
