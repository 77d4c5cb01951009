"""The quantization-parameter and packing kernels on the GPU: zero point
(zeropoint-cuda) and MXFP4 quantize-dequantize (mxfp4-cuda) against the CPU
oracle, the golden vectors recorded from the reference's host code, and the
reference's own CUDA kernels run beside ours on the same buffers; the packed
MXFP4 form through its round trip."""
import ctypes as C

import numpy as np
import pytest

from conftest import to_dev
from test_oracle_cpu import (GOLDEN, MXFP4_KNOWN, ZP_CONFIGS, _bf16_bits, _bf16_vals,
                             mxfp4_driver_case, spaced_levels)
import refgpu

pytestmark = pytest.mark.gpu


# ---------------- zero point ----------------

@pytest.mark.parametrize("qmin,qmax", ZP_CONFIGS)
@pytest.mark.parametrize("preserve", [0, 1])
def test_zero_point_matches_reference_golden(hq, dev, qmin, qmax, preserve):
    import torch
    g = np.load(GOLDEN / "zeropoint_golden.npz")
    n = g["x_min"].size
    scale = torch.empty(n, dtype=torch.float32, device=dev)
    zp = torch.empty(n, dtype=torch.int32, device=dev)
    hq.zero_point(to_dev(g["x_min"], dev), to_dev(g["x_max"], dev), qmin, qmax, n, bool(preserve),
                  scale, zp)
    assert np.array_equal(scale.cpu().numpy().view(np.uint32),
                          g[f"scale_{qmin}_{qmax}_{preserve}"].view(np.uint32))
    assert np.array_equal(zp.cpu().numpy(), g[f"zp_{qmin}_{qmax}_{preserve}"])


def test_zero_point_reference_driver_run_beside_reference_kernel(hq, oracle, dev):
    """The reference driver's own configuration (zeropoint-cuda/main.cu:89-109:
    int8 symmetric, bounds uniform in (-1, 1)) at its run size of 10^7 channels:
    ours, the oracle and the reference kernel agree on every channel."""
    import torch
    n = 10_000_000
    rng = np.random.default_rng(123)
    lo = rng.uniform(-1, 1, n).astype(np.float32)
    hi = rng.uniform(-1, 1, n).astype(np.float32)
    dlo, dhi = to_dev(lo, dev), to_dev(hi, dev)
    scale = torch.empty(n, dtype=torch.float32, device=dev)
    zp = torch.empty(n, dtype=torch.int32, device=dev)
    hq.zero_point(dlo, dhi, -127, 127, n, True, scale, zp)
    so, zo = oracle.zero_point(lo, hi, -127, 127, True)
    assert np.array_equal(scale.cpu().numpy().view(np.uint32), so.view(np.uint32))
    assert np.array_equal(zp.cpu().numpy(), zo)
    ref = refgpu.load()
    if ref is None or not hasattr(ref, "ref_zero_point_gpu"):
        pytest.skip("reference kernels not built")
    rs = torch.empty_like(scale)
    rz = torch.empty_like(zp)
    torch.cuda.synchronize()
    assert ref.ref_zero_point_gpu(C.c_void_p(dlo.data_ptr()), C.c_void_p(dhi.data_ptr()), -127, 127,
                                  n, 1, C.c_void_p(rs.data_ptr()), C.c_void_p(rz.data_ptr())) == 0
    torch.cuda.synchronize()
    assert torch.equal(rs.view(torch.int32), scale.view(torch.int32))
    assert torch.equal(rz, zp)


@pytest.mark.parametrize("qmin,qmax", ZP_CONFIGS + [(-255, 0), (-300, -45), (3, 1000),
                                                    (-2**31 + 1, 2**31 - 2), (-2**25, 2**25),
                                                    (0, 1), (-70000, 70000)])
@pytest.mark.parametrize("preserve", [0, 1])
def test_zero_point_one_sided_ranges_and_ties(hq, oracle, dev, qmin, qmax, preserve):
    """Ranges with one end at zero - where the kernel settles the zero point from an
    fp32 estimate of the one non-zero quotient and divides in fp64 only near a
    point of decision: quotients that land exactly on .5, near-ties between the two
    ends (negative-only ranges of an unsigned type), bounds over sixty decades."""
    import torch
    rng = np.random.default_rng(qmax - qmin)
    n = 200_000
    k = rng.integers(0, 300, n)
    s = 2.0 ** rng.integers(-8, 4, n)
    tie = ((k + 0.5) * s).astype(np.float32)
    wide = np.abs(rng.standard_normal(n) * 10.0 ** rng.integers(-30, 30, n)).astype(np.float32)
    zero = np.zeros(n, np.float32)
    lo = np.concatenate([zero, -tie, zero, -wide, -wide])
    hi = np.concatenate([tie, zero, wide, zero, wide])
    scale = torch.empty(lo.size, dtype=torch.float32, device=dev)
    zp = torch.empty(lo.size, dtype=torch.int32, device=dev)
    hq.zero_point(to_dev(lo, dev), to_dev(hi, dev), qmin, qmax, lo.size, bool(preserve), scale, zp)
    so, zo = oracle.zero_point(lo, hi, qmin, qmax, bool(preserve))
    ok = np.isfinite(so)   # an adjusted range that overflows fp32 has no defined zero point
    assert np.array_equal(scale.cpu().numpy().view(np.uint32)[ok], so.view(np.uint32)[ok])
    assert np.array_equal(zp.cpu().numpy()[ok], zo[ok])


def test_zero_point_argument_errors(hq, dev):
    import torch
    lib = hq.load_library()
    f = torch.zeros(8, dtype=torch.float32, device=dev)
    z = torch.zeros(8, dtype=torch.int32, device=dev)
    p = lambda t: t.data_ptr()
    assert lib.hq_zero_point(p(f), p(f), 5, 5, 8, 1, p(f), p(z), None) == -1
    assert lib.hq_zero_point(None, p(f), -127, 127, 8, 1, p(f), p(z), None) == -2
    assert lib.hq_zero_point(None, None, -127, 127, 0, 1, None, None, None) == 0


# ---------------- 3-bit quantizer and packer ----------------

def _q3_weights(K, N, seed, dtype):
    rng = np.random.default_rng(seed)
    W = (rng.standard_normal((K, N)) * rng.uniform(0.01, 2.0, N)).astype(np.float32)
    W[:, 0] = 0.0                                  # a column of zeros
    W[:, 1] = np.abs(W[:, 1]) + 0.5                # positive only
    W[:, 2] = -np.abs(W[:, 2]) - 0.5               # negative only
    W[:, 3] = 0.25                                 # constant
    if dtype == "float16":
        return W.astype(np.float16).astype(np.float32)
    if dtype == "bfloat16":
        return _bf16_vals(_bf16_bits(W)).reshape(K, N)
    return W


@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32"])
@pytest.mark.parametrize("K,N", [(32, 8), (96, 264), (4096, 4096), (1024, 136), (64, 12288)])
def test_q3_quantize_against_oracle(hq, oracle, dev, dtype, K, N):
    """Packed matrix, scales and zeros bit for bit: shapes that leave column tiles and
    K slices ragged, columns of one sign, of zeros, of one value."""
    W = _q3_weights(K, N, K + N, dtype)
    mat, scales, zeros = hq.quantize_q3(_to_torch(W, dtype, dev))
    om, osc, oz = oracle.q3_quantize(W)
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), osc.view(np.uint32))
    assert np.array_equal(zeros.cpu().numpy().view(np.uint32), oz.view(np.uint32))
    assert np.array_equal(mat.cpu().numpy(), om)


def test_q3_quantize_ties_and_mat_vec(hq, oracle, dev):
    """Weights exactly half way between two codes (ties go to the even code), and
    the quantized layer through the 3-bit mat-vec against the mat-vec of its own
    dequantised weights."""
    import torch
    K, N = 2048, 512
    rng = np.random.default_rng(4)
    # scale 0.5 per column: lo = -1.5, hi = 2 -> codes at -1.5, -1, ..., 2; ties at +-.25 steps
    W = (rng.integers(-6, 9, (K, N)) * 0.25).astype(np.float32)
    W[0], W[1] = -1.5, 2.0
    mat, scales, zeros = hq.quantize_q3(to_dev(W, dev))
    om, osc, oz = oracle.q3_quantize(W)
    assert np.array_equal(mat.cpu().numpy(), om)
    assert np.array_equal(scales.cpu().numpy(), osc) and np.array_equal(zeros.cpu().numpy(), oz)
    Wq = oracle.q3_dequant_f32(om, osc, oz)
    assert np.abs(Wq - W).max() <= 0.25 + 1e-6
    x = rng.standard_normal(K).astype(np.float32)
    y = torch.zeros(N, dtype=torch.float32, device=dev)
    hq.vecquant3matmul(to_dev(x, dev), mat, y, scales, zeros, K * 3 // 32, N)
    ref = x.astype(np.float64) @ Wq.astype(np.float64)
    assert oracle.rel_err(y.cpu().numpy().astype(np.float64), ref) < 1e-3


def test_q3_quantize_layer_size_properties(hq, dev):
    """12288 x 12288 fp16 weights: every dequantised weight within half a step of
    the original, steps = (max - min) / 7 of the column range widened to hold 0."""
    import torch
    K = N = 12288
    g = torch.Generator(device=dev).manual_seed(11)
    W = torch.empty((K, N), dtype=torch.float16, device=dev).normal_(0, 0.02, generator=g)
    mat, scales, zeros = hq.quantize_q3(W)
    lo = W.float().amin(dim=0).clamp(max=0)
    hi = W.float().amax(dim=0).clamp(min=0)
    assert np.array_equal(scales.cpu().numpy(), (hi - lo).cpu().numpy() / np.float32(7))
    lib = hq.load_library()
    Wq = torch.empty((K, N), dtype=torch.float32, device=dev)
    assert lib.hq_q3_dequant_f32(mat.data_ptr(), scales.data_ptr(), zeros.data_ptr(), Wq.data_ptr(),
                                 K * 3 // 32, N, None) == 0
    err = (Wq - W.float()).abs() / scales
    assert float(err.max()) <= 0.5 + 1e-3
    del Wq, err


def test_q3_quantize_argument_errors(hq, dev):
    import torch
    lib = hq.load_library()
    w = torch.zeros(64 * 16, dtype=torch.float16, device=dev)
    m = torch.zeros(6 * 16, dtype=torch.int32, device=dev)
    f = torch.zeros(16, dtype=torch.float32, device=dev)
    ws = torch.zeros(128, dtype=torch.uint8, device=dev)
    p = lambda t: t.data_ptr()
    assert lib.hq_q3_quantize_workspace_bytes(16) == 128
    assert lib.hq_q3_quantize(p(w), 0, 48, 16, p(m), p(f), p(f), p(ws), 128, None) == -1
    assert lib.hq_q3_quantize(p(w), 0, 64, 12, p(m), p(f), p(f), p(ws), 128, None) == -1
    assert lib.hq_q3_quantize(None, 0, 64, 16, p(m), p(f), p(f), p(ws), 128, None) == -2
    assert lib.hq_q3_quantize(p(w), 0, 64, 16, p(m), p(f), p(f), p(ws), 64, None) == -5
    assert lib.hq_q3_quantize(p(w), 0, 64, 16, p(m), p(f), p(f), None, 0, None) == -5
    assert lib.hq_q3_quantize(p(w), 7, 64, 16, p(m), p(f), p(f), p(ws), 128, None) == -6
    assert lib.hq_q3_quantize(p(w) + 2, 0, 32, 16, p(m), p(f), p(f), p(ws), 128, None) == -3
    torch.cuda.synchronize()


# ---------------- greedy binary-coding quantizer ----------------

@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32"])
@pytest.mark.parametrize("K,M,nb,gs,bias", [(128, 128, 3, 128, True), (256, 136, 4, 64, True),
                                            (512, 1024, 1, 32, False), (1024, 264, 3, 256, False),
                                            (384, 8, 8, 128, True), (1024, 72, 2, 512, True)])
def test_bcq_quantize_against_oracle(hq, oracle, dev, dtype, K, M, nb, gs, bias):
    """Sign planes, scales and offsets bit for bit; columns of zeros and of one value
    (zero residuals: the bit of a zero is 1)."""
    rng = np.random.default_rng(K + M + nb)
    W = (rng.standard_normal((K, M)) * 0.05).astype(np.float32)
    W[:, 0] = 0.0
    W[:, 1] = 0.125
    if dtype == "float16":
        W = W.astype(np.float16).astype(np.float32)
    elif dtype == "bfloat16":
        W = _bf16_vals(_bf16_bits(W)).reshape(K, M)
    bW, alpha, qb = hq.quantize_bcq(_to_torch(W, dtype, dev), nb, gs, bias)
    obW, oal, oqb = oracle.lutgemm_quantize(W, nb, gs, bias)
    assert np.array_equal(bW.cpu().numpy().view(np.uint32), obW)
    assert np.array_equal(alpha.cpu().numpy().view(np.uint16), oal.view(np.uint16))
    if bias:
        assert np.array_equal(qb.cpu().numpy().view(np.uint16), oqb.view(np.uint16))


def test_bcq_quantize_error_shrinks_and_feeds_the_mat_vec(hq, oracle, dev):
    """More planes, smaller error; and the quantized layer through the LUT-GEMM
    mat-vec equals the mat-vec of its own dequantised weights."""
    import torch
    K = M = 1024
    rng = np.random.default_rng(6)
    W = (rng.standard_normal((K, M)) * 0.03).astype(np.float16)
    x = rng.standard_normal(K).astype(np.float16)
    dW = to_dev(W.view(np.uint16).view(np.int16), dev).view(torch.float16)
    errs = []
    for nb in (1, 2, 3, 4):
        bW, alpha, qb = hq.quantize_bcq(dW, nb, 128, True)
        Wq = oracle.lutgemm_dequant_f32(bW.cpu().numpy().view(np.uint32),
                                        alpha.cpu().numpy(), qb.cpu().numpy(), M, K, nb, 128)
        errs.append(float(np.sqrt(np.mean((Wq - W.astype(np.float32)) ** 2))))
        if nb == 3:
            w = hq.nQWeight_fp16(bW.cpu().numpy().view(np.uint32), alpha.cpu().numpy().astype(np.float32),
                                 K, M, nb, False, K // 128, qb.cpu().numpy().astype(np.float32),
                                 device=dev)
            y = torch.empty(M, dtype=torch.float16, device=dev)
            hq.matmul(y, to_dev(x.view(np.uint16).view(np.int16), dev).view(torch.float16), w)
            ref = x.astype(np.float64) @ Wq.astype(np.float64)
            assert oracle.rel_err(y.cpu().numpy().astype(np.float64), ref) < 1e-2
    assert errs[0] > errs[1] > errs[2] > errs[3]
    assert errs[2] < 0.25 * 0.03      # three planes leave under a quarter of the spread


def test_bcq_quantize_argument_errors(hq, dev):
    import torch
    lib = hq.load_library()
    w = torch.zeros(128 * 16, dtype=torch.float16, device=dev)
    b = torch.zeros(4 * 3 * 16, dtype=torch.int32, device=dev)
    a = torch.zeros(3 * 16, dtype=torch.float16, device=dev)
    p = lambda t: t.data_ptr()
    assert lib.hq_lutgemm_quantize(p(w), 0, 128, 16, 3, 48, p(b), p(a), None, None) == -1
    assert lib.hq_lutgemm_quantize(p(w), 0, 128, 12, 3, 128, p(b), p(a), None, None) == -1
    assert lib.hq_lutgemm_quantize(p(w), 0, 128, 16, 9, 128, p(b), p(a), None, None) == -1
    assert lib.hq_lutgemm_quantize(p(w), 0, 128, 16, 3, 128, None, p(a), None, None) == -2
    assert lib.hq_lutgemm_quantize(p(w), 5, 128, 16, 3, 128, p(b), p(a), None, None) == -6
    assert lib.hq_lutgemm_quantize(p(w), 0, 1024, 16, 3, 1024, p(b), p(a), None, None) == -6
    torch.cuda.synchronize()


# ---------------- blockwise 4-bit quantizer ----------------

def _weights(n_blocks, bs, seed, dtype):
    rng = np.random.default_rng(seed)
    w = rng.standard_normal(n_blocks * bs) * np.repeat(10.0 ** rng.integers(-3, 3, n_blocks), bs)
    w = w.astype(np.float32)
    w[bs:2 * bs] = 0.0                                           # a block of zeros
    w[2 * bs:3 * bs] *= np.float32(1e-42) / np.abs(w[2 * bs:3 * bs]).max()   # a denormal absmax (fp32)
    if dtype == "float16":
        return w.astype(np.float16).astype(np.float32)
    if dtype == "bfloat16":
        return _bf16_vals(_bf16_bits(w))
    return w


def _to_torch(w32, dtype, dev):
    import torch
    t = to_dev(w32, dev)
    return t.to({"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}[dtype])


@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32"])
@pytest.mark.parametrize("bs", [32, 64, 128, 256, 512, 4096])
def test_nf4_quantize_against_oracle(hq, oracle, dev, dtype, bs):
    """Codes and absmax bit for bit, both nibble orders, every block size class
    (blocks inside a warp's lanes; blocks a warp walks twice), a ragged count."""
    w = _weights(1237 if bs <= 256 else 67, bs, bs, dtype)
    lut = spaced_levels(bs)
    for order in (0, 1):
        B, absmax = hq.quantize_nf4(_to_torch(w, dtype, dev), to_dev(lut, dev), bs, order)
        oB, oa = oracle.nf4_quantize(w, bs, lut, order)
        assert np.array_equal(absmax.cpu().numpy().view(np.uint32), oa.view(np.uint32))
        assert np.array_equal(B.cpu().numpy(), oB)


def test_nf4_quantize_ties_ends_and_close_levels(hq, oracle, dev):
    """Weights that sit exactly on a midpoint (the lower level wins), on the levels,
    at +-absmax; and a level table with neighbours closer than a table cell, which
    makes the kernel count midpoints instead of looking them up."""
    for lut in (spaced_levels(3),
                np.sort(np.concatenate([np.linspace(-1, 1, 12), [0.001, 0.002, 0.0035, 0.3001]])
                        ).astype(np.float32)):
        mids = (0.5 * (lut[:-1] + lut[1:])).astype(np.float32)
        blocks = []
        for scale in (1.0, 0.37, 512.0):
            v = np.concatenate([mids, lut, np.nextafter(mids, np.float32(2)),
                                np.nextafter(mids, np.float32(-2)), [1.0, -1.0]]).astype(np.float32)
            v = np.concatenate([v, np.zeros(64 - v.size % 64, np.float32)])
            v[-1] = 1.0                                          # absmax of every block is `scale`
            blk = v.reshape(-1, 64).copy()
            blk[:, -1] = 1.0
            blocks.append((blk * np.float32(scale)).astype(np.float32))
        w = np.concatenate(blocks).reshape(-1)
        B, absmax = hq.quantize_nf4(to_dev(w, dev), to_dev(lut, dev), 64, 0)
        oB, oa = oracle.nf4_quantize(w, 64, lut, 0)
        assert np.array_equal(B.cpu().numpy(), oB)
        assert np.array_equal(absmax.cpu().numpy(), oa)


def test_nf4_quantize_round_trip_at_layer_size(hq, dev):
    """An 11008 x 4096 fp16 layer: quantize -> dequantize -> quantize returns the same
    codes, the dequantised weights stay within half a level gap of the originals,
    and the mat-vec on the quantized layer is the mat-vec on the dequantised one."""
    import torch
    N, K, bs = 11008, 4096, 64
    lut = spaced_levels(9)
    g = torch.Generator(device=dev).manual_seed(3)
    W = torch.empty(N * K, dtype=torch.float16, device=dev).normal_(0, 0.02, generator=g)
    dl = to_dev(lut, dev)
    B, absmax = hq.quantize_nf4(W, dl, bs)
    Wq = hq.dequantize_nf4(B, absmax, dl, N * K, bs, 0)
    B2, absmax2 = hq.quantize_nf4(Wq, dl, bs)
    assert torch.equal(B2, B)
    gap = float(np.max(np.diff(lut)))
    err = (Wq.float() - W.float()).abs().view(-1, bs) / absmax.view(-1, 1)
    assert float(err.max()) <= gap / 2 + 1e-3
    x = torch.empty(K, dtype=torch.float16, device=dev).normal_(0, 1, generator=g)
    y = hq.gemv_nf4(x, B, absmax, dl, N, K, bs, 0)
    ref = Wq.view(N, K).float() @ x.float()
    assert float((y.float() - ref).abs().max() / ref.abs().max()) < 1e-2


def test_nf4_quantize_argument_errors(hq, dev):
    import torch
    lib = hq.load_library()
    w = torch.zeros(128, dtype=torch.float16, device=dev)
    b = torch.zeros(64, dtype=torch.uint8, device=dev)
    f = torch.zeros(16, dtype=torch.float32, device=dev)
    p = lambda t: t.data_ptr()
    assert lib.hq_nf4_quantize(p(w), 0, 128, 48, p(f), 0, p(b), p(f), None) == -1
    assert lib.hq_nf4_quantize(p(w), 0, 100, 64, p(f), 0, p(b), p(f), None) == -1
    assert lib.hq_nf4_quantize(p(w), 0, 128, 8192, p(f), 0, p(b), p(f), None) == -1
    assert lib.hq_nf4_quantize(p(w), 3, 128, 64, p(f), 0, p(b), p(f), None) == -6
    assert lib.hq_nf4_quantize(p(w), 0, 128, 64, None, 0, p(b), p(f), None) == -2
    assert lib.hq_nf4_quantize(p(w) + 2, 0, 64, 64, p(f), 0, p(b), p(f), None) == -3
    assert lib.hq_nf4_quantize(None, 0, 0, 64, p(f), 0, None, None, None) == 0
    torch.cuda.synchronize()


# ---------------- MXFP4 ----------------

def _bits(x32, bf16):
    return _bf16_bits(x32) if bf16 else x32.astype(np.float16).view(np.uint16)


def _t(bits, bf16, dev):
    import torch
    t = to_dev(bits.view(np.int16), dev)
    return t.view(torch.bfloat16 if bf16 else torch.float16)


def _run_qdq(hq, bits, bf16, dev):
    import torch
    a = _t(bits, bf16, dev)
    y = torch.empty_like(a)
    hq.mxfp4(y, a, a.numel())
    return y.view(torch.int16).cpu().numpy().view(np.uint16)


def _ref_qdq(bits, bf16, dev):
    import torch
    ref = refgpu.load()
    if ref is None or not hasattr(ref, "ref_mxfp4_qdq"):
        return None
    a = _t(bits, bf16, dev)
    y = torch.empty_like(a)
    torch.cuda.synchronize()
    assert ref.ref_mxfp4_qdq(C.c_void_p(a.data_ptr()), C.c_void_p(y.data_ptr()), a.numel(),
                             int(bf16)) == 0
    torch.cuda.synchronize()
    return y.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("bf16", [False, True])
def test_mxfp4_reference_driver_inputs(hq, oracle, dev, bf16):
    """The reference driver's inputs and its own expectations (verify.h), on ours,
    the oracle and the reference kernel: all three bit-equal."""
    x = mxfp4_driver_case(32 * 8192, 7, np.float32)
    bits = _bits(x, bf16)
    y = _run_qdq(hq, bits, bf16, dev)
    assert np.array_equal(y, oracle.mxfp4_qdq(bits, bf16))
    vals = _bf16_vals(y) if bf16 else y.view(np.float16).astype(np.float32)
    xin = _bf16_vals(bits) if bf16 else bits.view(np.float16).astype(np.float32)
    conv = (lambda v: float(_bf16_vals(_bf16_bits(np.array([v], np.float32)))[0])) if bf16 else \
        (lambda v: float(np.float16(v)))
    want = {conv(k): v for k, v in MXFP4_KNOWN.items()}
    want[6.0] = 6.0
    assert np.array_equal(vals, np.array([np.copysign(want[abs(float(v))], v) for v in xin],
                                         dtype=np.float32))
    r = _ref_qdq(bits, bf16, dev)
    if r is not None:
        assert np.array_equal(r, y)


@pytest.mark.parametrize("bf16", [False, True])
def test_mxfp4_every_bit_pattern_beside_reference_kernel(hq, oracle, dev, bf16):
    """Every finite 16-bit pattern as an element, in groups whose maximum is pinned
    at several binades (so each pattern meets several scales): ours == oracle ==
    reference kernel, bit for bit, wherever the pinned maximum really is the
    group's maximum (the reference's defined domain)."""
    exp_mask = 0x7f80 if bf16 else 0x7c00
    pats = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    pats = pats[(pats & exp_mask) != exp_mask]                  # no inf / nan
    one = 0x3f80 if bf16 else 0x3c00
    step = 0x80 if bf16 else 0x400
    checked = 0
    for de, mant in ((-6, 0), (-1, 0.3), (0, 0.7), (0, 0.76), (3, 0.5), (9, 0.99), (-12, 0.1)):
        mx = np.uint16(one + de * step + int(mant * step))      # (1 + mant) * 2^de
        el = pats[(pats & 0x7fff) <= mx]                         # the pinned value is the maximum
        el = el[:(el.size // 31) * 31].reshape(-1, 31)
        grp = np.concatenate([el, np.full((el.shape[0], 1), mx, np.uint16)], axis=1)
        grp = grp[:(grp.shape[0] // 4) * 4].reshape(-1)          # the reference wants multiples of 64
        y = _run_qdq(hq, grp, bf16, dev)
        assert np.array_equal(y, oracle.mxfp4_qdq(grp, bf16)), (de, mant)
        r = _ref_qdq(grp, bf16, dev)
        if r is not None:
            assert np.array_equal(r, y), (de, mant)
        checked += grp.size
    assert checked > 200_000


@pytest.mark.parametrize("bf16", [False, True])
def test_mxfp4_random_tensor_and_packed_round_trip(hq, oracle, dev, bf16):
    """N(0, 1) values times a per-group magnitude 2^-10 .. 2^10, a ragged number of
    groups: quantize-dequantize equals the oracle; the packed form equals the
    oracle's and decodes to the same values; a second pass changes nothing."""
    import torch
    rng = np.random.default_rng(17)
    groups = 40_013
    x = rng.standard_normal(groups * 32) * np.repeat(2.0 ** rng.integers(-10, 11, groups), 32)
    x[64:96] = 0.0                                               # a group of zeros
    bits = _bits(x.astype(np.float32), bf16)
    y = _run_qdq(hq, bits, bf16, dev)
    assert np.array_equal(y, oracle.mxfp4_qdq(bits, bf16))
    codes, scales = hq.mxfp4_quantize(_t(bits, bf16, dev))
    oc, osc = oracle.mxfp4_quantize(bits, bf16)
    assert np.array_equal(codes.cpu().numpy(), oc)
    assert np.array_equal(scales.cpu().numpy(), osc)
    back = hq.mxfp4_dequantize(codes, scales, torch.bfloat16 if bf16 else torch.float16)
    assert np.array_equal(back.view(torch.int16).cpu().numpy().view(np.uint16), y)
    assert np.array_equal(_run_qdq(hq, y, bf16, dev), y)         # idempotent
    r = _ref_qdq(bits[:groups // 4 * 128], bf16, dev)
    if r is not None:
        keep = np.ones(r.size, bool)
        keep[64:96] = False                                      # the zero group: undefined there
        assert np.array_equal(r[keep], y[:r.size][keep])


def test_mxfp4_full_size_properties(hq, dev):
    """2^28 fp16 values (512 MB in, 512 MB out): idempotence, and the packed round
    trip equal to the direct result, checked on the device."""
    import torch
    n = 1 << 28
    g = torch.Generator(device=dev).manual_seed(5)
    a = torch.empty(n, dtype=torch.float16, device=dev)
    a.normal_(0, 3, generator=g)
    y = torch.empty_like(a)
    hq.mxfp4(y, a, n)
    y2 = torch.empty_like(a)
    hq.mxfp4(y2, y, n)
    assert torch.equal(y2.view(torch.int16), y.view(torch.int16))
    del y2
    codes, scales = hq.mxfp4_quantize(a)
    back = hq.mxfp4_dequantize(codes, scales, torch.float16)
    assert torch.equal(back.view(torch.int16), y.view(torch.int16))
    # every value is one of the 15 grid values times its group's scale
    sc = torch.pow(2.0, scales.to(torch.float32) - 127).repeat_interleave(32)
    q = (y.float().abs() / sc)
    assert bool(torch.isin(q, torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6], device=dev)).all())


def test_mxfp4_argument_errors(hq, dev):
    import torch
    lib = hq.load_library()
    a = torch.zeros(64, dtype=torch.float16, device=dev)
    c = torch.zeros(32, dtype=torch.uint8, device=dev)
    p = lambda t: t.data_ptr()
    assert lib.hq_mxfp4_qdq(p(a), p(a), 48, 0, None) == -1       # whole groups of 32 only
    assert lib.hq_mxfp4_qdq(p(a), p(a), 64, 2, None) == -6       # fp16 or bf16
    assert lib.hq_mxfp4_qdq(None, p(a), 64, 0, None) == -2
    assert lib.hq_mxfp4_qdq(p(a) + 2, p(a), 32, 0, None) == -3
    assert lib.hq_mxfp4_quantize(p(a), p(c), None, 64, 0, None) == -2
    assert lib.hq_mxfp4_dequantize(p(c), None, p(a), 64, 0, None) == -2
    assert lib.hq_mxfp4_qdq(None, None, 0, 0, None) == 0
    torch.cuda.synchronize()
