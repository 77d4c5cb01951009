"""GPU parity tests: every kernel is called through the C ABI (ctypes) and
compared with the CPU oracle on the same seeded inputs; where the reference's
own CUDA kernel could be built (oracle/_ref/libref_gpu.so) it is run beside
ours on the same device buffers.

Tolerances: unpack / dequantised weights / integer outputs are bit exact; GEMV
outputs are within 1e-3 (fp32 accumulation, fp32 output) or 1e-2 (fp16
arithmetic or fp16 output) of the fp64 oracle, measured as
|y - ref| / max(|ref|, rms(ref)).
"""
import ctypes as C

import numpy as np
import pytest

from hecbench_b200 import synth
from conftest import GOLDEN, to_dev
import refgpu

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3
TOL_F16 = 1e-2


def _np(t):
    return t.detach().cpu().numpy()


# ------------------------------------------------------------------ q3

def _q3_setup(oracle, dev, K, width, seed, kat=False):
    if kat:
        codes = np.ones((K, width), dtype=np.uint8)
        vec = np.ones(K, dtype=np.float32)
        sc = -np.ones(width, dtype=np.float32)
        z = np.zeros(width, dtype=np.float32)
    else:
        vec, codes, sc, z = synth.q3_case(K, width, seed)
    mat = oracle.q3_pack(codes)
    return vec, codes, sc, z, mat


@pytest.mark.parametrize("K,width", [(256, 256), (1024, 384), (4096, 4096), (2048, 132), (32, 4)])
def test_q3_gemv_f32(hq, oracle, dev, K, width):
    import torch
    vec, codes, sc, z, mat = _q3_setup(oracle, dev, K, width, seed=K + width)
    d = [to_dev(a, dev) for a in (vec, mat, sc, z)]
    mul = torch.full((width,), 0.5, dtype=torch.float32, device=dev)  # accumulate semantics
    hq.vecquant3matmul(d[0], d[1], mul, d[2], d[3], mat.shape[0], width)
    ref = oracle.q3_gemv_f64(vec, mat, sc, z) + 0.5
    assert oracle.rel_err(_np(mul), ref) < TOL_F32


@pytest.mark.parametrize("K,width", [(256, 256), (1024, 384), (4096, 4096), (2048, 132), (32, 4)])
def test_q3_gemv_f16in(hq, oracle, dev, K, width):
    import torch
    vec, codes, sc, z, mat = _q3_setup(oracle, dev, K, width, seed=K + width + 1)
    vh = vec.astype(np.float16)
    mul = torch.zeros(width, dtype=torch.float32, device=dev)
    hq.vecquant3matmul_faster(to_dev(vh, dev).view(torch.float16), to_dev(mat, dev), mul,
                              to_dev(sc, dev), to_dev(z, dev), mat.shape[0], width)
    ref = oracle.q3_gemv_f64(vh.astype(np.float32), mat, sc, z, f16rule=True)
    assert oracle.rel_err(_np(mul), ref) < TOL_F16


def test_q3_reference_known_answer(hq, oracle, dev):
    """The check of quant3MatMul-cuda/main.cu:84-105 at a reduced width."""
    import torch
    K, width = 49152, 512
    vec, codes, sc, z, mat = _q3_setup(oracle, dev, K, width, 0, kat=True)
    dm, dsc, dz = to_dev(mat, dev), to_dev(sc, dev), to_dev(z, dev)
    mul = torch.zeros(width, dtype=torch.float32, device=dev)
    hq.vecquant3matmul(to_dev(vec, dev), dm, mul, dsc, dz, mat.shape[0], width)
    assert torch.all(mul == -49152.0)
    mul.zero_()
    hq.vecquant3matmul_faster(to_dev(vec.astype(np.float16), dev).view(torch.float16), dm, mul,
                              dsc, dz, mat.shape[0], width)
    assert torch.all(mul == -49152.0)


def test_q3_dequant_bit_exact(hq, oracle, dev):
    import torch
    K, width = 512, 260
    vec, codes, sc, z, mat = _q3_setup(oracle, dev, K, width, seed=77)
    dm, dsc, dz = to_dev(mat, dev), to_dev(sc, dev), to_dev(z, dev)
    W32 = hq.vecquant3_dequant(dm, dsc, dz, mat.shape[0], width, torch.float32)
    assert np.array_equal(_np(W32).view(np.uint32), oracle.q3_dequant_f32(mat, sc, z).view(np.uint32))
    W16 = hq.vecquant3_dequant(dm, dsc, dz, mat.shape[0], width, torch.float16)
    assert np.array_equal(_np(W16).view(np.uint16), oracle.q3_dequant_f16(mat, sc, z).view(np.uint16))


def test_q3_against_reference_kernels(hq, oracle, dev):
    """Our kernels beside the reference CUDA kernels on the same buffers; a
    one-hot input makes the reference kernel emit single dequantised weights,
    which pins the fp32 dequant rule (fma) bit for bit."""
    import torch
    ref = refgpu.load()
    if ref is None:
        pytest.skip("reference CUDA build not present")
    K, width = 1024, 512  # reference needs height % 24 == 0, width % 256 == 0
    vec, codes, sc, z, mat = _q3_setup(oracle, dev, K, width, seed=5)
    dm, dsc, dz = to_dev(mat, dev), to_dev(sc, dev), to_dev(z, dev)
    dv = to_dev(vec, dev)
    a = torch.zeros(width, dtype=torch.float32, device=dev)
    b = torch.zeros(width, dtype=torch.float32, device=dev)
    ref.ref_q3_gemv_f32(C.c_void_p(dv.data_ptr()), C.c_void_p(dm.data_ptr()), C.c_void_p(a.data_ptr()),
                        C.c_void_p(dsc.data_ptr()), C.c_void_p(dz.data_ptr()), mat.shape[0], width)
    hq.vecquant3matmul(dv, dm, b, dsc, dz, mat.shape[0], width)
    torch.cuda.synchronize()
    y64 = oracle.q3_gemv_f64(vec, mat, sc, z)
    assert oracle.rel_err(_np(a), y64) < TOL_F32
    assert oracle.rel_err(_np(b), y64) < TOL_F32
    assert oracle.rel_err(_np(b), _np(a).astype(np.float64)) < TOL_F32
    # fp32 oracle in the reference's own summation order
    assert oracle.rel_err(_np(a), oracle.q3_gemv_f32(vec, mat, np.zeros(width, np.float32), sc, z)) < 1e-5
    # one-hot rows: exact dequantised weights out of the reference kernel
    W = oracle.q3_dequant_f32(mat, sc, z)
    for k in (0, 10, 21, 31, 500, 1023):
        onehot = np.zeros(K, dtype=np.float32)
        onehot[k] = 1.0
        a.zero_()
        ref.ref_q3_gemv_f32(C.c_void_p(to_dev(onehot, dev).data_ptr()), C.c_void_p(dm.data_ptr()),
                            C.c_void_p(a.data_ptr()), C.c_void_p(dsc.data_ptr()),
                            C.c_void_p(dz.data_ptr()), mat.shape[0], width)
        torch.cuda.synchronize()
        assert np.array_equal(_np(a).view(np.uint32), W[k].view(np.uint32))
    # faster kernel
    vh = vec.astype(np.float16)
    dvh = to_dev(vh, dev)
    a.zero_(); b.zero_()
    ref.ref_q3_gemv_faster(C.c_void_p(dvh.data_ptr()), C.c_void_p(dm.data_ptr()), C.c_void_p(a.data_ptr()),
                           C.c_void_p(dsc.data_ptr()), C.c_void_p(dz.data_ptr()), mat.shape[0], width)
    hq.vecquant3matmul_faster(dvh.view(torch.float16), dm, b, dsc, dz, mat.shape[0], width)
    torch.cuda.synchronize()
    y64h = oracle.q3_gemv_f64(vh.astype(np.float32), mat, sc, z, f16rule=True)
    assert oracle.rel_err(_np(a), y64h) < TOL_F16
    assert oracle.rel_err(_np(b), y64h) < TOL_F16
    # the fp16 restatement follows the reference's order exactly (slab sums aside)
    assert oracle.rel_err(_np(a), oracle.q3_gemv_f16in(vh, mat, np.zeros(width, np.float32), sc, z)) < 1e-5


def test_q3_bad_arguments(hq, dev):
    import torch
    lib = hq.load_library()
    t = torch.zeros(1024, dtype=torch.float32, device=dev)
    p = C.c_void_p(t.data_ptr())
    assert lib.hq_q3_gemv_f32(p, p, p, p, p, 25, 256, None) == -1
    assert lib.hq_q3_gemv_f32(p, C.c_void_p(t.data_ptr() + 4), p, p, p, 24, 256, None) == -3
    assert lib.hq_q3_gemv_f32(None, p, p, p, p, 24, 256, None) == -2


# ------------------------------------------------------------------ bnb

def test_bnb_quantize_golden_and_random(hq, oracle, dev):
    import torch
    g = np.load(GOLDEN / "bnb_golden.npz")
    code, A, want = g["code"], g["A"], g["out"]
    dcode = to_dev(code, dev)
    out = torch.empty(A.size, dtype=torch.uint8, device=dev)
    hq.kQuantize(dcode, to_dev(A, dev), out, A.size)
    assert np.array_equal(_np(out), want)
    # ragged sizes and an unaligned start
    for n in (1, 3, 255, 1000003):
        x = np.random.default_rng(n).standard_normal(n + 1).astype(np.float32)
        dx = to_dev(x, dev)
        out = torch.empty(n + 1, dtype=torch.uint8, device=dev)
        hq.kQuantize(dcode, dx, out, n)
        assert np.array_equal(_np(out)[:n], oracle.bnb_quantize(code, x[:n]))
        out2 = torch.zeros(n + 1, dtype=torch.uint8, device=dev)
        hq.kQuantize(dcode, dx[1:], out2[1:], n)
        assert np.array_equal(_np(out2)[1:], oracle.bnb_quantize(code, x[1:]))
    # an unsorted table still follows the same compare sequence
    shuffled = np.random.default_rng(3).permutation(code).astype(np.float32)
    x = np.random.default_rng(4).uniform(-1.1, 1.1, 4096).astype(np.float32)
    out = torch.empty(4096, dtype=torch.uint8, device=dev)
    hq.kQuantize(to_dev(shuffled, dev), to_dev(x, dev), out, 4096)
    assert np.array_equal(_np(out), oracle.bnb_quantize(shuffled, x))
    # n = 0 is a no-op
    hq.kQuantize(dcode, to_dev(x, dev), out, 0)


def test_bnb_against_reference_kernel(hq, oracle, dev):
    import torch
    ref = refgpu.load()
    if ref is None:
        pytest.skip("reference CUDA build not present")
    g = np.load(GOLDEN / "bnb_golden.npz")
    n = 1 << 20
    x = np.random.default_rng(19937).standard_normal(n).astype(np.float32)
    dcode, dx = to_dev(g["code"], dev), to_dev(x, dev)
    a = torch.empty(n, dtype=torch.uint8, device=dev)
    b = torch.empty(n, dtype=torch.uint8, device=dev)
    ref.ref_bnb_quantize_gpu(C.c_void_p(dcode.data_ptr()), C.c_void_p(dx.data_ptr()),
                             C.c_void_p(a.data_ptr()), n)
    hq.kQuantize(dcode, dx, b, n)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    assert np.array_equal(_np(b), oracle.bnb_quantize(g["code"], x))


# ------------------------------------------------------------------ nf4

@pytest.mark.parametrize("N,K,bs,order", [
    (64, 256, 64, 0), (11008, 4096, 64, 0), (37, 1024, 64, 1), (5, 4096, 128, 0),
    (130, 96, 32, 1), (16, 8192, 64, 0),
    # one row, fewer rows than CTAs, one more than the CTA count, every K / 1024, large
    # and small blocks, low-nibble-first
    (1, 4096, 64, 0), (149, 2048, 64, 1), (2369, 3072, 64, 0), (40000, 1024, 256, 0),
    (24000, 4096, 1024, 1), (300, 4096, 32, 0),
    # ragged rows, long rows
    (33, 1056, 32, 0), (9, 12288, 64, 0), (3, 33792, 64, 1)])
@pytest.mark.parametrize("form", ["register", "bulk"])
def test_nf4_gemv_and_dequant(hq, oracle, dev, monkeypatch, N, K, bs, order, form):
    """form "bulk": the opt-in bulk-copy GEMV (rows of 1024 .. 4096 inputs; every
    other shape must still fall back to the register pipeline)."""
    import torch
    if form == "bulk":
        monkeypatch.setenv("HQ_NF4_BULK", "1")
    else:
        monkeypatch.delenv("HQ_NF4_BULK", raising=False)
    A, B, absmax, lut = synth.nf4_case(N, K, bs, seed=N + K)
    dA = to_dev(A.view(np.uint16), dev).view(torch.float16)
    dB, dabs, dlut = to_dev(B, dev), to_dev(absmax, dev), to_dev(lut, dev)
    deq = hq.dequantize_nf4(dB, dabs, dlut, N * K, bs, order)
    want = oracle.nf4_dequant_f16(B, absmax, lut, N * K, bs, order)
    assert np.array_equal(_np(deq).view(np.uint16), want.view(np.uint16))
    y = hq.gemv_nf4(dA, dB, dabs, dlut, N, K, bs, order)
    ref = oracle.nf4_gemv_f64(A, B, absmax, lut, N, K, bs, order)
    assert oracle.rel_err(_np(y).astype(np.float64), ref) < TOL_F16


def test_nf4_gemv_chain_with_resident_weights(hq, dev):
    """A chain of square layers in which every launch reads the previous
    launch's output: with the weights flagged resident a launch may start
    before its predecessor has finished, but must read its input only
    afterwards.  Eager and graph-replayed chains must equal the plain chain
    bit for bit."""
    import torch
    N = K = 4096
    layers = 6
    _, B0, absmax, lut = synth.nf4_case(N, K, 64, seed=9)
    x0 = torch.from_numpy((np.random.default_rng(3).standard_normal(K) * 4).astype(np.float16)).to(dev)
    Bs = [to_dev(np.roll(B0, 17 * i), dev) for i in range(layers)]
    dabs, dlut = to_dev(absmax * 0.2, dev), to_dev(lut, dev)

    def chain(flag):
        bufs = [torch.empty(N, dtype=torch.float16, device=dev) for _ in range(layers)]
        x = x0
        for i in range(layers):
            hq.gemv_nf4(x, Bs[i], dabs, dlut, N, K, 64, 0, bufs[i], weights_resident=flag)
            x = bufs[i]
        return bufs

    plain = [b.clone() for b in chain(False)]
    torch.cuda.synchronize()
    assert float(plain[-1].float().abs().max()) > 0
    for _ in range(5):
        got = chain(True)
        torch.cuda.synchronize()
        for a, b in zip(plain, got):
            assert torch.equal(a, b)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        chain(True)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            got = chain(True)
        for _ in range(5):
            for b in got:
                b.zero_()
            g.replay()
            stream.synchronize()
            for a, b in zip(plain, got):
                assert torch.equal(a, b)


def test_nf4_dequant_then_dense_matches_gemv(hq, oracle, dev):
    """Size-independent property at the full configuration: GEMV equals the
    dense product with the bit-exact dequantised weights."""
    import torch
    N, K, bs = 11008, 4096, 64
    A, B, absmax, lut = synth.nf4_case(N, K, bs, seed=1)
    dA = to_dev(A.view(np.uint16), dev).view(torch.float16)
    dB, dabs, dlut = to_dev(B, dev), to_dev(absmax, dev), to_dev(lut, dev)
    W = hq.dequantize_nf4(dB, dabs, dlut, N * K, bs).view(N, K)
    dense = (W.double() @ dA.double())
    y = hq.gemv_nf4(dA, dB, dabs, dlut, N, K, bs)
    assert oracle.rel_err(_np(y).astype(np.float64), _np(dense)) < TOL_F16


# ------------------------------------------------------------------ lut-gemm

@pytest.mark.parametrize("M,K,nb,gs,bias", [
    (2048, 1024, 3, 128, True), (4096, 1024, 3, 128, False), (1024, 512, 4, 128, True),
    (512, 256, 8, 128, True), (260, 160, 3, 32, True), (1024, 256, 2, 64, True),
    (12288, 12288, 3, 128, True), (256, 512, 1, 256, False), (64, 4096, 5, 512, True),
    (1024, 768, 3, 192, True), (516, 960, 5, 320, False)])  # groups of 192 / 320 inputs: 64-input tiles
@pytest.mark.parametrize("form", ["register", "bulk"])
def test_lutgemm_nqmv(hq, oracle, dev, monkeypatch, M, K, nb, gs, bias, form):
    """form "bulk": the opt-in bulk-copy kernel (shapes it does not take fall back)."""
    import torch
    if form == "bulk":
        monkeypatch.setenv("HQ_LUT_BULK", "1")
    else:
        monkeypatch.delenv("HQ_LUT_BULK", raising=False)
    x, bW, alpha, qb = synth.lutgemm_case(M, K, nb, gs, seed=M + K + nb, bias=bias)
    w = hq.nQWeight_fp16()
    w.parsing(bW, alpha.astype(np.float32), K, M, nb, False, K // gs,
              None if qb is None else qb.astype(np.float32), device=dev)
    dx = to_dev(x.view(np.uint16), dev).view(torch.float16)
    out = torch.full((M,), 7.0, dtype=torch.float16, device=dev)  # must be overwritten
    hq.matmul(out, dx, w)
    ref = oracle.lutgemm_gemv_f64(x, bW, alpha, qb, M, K, nb, gs)
    assert oracle.rel_err(_np(out).astype(np.float64), ref) < TOL_F16
    # the scratch is left zero: a second call gives the same answer
    out2 = torch.empty(M, dtype=torch.float16, device=dev)
    hq.matmul(out2, dx, w)
    assert oracle.rel_err(_np(out2).astype(np.float64), ref) < TOL_F16
    assert torch.count_nonzero(w.workspace()) == 0


def test_lutgemm_against_reference_kernel(hq, oracle, dev):
    import torch
    ref = refgpu.load()
    if ref is None:
        pytest.skip("reference CUDA build not present")
    M, K, nb, gs = 4096, 1024, 3, 128
    x, bW, alpha, qb = synth.lutgemm_case(M, K, nb, gs, seed=2)
    w = hq.nQWeight_fp16(bW, alpha.astype(np.float32), K, M, nb, False, K // gs,
                         qb.astype(np.float32), device=dev)
    dx = to_dev(x.view(np.uint16), dev).view(torch.float16)
    a = torch.empty(M, dtype=torch.float16, device=dev)
    b = torch.empty(M, dtype=torch.float16, device=dev)
    ref.ref_lutgemm_matmul(C.c_void_p(a.data_ptr()), C.c_void_p(dx.data_ptr()),
                           C.c_void_p(w.bWeight.data_ptr()), C.c_void_p(w.alpha.data_ptr()),
                           C.c_void_p(w.q_bias.data_ptr()), M, K, nb, K // gs)
    hq.matmul(b, dx, w)
    torch.cuda.synchronize()
    y64 = oracle.lutgemm_gemv_f64(x, bW, alpha, qb, M, K, nb, gs)
    # the reference accumulates in fp16 (tables, tile sums and atomics)
    assert oracle.rel_err(_np(a).astype(np.float64), y64) < 5e-2
    assert oracle.rel_err(_np(b).astype(np.float64), y64) < TOL_F16
    assert oracle.rel_err(_np(b).astype(np.float64), y64) <= oracle.rel_err(_np(a).astype(np.float64), y64)


# ------------------------------------------------------------------ aqlm

@pytest.mark.parametrize("m,k,ncb", [(4096, 4096, 1), (12288, 4096, 3), (100, 512, 1), (33, 8192, 1),
                                     (7, 64, 1)])
def test_aqlm_1x16(hq, oracle, dev, m, k, ncb):
    import torch
    codes, x, cb, scales = synth.aqlm_1x16_case(m, k, ncb, seed=m + k)
    sizes = [m, m, m, 1 << 30] if ncb == 1 else [m // 3, 2 * (m // 3), m, 1 << 30]
    stride = 65536 * 8 * 2 // 16
    dcodes = to_dev(codes, dev)
    dx = to_dev(x.view(np.uint16), dev).view(torch.float16)
    dcb = to_dev(cb.view(np.uint16), dev).view(torch.float16)
    out = torch.empty(m, dtype=torch.float16, device=dev)
    hq.code1x16_matvec(dcodes, dx, out, dcb, m, k, sizes, stride)
    # bit-identical to the restated reference arithmetic
    want = oracle.aqlm_1x16_ref(codes, x, cb, m, k, sizes, stride)
    assert np.array_equal(_np(out).view(np.uint16), want.view(np.uint16))
    assert oracle.rel_err(_np(out).astype(np.float64),
                          oracle.aqlm_1x16_f64(codes, x, cb, m, k, sizes, stride)) < TOL_F16
    # per-output scale (extension)
    ds = to_dev(scales.view(np.uint16), dev).view(torch.float16)
    hq.code1x16_matvec(dcodes, dx, out, dcb, m, k, sizes, stride, ds)
    want = oracle.aqlm_1x16_ref(codes, x, cb, m, k, sizes, stride, scales)
    assert np.array_equal(_np(out).view(np.uint16), want.view(np.uint16))


def test_aqlm_1x16_against_reference_kernel(hq, oracle, dev):
    import torch
    ref = refgpu.load()
    if ref is None:
        pytest.skip("reference CUDA build not present")
    m, k = 12288, 4096
    codes, x, cb, _ = synth.aqlm_1x16_case(m, k, 3, seed=3)
    sizes = [4096, 8192, 12288, 122880]  # quantAQLM-cuda/main.cu:160
    stride = 65536 * 8 * 2 // 16
    dcodes = to_dev(codes, dev)
    dx = to_dev(x.view(np.uint16), dev)
    dcb = to_dev(cb.view(np.uint16), dev)
    a = torch.zeros(m, dtype=torch.float16, device=dev)
    b = torch.zeros(m, dtype=torch.float16, device=dev)
    ref.ref_aqlm_1x16(C.c_void_p(dcodes.data_ptr()), C.c_void_p(dx.data_ptr()), C.c_void_p(a.data_ptr()),
                      C.c_void_p(dcb.data_ptr()), m, k, (C.c_int * 4)(*sizes), stride)
    hq.code1x16_matvec(dcodes, dx.view(torch.float16), b, dcb.view(torch.float16), m, k, sizes, stride)
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    want = oracle.aqlm_1x16_ref(codes, x, cb, m, k, sizes, stride)
    assert np.array_equal(_np(a).view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("m,k", [(4096, 4096), (100, 512), (5, 64), (1000, 8192)])
def test_aqlm_2x8(hq, oracle, dev, m, k):
    import torch
    codes, x, cbs, scales = synth.aqlm_2x8_case(m, k, seed=m + k)
    dcodes = to_dev(codes, dev)
    dx = to_dev(x.view(np.uint16), dev).view(torch.float16)
    dcb = to_dev(cbs.view(np.uint16), dev).view(torch.float16)
    ds = to_dev(scales.view(np.uint16), dev).view(torch.float16)
    out = torch.empty(m, dtype=torch.float16, device=dev)
    hq.code2x8_matvec(dcodes, dx, out, dcb, m, k, ds)
    assert oracle.rel_err(_np(out).astype(np.float64),
                          oracle.aqlm_2x8_f64(codes, x, cbs, m, k, scales)) < TOL_F16
    hq.code2x8_matvec(dcodes, dx, out, dcb, m, k)
    assert oracle.rel_err(_np(out).astype(np.float64),
                          oracle.aqlm_2x8_f64(codes, x, cbs, m, k)) < TOL_F16
