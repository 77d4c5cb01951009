"""RMSNorm -> weight-only mat-vec -> gated activation in one launch
(hq_gemv_fused_*), against the fp64 CPU oracle that restates the host references
of rmsnorm-cuda, geglu-cuda and swish-cuda around the format's mat-vec, and
against the same computation done with the library's separate kernels."""
import numpy as np
import pytest

from hecbench_b200 import synth
from conftest import to_dev

pytestmark = pytest.mark.gpu
TOL_F16 = 1e-2


def _case(fmt, rows_mat, n, seed):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(n) * 3).astype(np.float16)
    gamma = rng.uniform(0.5, 1.5, n).astype(np.float16)
    kw = {}
    if fmt == "nf4":
        _, B, absmax, lut = synth.nf4_case(rows_mat, n, 64, seed)
        mat = B.reshape(rows_mat, n // 2)
        kw = dict(absmax=absmax, lut16=lut, blocksize=64)
    else:
        bits = {"f16": 16, "int8": 8, "int4": 4}[fmt]
        mat, _ = synth.gemv_uniform_case(rows_mat, n, bits, seed)
        if fmt == "f16":
            mat = (mat - np.float16(0.5)).astype(np.float16)
        else:
            # small enough that value * gate of un-normalised inputs stays inside fp16
            kw = dict(scale=0.002 if fmt == "int8" else 0.02,
                      zero_point=1.5 if fmt == "int8" else 7.5)
    return x, gamma, mat, kw


def _dev_kw(kw, dev):
    return {k: (to_dev(v, dev) if isinstance(v, np.ndarray) else v) for k, v in kw.items()}


@pytest.mark.parametrize("fmt", ["nf4", "int4", "int8", "f16"])
@pytest.mark.parametrize("rows_out,n,act,norm", [
    (1024, 4096, 1, True),     # SwiGLU gate/up pairs with RMSNorm: the decoder MLP entry
    (1000, 2048, 2, True),     # GeGLU
    (512, 1024, 0, True),      # RMSNorm + plain mat-vec
    (333, 2048, 1, False),     # no normalisation, an odd number of outputs
    (7, 8192, 0, False)])      # plain mat-vec, an odd number of rows (a lone last row)
def test_fused_against_oracle(hq, oracle, dev, fmt, rows_out, n, act, norm):
    rows_mat = rows_out * (2 if act else 1)
    x, gamma, mat, kw = _case(fmt, rows_mat, n, seed=rows_out + n + act)
    y = hq.gemv_fused(fmt, to_dev(x, dev), to_dev(mat, dev), rows_out,
                      gamma=to_dev(gamma, dev) if norm else None, eps=1e-5, act=act,
                      **_dev_kw(kw, dev))
    okw = dict(kw)
    ref = oracle.gemv_fused_f64(fmt, mat, x, gamma if norm else None, 1e-5, rows_out, act, **okw)
    assert y.shape == (rows_out,)
    assert oracle.rel_err(y.cpu().numpy().astype(np.float64), ref) < TOL_F16


@pytest.mark.parametrize("rows_out,n,bs,act", [
    (300, 1024, 64, 1),      # one warp per row
    (300, 512, 128, 2),      # rows shorter than a warp's 1024 inputs
    (1024, 4096, 64, 1),     # two warps per row, compile-time form
    (777, 8192, 64, 2),      # run-time number of warps per row
    (96, 11008, 64, 1),      # ragged last slice (11008 = 10 * 1024 + 768)
    (64, 2080, 96, 1),       # blocks that straddle rows (not a power of two)
    (40, 40960, 64, 0)])     # four chunks per lane
def test_fused_nf4_kernel_forms(hq, oracle, dev, rows_out, n, bs, act):
    """Every form of the NF4 kernel (chunks per lane, warps per row, aligned or
    straddling absmax blocks) with the RMSNorm and the row pairing switched on,
    in both nibble orders."""
    rows_mat = rows_out * (2 if act else 1)
    rng = np.random.default_rng(n + act)
    x = (rng.standard_normal(n) * 3).astype(np.float16)
    gamma = rng.uniform(0.5, 1.5, n).astype(np.float16)
    _, B, absmax, lut = synth.nf4_case(rows_mat, n, bs, seed=n)
    mat = B.reshape(rows_mat, n // 2)
    for order in (0, 1):
        y = hq.gemv_fused("nf4", to_dev(x, dev), to_dev(mat, dev), rows_out,
                          gamma=to_dev(gamma, dev), eps=1e-5, act=act, absmax=to_dev(absmax, dev),
                          lut16=to_dev(lut, dev), blocksize=bs, nibble_order=order)
        ref = oracle.gemv_fused_f64("nf4", mat, x, gamma, 1e-5, rows_out, act, absmax=absmax,
                                    lut16=lut, blocksize=bs, low_first=order)
        assert oracle.rel_err(y.cpu().numpy().astype(np.float64), ref) < TOL_F16


def test_fused_equals_separate_kernels_nf4(hq, oracle, dev):
    """Without normalisation and activation the fused NF4 form is the plain NF4
    GEMV: both must agree to fp16 rounding on the same inputs (low-nibble-first
    order included)."""
    import torch
    N, K = 2048, 4096
    A, B, absmax, lut = synth.nf4_case(N, K, 64, seed=3)
    dA = to_dev(A.view(np.uint16), dev).view(torch.float16)
    dB, dabs, dlut = to_dev(B, dev), to_dev(absmax, dev), to_dev(lut, dev)
    for order in (0, 1):
        plain = hq.gemv_nf4(dA, dB, dabs, dlut, N, K, 64, order)
        fused = hq.gemv_fused("nf4", dA, dB.view(N, K // 2), N, absmax=dabs, lut16=dlut,
                              blocksize=64, nibble_order=order)
        ref = oracle.nf4_gemv_f64(A, B, absmax, lut, N, K, 64, order)
        assert oracle.rel_err(fused.cpu().numpy().astype(np.float64), ref) < TOL_F16
        assert oracle.rel_err(fused.cpu().numpy().astype(np.float64),
                              plain.cpu().numpy().astype(np.float64)) < TOL_F16


def test_fused_argument_errors(hq, dev):
    import torch
    lib = hq.load_library()
    m = torch.zeros(64 * 64, dtype=torch.uint8, device=dev)
    v = torch.zeros(64, dtype=torch.float16, device=dev)
    o = torch.zeros(64, dtype=torch.float16, device=dev)
    f = torch.zeros(64, dtype=torch.float32, device=dev)
    p = lambda t: t.data_ptr()
    assert lib.hq_gemv_fused_int8_f16(p(v), None, 1e-5, None, p(o), 8, 64, 1.0, 0.0, 0, None) == -2
    assert lib.hq_gemv_fused_int8_f16(p(v), None, 1e-5, p(m), p(o), 8, 64, 1.0, 0.0, 3, None) == -1
    assert lib.hq_gemv_fused_int4_f16(p(v), None, 1e-5, p(m), p(o), 8, 48, 1.0, 0.0, 0, None) == -1
    assert lib.hq_gemv_fused_nf4_f16(p(v), None, 1e-5, p(m), None, p(f), p(o), 8, 64, 64, 0, 0,
                                     None) == -2
    assert lib.hq_gemv_fused_nf4_f16(p(v), None, 1e-5, p(m), p(f), p(f), p(o), 8, 64, 48, 0, 0,
                                     None) == -1   # blocks are multiples of 32 codes
    assert lib.hq_gemv_fused_nf4_f16(p(v), None, 1e-5, p(m), p(f), p(f), p(o), 8, 64, 64, 0, 5,
                                     None) == -1   # unknown activation
    assert lib.hq_gemv_fused_nf4_f16(p(v), p(v) + 2, 1e-5, p(m), p(f), p(f), p(o), 8, 64, 64, 0, 0,
                                     None) == -3
    assert lib.hq_gemv_fused_f16(p(v) + 2, None, 1e-5, p(m), p(o), 8, 64, 0, None) == -3
    torch.cuda.synchronize()
