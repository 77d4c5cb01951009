"""gemv (uniform int8 / int4 weight-only mat-vec, plus the fp16 baseline) on the
GPU through the mirrored launchers: against the fp64 CPU oracle, which restates
the reference's own device-side checks (gemv-cuda/gemv.cu:83-141), and against
the reference's CUDA kernels run beside ours on the same buffers with the
reference launch shapes.  Inputs are drawn like the reference's
(simple_tensor.h:63-87)."""
import ctypes as C

import numpy as np
import pytest

from hecbench_b200 import synth
from conftest import to_dev
import refgpu

pytestmark = pytest.mark.gpu
TOL_F16 = 1e-2


def _run(hq, bits, mat, vec, scale, zp, dev):
    dm, dv = to_dev(mat, dev), to_dev(vec, dev)
    if bits == 16:
        return hq.gemv_fp16(dm, dv)
    if bits == 8:
        return hq.gemv_int8_quantized(dm, dv, scale, zp)
    return hq.gemv_int4_quantized(dm, dv, scale, zp)


@pytest.mark.parametrize("bits", [8, 4, 16])
@pytest.mark.parametrize("rows,n,scale,zp", [
    (512, 512, 0.0625, 0.01),      # the reference driver's defaults (main.cu:31-36)
    (4096, 4096, 0.0625, 0.01),
    (1000, 2048, 0.0123, 3.0),     # rows != n, a zero point that matters
    (37, 32, 1.0, 0.0),            # one chunk per row, fewer rows than warps
    (3, 24576, 0.001, 7.5),        # long rows, fewer rows than a CTA has warps
    (20, 65536, 0.001, 0.5),       # rows that leave room for one CTA per SM only
    (8192, 1056, 0.5, -2.0)])      # a row that is not a whole number of warp steps
def test_gemv_uniform_against_oracle(hq, oracle, dev, bits, rows, n, scale, zp):
    mat, vec = synth.gemv_uniform_case(rows, n, bits, seed=rows + n + bits)
    y = _run(hq, bits, mat, vec, scale, zp, dev)
    ref = oracle.gemv_uniform_f64(mat, vec, bits, scale, zp)
    assert y.shape == (rows,)
    assert oracle.rel_err(y.cpu().numpy().astype(np.float64), ref) < TOL_F16


def test_gemv_uniform_signed_inputs_and_extreme_codes(hq, oracle, dev):
    """Inputs of both signs (the reference only draws U(0,1)), all-minimum and
    all-maximum codes: the sign-flip / exponent-byte conversion of int8 and the
    nibble table of int4 must be exact at the ends of their ranges."""
    import torch
    n, rows = 2048, 64
    vec = (np.random.default_rng(5).standard_normal(n) * 2).astype(np.float16)
    for bits, lo, hi, dt in ((8, -128, 127, np.int8), (4, 0x00, 0xFF, np.uint8)):
        cols = n if bits == 8 else n // 2
        mat = np.empty((rows, cols), dtype=dt)
        mat[0::2] = lo
        mat[1::2] = hi
        y = _run(hq, bits, mat, vec, 0.25, 1.0, dev)
        ref = oracle.gemv_uniform_f64(mat, vec, bits, 0.25, 1.0)
        assert oracle.rel_err(y.cpu().numpy().astype(np.float64), ref) < TOL_F16
    # overwrite semantics: the result does not depend on what `out` held
    mat, vec = synth.gemv_uniform_case(256, 1024, 8, seed=2)
    out = torch.full((256,), 77.0, dtype=torch.float16, device=dev)
    hq.gemv_int8_quantized(to_dev(mat, dev), to_dev(vec, dev), 0.0625, 0.01, out=out)
    ref = oracle.gemv_uniform_f64(mat, vec, 8, 0.0625, 0.01)
    assert oracle.rel_err(out.cpu().numpy().astype(np.float64), ref) < TOL_F16


def test_gemv_uniform_argument_errors(hq, dev):
    import torch
    lib = hq.load_library()
    m = torch.zeros(64 * 64, dtype=torch.int8, device=dev)
    v = torch.zeros(64, dtype=torch.float16, device=dev)
    o = torch.zeros(64, dtype=torch.float16, device=dev)
    p = lambda t: t.data_ptr()
    assert lib.hq_gemv_int8_f16(None, p(v), p(o), 64, 64, 1.0, 0.0, None) == -2
    assert lib.hq_gemv_int8_f16(p(m), p(v), p(o), 64, 40, 1.0, 0.0, None) == -1      # n % 16
    assert lib.hq_gemv_int4_f16(p(m), p(v), p(o), 64, 48, 1.0, 0.0, None) == -1      # n % 32
    assert lib.hq_gemv_int8_f16(p(m) + 4, p(v), p(o), 4, 64, 1.0, 0.0, None) == -3   # alignment
    assert lib.hq_gemv_int4_f16(p(m), p(v), p(o), 1, 131072, 1.0, 0.0, None) == -7   # too long
    torch.cuda.synchronize()


@pytest.mark.parametrize("bits", [8, 4, 16])
def test_gemv_uniform_against_reference_kernel(hq, oracle, dev, bits):
    """The reference kernels with the reference driver's block shape (32 x 4,
    main.cu:33-34) on a square matrix: both results against the fp64 oracle; ours
    must be inside the tolerance and the two must agree to fp16 rounding."""
    import torch
    ref = refgpu.load()
    if ref is None or not hasattr(ref, "ref_gemv_int8"):
        pytest.skip("reference CUDA build not present")
    size, scale, zp = 2048, 0.0625, 0.01
    mat, vec = synth.gemv_uniform_case(size, size, bits, seed=bits)
    dm, dv = to_dev(mat, dev), to_dev(vec, dev)
    a = torch.empty(size, dtype=torch.float16, device=dev)
    args = (C.c_void_p(dm.data_ptr()), C.c_void_p(dv.data_ptr()), C.c_void_p(a.data_ptr()),
            C.c_uint(size))
    if bits == 8:
        ref.ref_gemv_int8(*args, C.c_float(scale), C.c_float(zp), C.c_uint(32), C.c_uint(4))
    elif bits == 4:
        ref.ref_gemv_int4(*args, C.c_float(scale), C.c_float(zp), C.c_uint(32), C.c_uint(4))
    else:
        ref.ref_gemv_f16(*args, C.c_uint(32), C.c_uint(4))
    b = _run(hq, bits, mat, vec, scale, zp, dev)
    torch.cuda.synchronize()
    y64 = oracle.gemv_uniform_f64(mat, vec, bits, scale, zp)
    ea = oracle.rel_err(a.cpu().numpy().astype(np.float64), y64)
    eb = oracle.rel_err(b.cpu().numpy().astype(np.float64), y64)
    assert ea < TOL_F16 and eb < TOL_F16
    assert oracle.rel_err(b.cpu().numpy().astype(np.float64),
                          a.cpu().numpy().astype(np.float64)) < TOL_F16
