"""The index-checked build (libhq_checked.so, -DHQ_BOUNDS_CHECK) on the GPU.

compute-sanitizer is not available where this library is developed, so the
instrumented kernels test every global access against the extent of the buffer
the caller described, record a violation and skip the access (nothing traps).
These tests run small and ragged parity cases of those kernels through the
checked library, compare the results with the oracle as usual, and then require
that not a single access was recorded."""
import ctypes as C

import numpy as np
import pytest

from hecbench_b200 import synth
from conftest import GOLDEN, to_dev

pytestmark = pytest.mark.gpu
TOL_F16 = 1e-2


@pytest.fixture()
def checked(hq, monkeypatch):
    from hecbench_b200 import _lib
    lib = _lib.load_checked_library()
    if lib is None:
        pytest.skip("libhq_checked.so was not built")
    hq.load_library()
    monkeypatch.setattr(_lib, "_lib", lib)  # the mirrored launchers now call the checked build
    assert lib.hq_bounds_check_report(None, None, None, None, 1) == 0
    return lib


def _violations(lib):
    n, site = C.c_uint(), C.c_uint()
    off, ext = C.c_ulonglong(), C.c_ulonglong()
    assert lib.hq_bounds_check_report(C.byref(n), C.byref(site), C.byref(off), C.byref(ext), 1) == 0
    return n.value, site.value, off.value, ext.value


def test_ordinary_build_has_no_checks(hq):
    assert hq.load_library().hq_bounds_check_report(None, None, None, None, 0) == -6


@pytest.mark.parametrize("N,K,bs", [(11008, 4096, 64), (333, 4096, 64), (5, 96, 32), (64, 2048, 128),
                                     (17, 8192, 64), (3, 33792, 64), (100, 1024, 64)])
def test_nf4_gemv_and_dequant_checked(hq, oracle, dev, checked, N, K, bs):
    A, B, absmax, lut = synth.nf4_case(N, K, bs, seed=N + K)
    dA, dB, da, dl = (to_dev(v, dev) for v in (A, B, absmax, lut))
    y = hq.gemv_nf4(dA, dB, da, dl, N, K, bs)
    ref = oracle.nf4_gemv_f64(A, B, absmax, lut, N, K, bs)
    assert oracle.rel_err(y.cpu().numpy().astype(np.float64), ref) < TOL_F16
    W = hq.dequantize_nf4(dB, da, dl, N * K, bs)
    assert np.array_equal(W.cpu().numpy().view(np.uint16),
                          oracle.nf4_dequant_f16(B, absmax, lut, N * K, bs).view(np.uint16))
    assert _violations(checked)[0] == 0, _violations(checked)


@pytest.mark.parametrize("M,K,nb,gs,bias", [(2048, 1024, 3, 128, True), (260, 160, 3, 32, True),
                                            (1024, 256, 2, 64, True), (516, 960, 5, 320, False),
                                            (64, 4096, 5, 512, True)])
def test_lutgemm_checked(hq, oracle, dev, checked, M, K, nb, gs, bias):
    import torch
    x, bW, alpha, qb = synth.lutgemm_case(M, K, nb, gs, seed=M + K + nb, bias=bias)
    w = hq.nQWeight_fp16(bW, alpha.astype(np.float32), K, M, nb, False, K // gs,
                         None if qb is None else qb.astype(np.float32), device=dev)
    out = torch.empty(M, dtype=torch.float16, device=dev)
    hq.matmul(out, to_dev(x.view(np.uint16), dev).view(torch.float16), w)
    ref = oracle.lutgemm_gemv_f64(x, bW, alpha, qb, M, K, nb, gs)
    assert oracle.rel_err(out.cpu().numpy().astype(np.float64), ref) < TOL_F16
    assert _violations(checked)[0] == 0


def test_kquantize_and_vllm_quant_checked(hq, oracle, dev, checked):
    import torch
    g = np.load(GOLDEN / "bnb_golden.npz")
    out = torch.empty(g["A"].size, dtype=torch.uint8, device=dev)
    hq.kQuantize(to_dev(g["code"], dev), to_dev(g["A"], dev), out, g["A"].size)
    assert np.array_equal(out.cpu().numpy(), g["out"])
    gv = np.load(GOLDEN / "vllm_golden.npz")
    x = to_dev(gv["x_float16"], dev)
    q = torch.empty(x.shape, dtype=torch.int8, device=dev)
    sc = torch.empty(x.shape[0], dtype=torch.float32, device=dev)
    hq.static_scaled_int8_quant(q, x, x.shape[1], x.shape[0], 0.1, 0)
    assert np.array_equal(q.cpu().numpy(), gv["static_float16"])
    hq.dynamic_scaled_int8_quant(q, x, x.shape[1], x.shape[0], sc, None)
    assert np.array_equal(q.cpu().numpy(), gv["dyn_float16"])
    assert _violations(checked)[0] == 0
