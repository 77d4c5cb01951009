"""numpy front end of oracle/liboracle.so (hq_oracle.c) and, when present, of
the reference-built oracle/_ref/libref_cpu.so.  TEST INFRASTRUCTURE ONLY.

fp16 tensors travel as numpy float16 arrays (viewed as uint16 for the C side).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_lib = None
_ref_cpu = None


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def lib():
    global _lib
    if _lib is None:
        p = HERE / "liboracle.so"
        if not p.exists():
            from . import build
            build.build_oracle()
        _lib = C.CDLL(str(p))
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def ref_cpu():
    """The reference's own quantBnB CPU code (None if it was never built)."""
    global _ref_cpu
    if _ref_cpu is None:
        p = HERE / "_ref" / "libref_cpu.so"
        if not p.exists():
            return None
        _ref_cpu = C.CDLL(str(p))
        _ref_cpu.ref_bnb_code_table.restype = C.POINTER(C.c_float)
    return _ref_cpu


def num_threads() -> int:
    return int(lib().orc_num_threads())


def _c(a, dtype):
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16 and dtype == np.uint16:
        a = a.view(np.uint16)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a


# ---------------- q3 ----------------

def q3_pack(codes: np.ndarray) -> np.ndarray:
    """codes uint8[K][width] -> int32[K*3/32][width]."""
    codes = _c(codes, np.uint8)
    K, width = codes.shape
    assert K % 32 == 0
    mat = np.empty((K * 3 // 32, width), dtype=np.int32)
    lib().orc_q3_pack(_ptr(codes), _ptr(mat), C.c_int(K), C.c_int(width))
    return mat


def q3_unpack(mat: np.ndarray) -> np.ndarray:
    mat = _c(mat, np.int32)
    height, width = mat.shape
    codes = np.empty((height * 32 // 3, width), dtype=np.uint8)
    lib().orc_q3_unpack(_ptr(mat), _ptr(codes), C.c_int(height), C.c_int(width))
    return codes


def q3_dequant_f32(mat, scales, zeros) -> np.ndarray:
    mat, scales, zeros = _c(mat, np.int32), _c(scales, np.float32), _c(zeros, np.float32)
    height, width = mat.shape
    W = np.empty((height * 32 // 3, width), dtype=np.float32)
    lib().orc_q3_dequant_f32(_ptr(mat), _ptr(scales), _ptr(zeros), _ptr(W), C.c_int(height),
                             C.c_int(width))
    return W


def q3_dequant_f16(mat, scales, zeros) -> np.ndarray:
    mat, scales, zeros = _c(mat, np.int32), _c(scales, np.float32), _c(zeros, np.float32)
    height, width = mat.shape
    W = np.empty((height * 32 // 3, width), dtype=np.uint16)
    lib().orc_q3_dequant_f16(_ptr(mat), _ptr(scales), _ptr(zeros), _ptr(W), C.c_int(height),
                             C.c_int(width))
    return W.view(np.float16)


def q3_gemv_f32(vec, mat, mul, scales, zeros) -> np.ndarray:
    """Reference-order fp32 result; returns mul + product."""
    vec, mat = _c(vec, np.float32), _c(mat, np.int32)
    out = np.array(mul, dtype=np.float32, copy=True)
    height, width = mat.shape
    lib().orc_q3_gemv_f32(_ptr(vec), _ptr(mat), _ptr(out), _ptr(_c(scales, np.float32)),
                          _ptr(_c(zeros, np.float32)), C.c_int(height), C.c_int(width))
    return out


def q3_gemv_f16in(vec_half, mat, mul, scales, zeros) -> np.ndarray:
    vec, mat = _c(vec_half, np.uint16), _c(mat, np.int32)
    out = np.array(mul, dtype=np.float32, copy=True)
    height, width = mat.shape
    lib().orc_q3_gemv_f16in(_ptr(vec), _ptr(mat), _ptr(out), _ptr(_c(scales, np.float32)),
                            _ptr(_c(zeros, np.float32)), C.c_int(height), C.c_int(width))
    return out


def q3_gemv_f64(vec, mat, scales, zeros, f16rule: bool = False) -> np.ndarray:
    vec = np.ascontiguousarray(np.asarray(vec, dtype=np.float32))
    mat = _c(mat, np.int32)
    height, width = mat.shape
    out = np.empty(width, dtype=np.float64)
    lib().orc_q3_gemv_f64(_ptr(vec), _ptr(mat), _ptr(out), _ptr(_c(scales, np.float32)),
                          _ptr(_c(zeros, np.float32)), C.c_int(height), C.c_int(width),
                          C.c_int(1 if f16rule else 0))
    return out


# ---------------- bnb ----------------

def bnb_quantize(code, A) -> np.ndarray:
    code, A = _c(code, np.float32), _c(A, np.float32)
    assert code.size == 256
    out = np.empty(A.size, dtype=np.uint8)
    lib().orc_bnb_quantize(_ptr(code), _ptr(A), _ptr(out), C.c_size_t(A.size))
    return out


def ref_bnb_code_table():
    r = ref_cpu()
    if r is None:
        return None
    return np.ctypeslib.as_array(r.ref_bnb_code_table(), shape=(256,)).copy()


def ref_bnb_quantize(A, threads: int = 0):
    r = ref_cpu()
    if r is None:
        return None
    A = _c(A, np.float32)
    out = np.empty(A.size, dtype=np.uint8)
    r.ref_bnb_quantize(_ptr(A), _ptr(out), C.c_size_t(A.size),
                       C.c_int(threads or (os.cpu_count() or 1)))
    return out


# ---------------- quantVLLM: per-token int8 activation quantization ----------------

VLLM_DTYPES = {"float16": 0, "bfloat16": 1, "float32": 2}


def _vllm_in(x, dtype: str):
    """fp16 arrays travel as float16, bf16 as uint16 bit patterns, fp32 as float32."""
    code = VLLM_DTYPES[dtype]
    want = {0: np.float16, 1: np.uint16, 2: np.float32}[code]
    x = np.ascontiguousarray(x)
    assert x.dtype == want and x.ndim == 2, (x.dtype, want)
    return x, code


def _vllm_static(fn, x, dtype, scale, azp):
    x, code = _vllm_in(x, dtype)
    out = np.empty(x.shape, dtype=np.int8)
    fn(_ptr(x), C.c_int(code), _ptr(out), C.c_float(scale), C.c_int32(azp),
       C.c_longlong(x.shape[0]), C.c_int(x.shape[1]))
    return out


def _vllm_dynamic(fn, x, dtype, with_azp):
    x, code = _vllm_in(x, dtype)
    out = np.empty(x.shape, dtype=np.int8)
    scale = np.empty(x.shape[0], dtype=np.float32)
    azp = np.empty(x.shape[0], dtype=np.int32) if with_azp else None
    fn(_ptr(x), C.c_int(code), _ptr(out), _ptr(scale), _ptr(azp) if with_azp else None,
       C.c_longlong(x.shape[0]), C.c_int(x.shape[1]))
    return out, scale, azp


def vllm_static_quant(x, dtype: str, scale: float, azp: int = 0) -> np.ndarray:
    """static_scaled_int8_quant (quantVLLM-cuda/reference.h:1-31); azp == 0 = no zero point."""
    return _vllm_static(lib().orc_vllm_static_quant, x, dtype, scale, azp)


def vllm_dynamic_quant(x, dtype: str, with_azp: bool = False):
    """dynamic_scaled_int8_quant (reference.h:33-93): (int8 out, fp32 scale per token,
    int32 azp per token or None)."""
    return _vllm_dynamic(lib().orc_vllm_dynamic_quant, x, dtype, with_azp)


def ref_vllm_static_quant(x, dtype: str, scale: float, azp: int = 0):
    r = ref_cpu()
    if r is None or not hasattr(r, "ref_vllm_static_quant"):
        return None
    return _vllm_static(r.ref_vllm_static_quant, x, dtype, scale, azp)


def ref_vllm_dynamic_quant(x, dtype: str, with_azp: bool = False):
    r = ref_cpu()
    if r is None or not hasattr(r, "ref_vllm_dynamic_quant"):
        return None
    return _vllm_dynamic(r.ref_vllm_dynamic_quant, x, dtype, with_azp)


# ---------------- nf4 ----------------

def nf4_dequant_f16(B, absmax, lut16, n, blocksize=64, low_first=0) -> np.ndarray:
    B, absmax, lut16 = _c(B, np.uint8), _c(absmax, np.float32), _c(lut16, np.float32)
    out = np.empty(n, dtype=np.uint16)
    lib().orc_nf4_dequant_f16(_ptr(B), _ptr(absmax), _ptr(lut16), _ptr(out), C.c_size_t(n),
                              C.c_int(blocksize), C.c_int(low_first))
    return out.view(np.float16)


def nf4_gemv_f64(A, B, absmax, lut16, N, K, blocksize=64, low_first=0) -> np.ndarray:
    A, B = _c(A, np.uint16), _c(B, np.uint8)
    out = np.empty(N, dtype=np.float64)
    lib().orc_nf4_gemv_f64(_ptr(A), _ptr(B), _ptr(_c(absmax, np.float32)),
                           _ptr(_c(lut16, np.float32)), _ptr(out), C.c_int(N), C.c_int(K),
                           C.c_int(blocksize), C.c_int(low_first))
    return out


def nf4_gemv_f32(A, B, absmax, lut16, N, K, blocksize=64, low_first=0) -> np.ndarray:
    A, B = _c(A, np.uint16), _c(B, np.uint8)
    out = np.empty(N, dtype=np.uint16)
    lib().orc_nf4_gemv_f32(_ptr(A), _ptr(B), _ptr(_c(absmax, np.float32)),
                           _ptr(_c(lut16, np.float32)), _ptr(out), C.c_int(N), C.c_int(K),
                           C.c_int(blocksize), C.c_int(low_first))
    return out.view(np.float16)


# ---------------- gemv (uniform int8 / int4) ----------------

def gemv_uniform_f64(mat, vec, bits: int, scale: float = 1.0, zero_point: float = 0.0) -> np.ndarray:
    """fp64 truth of gemv-cuda's kernels: mat fp16 [rows][n] (bits 16), int8
    [rows][n] (bits 8) or uint8 [rows][n/2] (bits 4); scale and zero point are
    rounded to fp16 first, as the reference launchers do."""
    dt = {16: np.uint16, 8: np.int8, 4: np.uint8}[bits]
    mat = _c(mat.view(np.uint16) if mat.dtype == np.float16 else mat, dt)
    rows = mat.shape[0]
    n = mat.shape[1] * (2 if bits == 4 else 1)
    vec = _c(vec, np.uint16)
    out = np.empty(rows, dtype=np.float64)
    sh = int(np.float16(scale).view(np.uint16))
    zh = int(np.float16(zero_point).view(np.uint16))
    lib().orc_gemv_uniform_f64(_ptr(mat), _ptr(vec), _ptr(out), C.c_int(rows), C.c_int(n),
                               C.c_int(bits), C.c_uint16(sh), C.c_uint16(zh))
    return out


def gemv_fused_f64(fmt: str, mat, x, gamma, eps: float, rows_out: int, act: int = 0, scale: float = 1.0,
                   zero_point: float = 0.0, absmax=None, lut16=None, blocksize: int = 64,
                   low_first: int = 0) -> np.ndarray:
    """fp64 truth of RMSNorm -> mat-vec -> gated activation (rmsnorm-cuda,
    geglu-cuda and swish-cuda host references around the format's mat-vec).
    fmt: "f16", "int8", "int4" or "nf4"; gamma None = no normalisation; act 0
    none, 1 SwiGLU, 2 GeGLU (then mat has 2 * rows_out rows, value / gate
    interleaved)."""
    code = {"f16": 16, "int8": 8, "int4": 4, "nf4": 40}[fmt]
    dt = {16: np.uint16, 8: np.int8, 4: np.uint8, 40: np.uint8}[code]
    mat = _c(mat.view(np.uint16) if mat.dtype == np.float16 else mat, dt)
    x = _c(x, np.uint16)
    n = x.size
    out = np.empty(rows_out, dtype=np.float64)
    g = None if gamma is None else _c(gamma, np.uint16)
    am = None if absmax is None else _c(absmax, np.float32)
    lt = None if lut16 is None else _c(lut16, np.float32)
    sh = int(np.float16(scale).view(np.uint16))
    zh = int(np.float16(zero_point).view(np.uint16))
    lib().orc_gemv_fused_f64(C.c_int(code), _ptr(mat), None if am is None else _ptr(am),
                             None if lt is None else _ptr(lt), C.c_int(low_first),
                             C.c_int(blocksize), _ptr(x), None if g is None else _ptr(g),
                             C.c_double(eps), _ptr(out), C.c_int(rows_out), C.c_int(n),
                             C.c_int(act), C.c_uint16(sh), C.c_uint16(zh))
    return out


def ref_fused_f32(W, x, gamma, rows_out: int, act: int):
    """RMSNorm -> W @ xn -> gated activation where the three operators are the
    reference's own host checks (oracle/_ref: rmsnorm_forward_cpu, geglu_reference,
    swish reference; eps fixed at 1e-5) and only the product between them is numpy
    (fp64, rounded to fp32).  W: dequantized fp32 weights [rows][n].  None if the
    reference build is absent."""
    r = ref_cpu()
    if r is None or not hasattr(r, "ref_rmsnorm_f32"):
        return None
    W = np.asarray(W, dtype=np.float32)
    xf = _c(np.asarray(x, dtype=np.float32), np.float32)
    n = xf.size
    xn = xf
    if gamma is not None:
        g = _c(np.asarray(gamma, dtype=np.float32), np.float32)
        xn = np.empty(n, dtype=np.float32)
        r.ref_rmsnorm_f32(_ptr(xn), _ptr(xf), _ptr(g), C.c_int64(1), C.c_int64(n))
    y = _c((W.astype(np.float64) @ xn.astype(np.float64)).astype(np.float32), np.float32)
    if act == 0:
        return y
    out = np.empty(rows_out, dtype=np.float32)
    if act == 2:
        r.ref_geglu_f32(_ptr(out), _ptr(y), C.c_int(rows_out), C.c_int(1))
        return out
    gate = _c(y[1::2], np.float32)
    sw = np.empty(rows_out, dtype=np.float32)
    r.ref_swish_f32(_ptr(gate), _ptr(sw), C.c_int(rows_out))
    return y[0::2] * sw


def q3_quantize(W):
    """(mat int32[K*3/32][N], scales fp32[N], zeros fp32[N]) of fp32-widened W[K][N]."""
    W = _c(np.asarray(W, dtype=np.float32), np.float32)
    K, N = W.shape
    mat = np.empty((K * 3 // 32, N), dtype=np.int32)
    scales = np.empty(N, dtype=np.float32)
    zeros = np.empty(N, dtype=np.float32)
    lib().orc_q3_quantize(_ptr(W), C.c_int(K), C.c_int(N), _ptr(mat), _ptr(scales), _ptr(zeros))
    return mat, scales, zeros


def nf4_quantize(w, blocksize: int, lut16, low_first: int = 0):
    """(codes uint8[n / 2], absmax fp32[n / blocksize]) of fp32-widened weights."""
    w = _c(np.asarray(w, dtype=np.float32).reshape(-1), np.float32)
    lut16 = _c(lut16, np.float32)
    B = np.empty(w.size // 2, dtype=np.uint8)
    absmax = np.empty(w.size // blocksize, dtype=np.float32)
    lib().orc_nf4_quantize(_ptr(w), C.c_size_t(w.size), C.c_int(blocksize), _ptr(lut16),
                           C.c_int(low_first), _ptr(B), _ptr(absmax))
    return B, absmax


# ---------------- zero point ----------------

def _zero_point(fn, x_min, x_max, qmin, qmax, preserve_sparsity):
    x_min, x_max = _c(x_min, np.float32), _c(x_max, np.float32)
    scale = np.empty(x_min.size, dtype=np.float32)
    zp = np.empty(x_min.size, dtype=np.int32)
    fn(_ptr(x_min), _ptr(x_max), C.c_int32(qmin), C.c_int32(qmax), C.c_int(x_min.size),
       C.c_int(int(preserve_sparsity)), _ptr(scale), _ptr(zp))
    return scale, zp


def zero_point(x_min, x_max, qmin: int, qmax: int, preserve_sparsity: bool):
    """(scale fp32, zero point int32) per channel: the C restatement."""
    return _zero_point(lib().orc_zero_point, x_min, x_max, qmin, qmax, preserve_sparsity)


def ref_zero_point(x_min, x_max, qmin: int, qmax: int, preserve_sparsity: bool):
    """The same from the reference's own host function (None if it was never built)."""
    r = ref_cpu()
    if r is None or not hasattr(r, "ref_zero_point"):
        return None
    return _zero_point(r.ref_zero_point, x_min, x_max, qmin, qmax, preserve_sparsity)


# ---------------- MXFP4 ----------------

def mxfp4_qdq(x_bits, bf16: bool = False) -> np.ndarray:
    """Quantize-dequantize of 16-bit patterns of fp16 (or bf16) values, groups of 32."""
    x = _c(x_bits, np.uint16).reshape(-1)
    out = np.empty_like(x)
    lib().orc_mxfp4(_ptr(x), _ptr(out), None, None, C.c_size_t(x.size), C.c_int(int(bf16)))
    return out


def mxfp4_quantize(x_bits, bf16: bool = False):
    """(codes uint8[n/2], scales uint8[n/32]) of the packed form."""
    x = _c(x_bits, np.uint16).reshape(-1)
    codes = np.zeros(x.size // 2, dtype=np.uint8)
    scales = np.zeros(x.size // 32, dtype=np.uint8)
    lib().orc_mxfp4(_ptr(x), None, _ptr(codes), _ptr(scales), C.c_size_t(x.size),
                    C.c_int(int(bf16)))
    return codes, scales


def mxfp4_dequantize(codes, scales, bf16: bool = False) -> np.ndarray:
    codes, scales = _c(codes, np.uint8), _c(scales, np.uint8)
    out = np.empty(codes.size * 2, dtype=np.uint16)
    lib().orc_mxfp4_dequant(_ptr(codes), _ptr(scales), _ptr(out), C.c_size_t(out.size),
                            C.c_int(int(bf16)))
    return out


def mxfp4_scale_exponents(max_bits: int, bf16: bool = False):
    """(exponent used here, exponent by the reference's expression or None where
    that is undefined)."""
    ours = int(lib().orc_mxfp4_scale_exponent(C.c_uint16(max_bits), C.c_int(int(bf16))))
    ref = int(lib().orc_mxfp4_scale_exponent_ref(C.c_uint16(max_bits), C.c_int(int(bf16))))
    return ours, (None if ref == -1000 else ref)


# ---------------- lut-gemm ----------------

def lutgemm_dequant_f32(bW, alpha, q_bias, M, K, nb, group_size) -> np.ndarray:
    bW, alpha = _c(bW, np.uint32), _c(alpha, np.uint16)
    qb = None if q_bias is None else _c(q_bias, np.uint16)
    W = np.empty((K, M), dtype=np.float32)
    lib().orc_lutgemm_dequant_f32(_ptr(bW), _ptr(alpha), _ptr(qb) if qb is not None else None,
                                  _ptr(W), C.c_int(M), C.c_int(K), C.c_int(nb),
                                  C.c_int(group_size))
    return W


def lutgemm_quantize(W, nb: int, group_size: int, bias: bool = True):
    """(bW uint32[K/32][nb][M], alpha fp16[G][nb][M], q_bias fp16[G][M] or None) of
    fp32-widened W[K][M]."""
    W = _c(np.asarray(W, dtype=np.float32), np.float32)
    K, M = W.shape
    G = K // group_size
    bW = np.empty((K // 32, nb, M), dtype=np.uint32)
    alpha = np.empty((G, nb, M), dtype=np.uint16)
    qb = np.empty((G, M), dtype=np.uint16) if bias else None
    lib().orc_lutgemm_quantize(_ptr(W), C.c_int(K), C.c_int(M), C.c_int(nb), C.c_int(group_size),
                               _ptr(bW), _ptr(alpha), _ptr(qb) if bias else None)
    return bW, alpha.view(np.float16), (qb.view(np.float16) if bias else None)


def lutgemm_gemv_f64(x, bW, alpha, q_bias, M, K, nb, group_size) -> np.ndarray:
    x, bW, alpha = _c(x, np.uint16), _c(bW, np.uint32), _c(alpha, np.uint16)
    qb = None if q_bias is None else _c(q_bias, np.uint16)
    out = np.empty(M, dtype=np.float64)
    lib().orc_lutgemm_gemv_f64(_ptr(x), _ptr(bW), _ptr(alpha),
                               _ptr(qb) if qb is not None else None, _ptr(out), C.c_int(M),
                               C.c_int(K), C.c_int(nb), C.c_int(group_size))
    return out


def lutgemm_gemv_f32(x, bW, alpha, q_bias, M, K, nb, group_size) -> np.ndarray:
    x, bW, alpha = _c(x, np.uint16), _c(bW, np.uint32), _c(alpha, np.uint16)
    qb = None if q_bias is None else _c(q_bias, np.uint16)
    out = np.empty(M, dtype=np.uint16)
    lib().orc_lutgemm_gemv_f32(_ptr(x), _ptr(bW), _ptr(alpha),
                               _ptr(qb) if qb is not None else None, _ptr(out), C.c_int(M),
                               C.c_int(K), C.c_int(nb), C.c_int(group_size))
    return out.view(np.float16)


# ---------------- aqlm ----------------

def _sizes(cb_sizes):
    return (C.c_int * 4)(*[int(v) for v in cb_sizes])


def aqlm_1x16_ref(codes, x, codebook, prob_m, prob_k, cb_sizes, cb_stride_int4, scales=None):
    codes, x, codebook = _c(codes, np.uint16), _c(x, np.uint16), _c(codebook, np.uint16)
    sc = None if scales is None else _c(scales, np.uint16)
    out = np.empty(prob_m, dtype=np.uint16)
    lib().orc_aqlm_1x16_ref(_ptr(codes), _ptr(x), _ptr(out), _ptr(codebook), C.c_int(prob_m),
                            C.c_int(prob_k), _sizes(cb_sizes), C.c_int(cb_stride_int4),
                            _ptr(sc) if sc is not None else None)
    return out.view(np.float16)


def aqlm_1x16_f64(codes, x, codebook, prob_m, prob_k, cb_sizes, cb_stride_int4, scales=None):
    codes, x, codebook = _c(codes, np.uint16), _c(x, np.uint16), _c(codebook, np.uint16)
    sc = None if scales is None else _c(scales, np.uint16)
    out = np.empty(prob_m, dtype=np.float64)
    lib().orc_aqlm_1x16_f64(_ptr(codes), _ptr(x), _ptr(out), _ptr(codebook), C.c_int(prob_m),
                            C.c_int(prob_k), _sizes(cb_sizes), C.c_int(cb_stride_int4),
                            _ptr(sc) if sc is not None else None)
    return out


def aqlm_1x16_f32(codes, x, codebook, prob_m, prob_k, cb_sizes, cb_stride_int4, scales=None):
    codes, x, codebook = _c(codes, np.uint16), _c(x, np.uint16), _c(codebook, np.uint16)
    sc = None if scales is None else _c(scales, np.uint16)
    out = np.empty(prob_m, dtype=np.uint16)
    lib().orc_aqlm_1x16_f32(_ptr(codes), _ptr(x), _ptr(out), _ptr(codebook), C.c_int(prob_m),
                            C.c_int(prob_k), _sizes(cb_sizes), C.c_int(cb_stride_int4),
                            _ptr(sc) if sc is not None else None)
    return out.view(np.float16)


def aqlm_2x8_f64(codes, x, codebooks, prob_m, prob_k, scales=None):
    codes, x, codebooks = _c(codes, np.uint8), _c(x, np.uint16), _c(codebooks, np.uint16)
    sc = None if scales is None else _c(scales, np.uint16)
    out = np.empty(prob_m, dtype=np.float64)
    lib().orc_aqlm_2x8_f64(_ptr(codes), _ptr(x), _ptr(out), _ptr(codebooks), C.c_int(prob_m),
                           C.c_int(prob_k), _ptr(sc) if sc is not None else None)
    return out


# ---------------- batched ----------------

def gemm_f16_f64(X, Wd_kn) -> np.ndarray:
    """Y[Mb][N] = X[Mb][K] @ Wd[K][N], fp64 accumulation of fp16 operands."""
    X, Wd = _c(X, np.uint16), _c(Wd_kn, np.uint16)
    Mb, K = X.shape
    K2, N = Wd.shape
    assert K == K2
    Y = np.empty((Mb, N), dtype=np.float64)
    lib().orc_gemm_f16_f64(_ptr(X), _ptr(Wd), _ptr(Y), C.c_int(Mb), C.c_int(N), C.c_int(K))
    return Y


def gemm_f16_nk_f64(X, Wd_nk) -> np.ndarray:
    X, Wd = _c(X, np.uint16), _c(Wd_nk, np.uint16)
    Mb, K = X.shape
    N, K2 = Wd.shape
    assert K == K2
    Y = np.empty((Mb, N), dtype=np.float64)
    lib().orc_gemm_f16_nk_f64(_ptr(X), _ptr(Wd), _ptr(Y), C.c_int(Mb), C.c_int(N), C.c_int(K))
    return Y


def q3g_dequant_f16(mat, scales_h, zeros_h, K, N, group) -> np.ndarray:
    mat = _c(mat, np.int32)
    W = np.empty((K, N), dtype=np.uint16)
    lib().orc_q3g_dequant_f16(_ptr(mat), _ptr(_c(scales_h, np.uint16)),
                              _ptr(_c(zeros_h, np.uint16)), _ptr(W), C.c_int(K), C.c_int(N),
                              C.c_int(group))
    return W.view(np.float16)


def rel_err(y, ref) -> float:
    """max_i |y_i - ref_i| / max(|ref_i|, rms(ref)).

    A dot product whose terms cancel has no bounded element-wise relative
    error in any finite precision (the reference kernels included), so
    outputs smaller than the vector's RMS are measured against the RMS."""
    y = np.asarray(y, dtype=np.float64).ravel()
    ref = np.asarray(ref, dtype=np.float64).ravel()
    if ref.size == 0:
        return 0.0
    rms = float(np.sqrt(np.mean(ref * ref)))
    den = np.maximum(np.abs(ref), rms)
    den[den == 0] = 1.0
    return float(np.max(np.abs(y - ref) / den))


def rel_err_linf(y, ref, eps: float = 1e-3) -> float:
    """max_i |y_i - ref_i| / max(|ref_i|, eps * max_j |ref_j|): the element-wise
    relative error with only a small floor (eps of the largest output).  It is
    reported beside rel_err; for outputs that are the small difference of large
    terms it is dominated by cancellation, not by the kernel."""
    y = np.asarray(y, dtype=np.float64).ravel()
    ref = np.asarray(ref, dtype=np.float64).ravel()
    if ref.size == 0:
        return 0.0
    den = np.maximum(np.abs(ref), eps * float(np.max(np.abs(ref))))
    den[den == 0] = 1.0
    return float(np.max(np.abs(y - ref) / den))


def rel_err_above_floor(y, ref) -> float:
    """Worst plain relative error |y_i - ref_i| / |ref_i| over the outputs whose
    magnitude reaches the vector's RMS (the ones rel_err measures element-wise)."""
    y = np.asarray(y, dtype=np.float64).ravel()
    ref = np.asarray(ref, dtype=np.float64).ravel()
    if ref.size == 0:
        return 0.0
    rms = float(np.sqrt(np.mean(ref * ref)))
    big = np.abs(ref) >= max(rms, np.finfo(np.float64).tiny)
    if not np.any(big):
        return 0.0
    return float(np.max(np.abs(y[big] - ref[big]) / np.abs(ref[big])))
