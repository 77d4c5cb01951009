"""Host-side mirror of the reference launchers, on torch CUDA tensors.

Each function keeps the name, argument order and in/out convention of the
HeCBench launcher it stands in for (file:line given per function; paths
relative to the HeCBench source tree) and forwards to the C ABI of libhq.so on
the current torch CUDA stream.  Arguments are validated here the way the C ABI
validates them; errors surface as HqError / TypeError, never as a silent
fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from ._lib import check, load_library

NF4_HIGH_NIBBLE_FIRST = 0
NF4_WEIGHTS_RESIDENT = 2
NF4_LOW_NIBBLE_FIRST = 1


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dev(t: torch.Tensor, dtype: torch.dtype, name: str) -> int:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name}: expected a torch.Tensor")
    if not t.is_cuda:
        raise TypeError(f"{name}: must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name}: expected dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise TypeError(f"{name}: must be contiguous")
    return t.data_ptr()


# --------------------------------------------------------------------------
# quant3MatMul
# --------------------------------------------------------------------------

def vecquant3matmul(vec, mat, mul, scales, zeros, height: int, width: int) -> None:
    """vecquant3matmul<float> (quant3MatMul-cuda/kernels.h:171-190).

    mul[c] += sum_k (scales[c]*q[k][c] - zeros[c]) * vec[k]; `mul` is
    accumulated into, exactly like the reference (the caller zeroes it)."""
    lib = load_library()
    args = (
        _dev(vec, torch.float32, "vec"), _dev(mat, torch.int32, "mat"),
        _dev(mul, torch.float32, "mul"), _dev(scales, torch.float32, "scales"),
        _dev(zeros, torch.float32, "zeros"), height, width)
    with torch.cuda.device(mat.device):
        check("hq_q3_gemv_f32", lib.hq_q3_gemv_f32(*args, _stream()))


def vecquant3matmul_faster(vec, mat, mul, scales, zeros, height: int, width: int) -> None:
    """vecquant3matmul_faster (quant3MatMul-cuda/kernels.h:193-217): fp16 input."""
    lib = load_library()
    args = (
        _dev(vec, torch.float16, "vec"), _dev(mat, torch.int32, "mat"),
        _dev(mul, torch.float32, "mul"), _dev(scales, torch.float32, "scales"),
        _dev(zeros, torch.float32, "zeros"), height, width)
    with torch.cuda.device(mat.device):
        check("hq_q3_gemv_f16in", lib.hq_q3_gemv_f16in(*args, _stream()))


def vecquant3_dequant(mat, scales, zeros, height: int, width: int,
                      dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Dequantised weights W[K][width] by the fp32 rule (kernels.h:43) or the
    fp16 rule (kernels.h:121-122,137)."""
    lib = load_library()
    K = height * 32 // 3
    W = torch.empty((K, width), dtype=dtype, device=mat.device)
    fn = {torch.float32: "hq_q3_dequant_f32", torch.float16: "hq_q3_dequant_f16"}[dtype]
    args = (
        _dev(mat, torch.int32, "mat"), _dev(scales, torch.float32, "scales"),
        _dev(zeros, torch.float32, "zeros"), W.data_ptr(), height, width)
    with torch.cuda.device(mat.device):
        check(fn, getattr(lib, fn)(*args, _stream()))
    return W


# --------------------------------------------------------------------------
# quantBnB
# --------------------------------------------------------------------------

def kQuantize(code, A, out, n: int) -> None:
    """kQuantize<256,256><<<grid,block>>>(code, A, out, n)
    (quantBnB-cuda/main.cu:90-130,176)."""
    lib = load_library()
    if n > A.numel() or n > out.numel():
        raise ValueError("n exceeds the buffers")
    args = (
        _dev(code, torch.float32, "code"), _dev(A, torch.float32, "A"),
        _dev(out, torch.uint8, "out"), n)
    with torch.cuda.device(A.device):
        check("hq_bnb_quantize_u8", lib.hq_bnb_quantize_u8(*args, _stream()))


def dequantize_nf4(B, absmax, lut16, n: int, blocksize: int = 64,
                   nibble_order: int = NF4_HIGH_NIBBLE_FIRST,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """NF4 blockwise dequantize to fp16 (no counterpart in the reference tree):
    out[e] = half_rn(lut16[code_e] * absmax[e // blocksize])."""
    lib = load_library()
    if out is None:
        out = torch.empty(n, dtype=torch.float16, device=B.device)
    args = (
        _dev(B, torch.uint8, "B"), _dev(absmax, torch.float32, "absmax"),
        _dev(lut16, torch.float32, "lut16"), _dev(out, torch.float16, "out"),
        n, blocksize, nibble_order)
    with torch.cuda.device(B.device):
        check("hq_nf4_dequant_f16", lib.hq_nf4_dequant_f16(*args, _stream()))
    return out


def gemv_nf4(A, B, absmax, lut16, N: int, K: int, blocksize: int = 64,
             nibble_order: int = NF4_HIGH_NIBBLE_FIRST,
             out: Optional[torch.Tensor] = None, weights_resident: bool = False) -> torch.Tensor:
    """NF4 4-bit GEMV (no counterpart in the reference tree):
    out[n] = half(sum_k A[k] * lut16[code[n][k]] * absmax[(n*K+k)//blocksize]).
    weights_resident: B, absmax and lut16 are not written by earlier work in the
    stream, so the kernel may fetch them while the preceding kernel is finishing."""
    lib = load_library()
    if out is None:
        out = torch.empty(N, dtype=torch.float16, device=B.device)
    args = (
        _dev(A, torch.float16, "A"), _dev(B, torch.uint8, "B"),
        _dev(absmax, torch.float32, "absmax"), _dev(lut16, torch.float32, "lut16"),
        _dev(out, torch.float16, "out"), N, K, blocksize,
        nibble_order | (NF4_WEIGHTS_RESIDENT if weights_resident else 0))
    with torch.cuda.device(B.device):
        check("hq_nf4_gemv_f16", lib.hq_nf4_gemv_f16(*args, _stream()))
    return out


# --------------------------------------------------------------------------
# quantVLLM: per-token int8 activation quantization
# --------------------------------------------------------------------------

_VLLM_DTYPE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _vllm_input(input, hidden_size: int, num_tokens: int) -> int:
    if not isinstance(input, torch.Tensor) or not input.is_cuda:
        raise TypeError("input: must be a CUDA tensor (there is no CPU path)")
    if input.dtype not in _VLLM_DTYPE:
        raise TypeError(f"input: expected float16, bfloat16 or float32, got {input.dtype}")
    if not input.is_contiguous() or input.numel() != hidden_size * num_tokens:
        raise TypeError("input: must be contiguous [num_tokens][hidden_size]")
    return _VLLM_DTYPE[input.dtype]


def static_scaled_int8_quant(output, input, hidden_size: int, num_tokens: int, scale: float,
                             azp: int = 0) -> None:
    """static_scaled_int8_quant<scalar_t>(output, input, hidden_size, num_tokens,
    scale, azp) (quantVLLM-cuda/main.cu:137-153): azp == 0 selects the form
    without zero point, as in the reference."""
    lib = load_library()
    code = _vllm_input(input, hidden_size, num_tokens)
    if output.numel() != input.numel():
        raise ValueError("output and input differ in size")
    with torch.cuda.device(input.device):
        check("hq_vllm_static_scaled_int8_quant", lib.hq_vllm_static_scaled_int8_quant(
            _dev(output, torch.int8, "output"), input.data_ptr(), code, hidden_size, num_tokens,
            float(scale), int(azp), _stream()))


def dynamic_scaled_int8_quant(output, input, hidden_size: int, num_tokens: int, scales,
                              azp=None) -> None:
    """dynamic_scaled_int8_quant<scalar_t>(output, input, hidden_size, num_tokens,
    scales, azp) (quantVLLM-cuda/main.cu:155-172): scales float32[num_tokens]
    and, when azp (int32[num_tokens]) is given, the per-token zero points are
    written too."""
    lib = load_library()
    code = _vllm_input(input, hidden_size, num_tokens)
    if output.numel() != input.numel() or scales.numel() < num_tokens:
        raise ValueError("output / scales are too small")
    if azp is not None and azp.numel() < num_tokens:
        raise ValueError("azp is too small")
    with torch.cuda.device(input.device):
        check("hq_vllm_dynamic_scaled_int8_quant", lib.hq_vllm_dynamic_scaled_int8_quant(
            _dev(output, torch.int8, "output"), input.data_ptr(), code, hidden_size, num_tokens,
            _dev(scales, torch.float32, "scales"),
            0 if azp is None else _dev(azp, torch.int32, "azp"), _stream()))


# --------------------------------------------------------------------------
# gemv: uniform int8 / int4 weight-only mat-vec
# --------------------------------------------------------------------------

def _gemv_out(mat, vec, n: int, out):
    rows = mat.shape[0]
    if vec.numel() != n:
        raise ValueError(f"vec has {vec.numel()} elements, a row of mat {n}")
    if out is None:
        out = torch.empty(rows, dtype=torch.float16, device=mat.device)
    elif out.numel() < rows:
        raise ValueError("out is too small")
    return rows, out


def gemv_fp16(mat, vec, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """gemv_fp16 behind solve_gemv_with_params (gemv-cuda/kernels.h:64-123,
    gemv.cu:61-81): mat fp16 [rows][n], vec fp16 [n] -> fp16 [rows]."""
    n = mat.shape[1]
    rows, out = _gemv_out(mat, vec, n, out)
    with torch.cuda.device(mat.device):
        check("hq_gemv_f16", load_library().hq_gemv_f16(
            _dev(mat, torch.float16, "mat"), _dev(vec, torch.float16, "vec"),
            _dev(out, torch.float16, "out"), rows, n, _stream()))
    return out


def gemv_int8_quantized(mat, vec, scale: float, zero_point: float,
                        out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """gemv_quantized_int8 behind solve_gemv_int8_quantized_with_params
    (gemv-cuda/kernels.h:127-200, gemv.cu:38-59): mat int8 [rows][n]; scale and
    zero_point are rounded to fp16 as the reference launcher does."""
    n = mat.shape[1]
    rows, out = _gemv_out(mat, vec, n, out)
    with torch.cuda.device(mat.device):
        check("hq_gemv_int8_f16", load_library().hq_gemv_int8_f16(
            _dev(mat, torch.int8, "mat"), _dev(vec, torch.float16, "vec"),
            _dev(out, torch.float16, "out"), rows, n, float(scale), float(zero_point), _stream()))
    return out


def gemv_int4_quantized(mat, vec, scale: float, zero_point: float,
                        out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """gemv_quantized_int4 behind solve_gemv_int4_quantized_with_params
    (gemv-cuda/kernels.h:205-307, gemv.cu:15-36): mat uint8 [rows][n/2], element
    2j in the low nibble of byte j (uint4_2, kernels.h:9-32)."""
    n = 2 * mat.shape[1]
    rows, out = _gemv_out(mat, vec, n, out)
    with torch.cuda.device(mat.device):
        check("hq_gemv_int4_f16", load_library().hq_gemv_int4_f16(
            _dev(mat, torch.uint8, "mat"), _dev(vec, torch.float16, "vec"),
            _dev(out, torch.float16, "out"), rows, n, float(scale), float(zero_point), _stream()))
    return out


# --------------------------------------------------------------------------
# quantization parameters and packers
# --------------------------------------------------------------------------

def zero_point(x_min, x_max, qmin: int, qmax: int, size: int, preserve_sparsity: bool, scale,
               zero_point_out) -> None:
    """zero_point<<<...>>>(x_min, x_max, qmin, qmax, size, preserve_sparsity, scale,
    zero_point) (zeropoint-cuda/main.cu:10-18): fp32 scale and int32 zero point of
    every channel from its minimum and maximum."""
    lib = load_library()
    if min(x_min.numel(), x_max.numel(), scale.numel(), zero_point_out.numel()) < size:
        raise ValueError("a tensor is shorter than size")
    with torch.cuda.device(x_min.device):
        check("hq_zero_point", lib.hq_zero_point(
            _dev(x_min, torch.float32, "x_min"), _dev(x_max, torch.float32, "x_max"), int(qmin),
            int(qmax), int(size), int(bool(preserve_sparsity)), _dev(scale, torch.float32, "scale"),
            _dev(zero_point_out, torch.int32, "zero_point"), _stream()))


def quantize_q3(W, mat=None, scales=None, zeros=None):
    """Round-to-nearest 3-bit quantizer and packer (per-column min / max, the layout
    of quant3MatMul-cuda/kernels.h:41-87; no counterpart in the reference tree):
    W[K][N] float16 / bfloat16 / float32 -> (mat int32[K*3/32][N], scales float32[N],
    zeros float32[N]) as vecquant3matmul consumes them."""
    lib = load_library()
    code = _VLLM_DTYPE.get(W.dtype)
    if code is None:
        raise TypeError("W must be float16, bfloat16 or float32")
    if W.dim() != 2 or not W.is_cuda or not W.is_contiguous():
        raise ValueError("W must be a contiguous 2-D CUDA tensor")
    K, N = W.shape
    dev = W.device
    if mat is None:
        mat = torch.empty((K * 3 // 32, N), dtype=torch.int32, device=dev)
    if scales is None:
        scales = torch.empty(N, dtype=torch.float32, device=dev)
    if zeros is None:
        zeros = torch.empty(N, dtype=torch.float32, device=dev)
    nbytes = int(lib.hq_q3_quantize_workspace_bytes(N))
    ws = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        check("hq_q3_quantize", lib.hq_q3_quantize(
            W.data_ptr(), code, K, N, _dev(mat, torch.int32, "mat"),
            _dev(scales, torch.float32, "scales"), _dev(zeros, torch.float32, "zeros"),
            ws.data_ptr(), nbytes, _stream()))
    return mat, scales, zeros


def quantize_bcq(W, nb: int = 3, group_size: int = 128, bias: bool = True):
    """Greedy binary-coding quantizer (no counterpart in the reference tree): W[K][M]
    float16 / bfloat16 / float32 -> (bW int32[K/32][nb][M] sign planes, alpha
    float16[K/group_size][nb][M], q_bias float16[K/group_size][M] or None), the
    arrays nQWeight_fp16 takes."""
    lib = load_library()
    code = _VLLM_DTYPE.get(W.dtype)
    if code is None:
        raise TypeError("W must be float16, bfloat16 or float32")
    if W.dim() != 2 or not W.is_cuda or not W.is_contiguous():
        raise ValueError("W must be a contiguous 2-D CUDA tensor")
    K, M = W.shape
    dev = W.device
    G = K // group_size
    bW = torch.empty((K // 32, nb, M), dtype=torch.int32, device=dev)
    alpha = torch.empty((G, nb, M), dtype=torch.float16, device=dev)
    qb = torch.empty((G, M), dtype=torch.float16, device=dev) if bias else None
    with torch.cuda.device(dev):
        check("hq_lutgemm_quantize", lib.hq_lutgemm_quantize(
            W.data_ptr(), code, K, M, nb, group_size, bW.data_ptr(), alpha.data_ptr(),
            qb.data_ptr() if bias else None, _stream()))
    return bW, alpha, qb


def quantize_nf4(W, lut16, blocksize: int = 64, nibble_order: int = NF4_HIGH_NIBBLE_FIRST,
                 B=None, absmax=None):
    """Blockwise 4-bit quantizer (the inverse of dequantize_nf4; no counterpart in
    the reference tree): W float16 / bfloat16 / float32 -> (B uint8[n / 2], absmax
    float32[n / blocksize]); code = the nearest of the 16 ascending levels lut16 to
    w / absmax, a tie going to the lower level."""
    lib = load_library()
    code = _VLLM_DTYPE.get(W.dtype)
    if code is None:
        raise TypeError("W must be float16, bfloat16 or float32")
    if not W.is_cuda or not W.is_contiguous():
        raise ValueError("W must be a contiguous CUDA tensor")
    n = W.numel()
    if B is None:
        B = torch.empty(n // 2, dtype=torch.uint8, device=W.device)
    if absmax is None:
        absmax = torch.empty(n // blocksize, dtype=torch.float32, device=W.device)
    with torch.cuda.device(W.device):
        check("hq_nf4_quantize", lib.hq_nf4_quantize(
            W.data_ptr(), code, n, blocksize, _dev(lut16, torch.float32, "lut16"), nibble_order,
            _dev(B, torch.uint8, "B"), _dev(absmax, torch.float32, "absmax"), _stream()))
    return B, absmax


_MX_DTYPE = {torch.float16: 0, torch.bfloat16: 1}


def _mx_code(t) -> int:
    if t.dtype not in _MX_DTYPE:
        raise TypeError("MXFP4 takes float16 or bfloat16 tensors")
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("tensors must be contiguous CUDA tensors")
    return _MX_DTYPE[t.dtype]


def mxfp4(y, a, numel: int) -> None:
    """mxfp4<T>(y, a, numel, ...) (mxfp4-cuda/main.cu:152-176, without its timing
    loop): y = a quantized to MXFP4 and back, groups of 32, T = float16 or
    bfloat16."""
    lib = load_library()
    code = _mx_code(a)
    if y.dtype != a.dtype or min(y.numel(), a.numel()) < numel:
        raise ValueError("y and a must have the same type and numel elements")
    with torch.cuda.device(a.device):
        check("hq_mxfp4_qdq", lib.hq_mxfp4_qdq(a.data_ptr(), y.data_ptr(), int(numel), code,
                                               _stream()))


def mxfp4_quantize(a, codes=None, scales=None):
    """Packed MXFP4 of a float16 / bfloat16 tensor: (codes uint8[numel / 2], element
    2j in the low nibble; scales uint8[numel / 32], E8M0)."""
    lib = load_library()
    code = _mx_code(a)
    n = a.numel()
    if codes is None:
        codes = torch.empty(n // 2, dtype=torch.uint8, device=a.device)
    if scales is None:
        scales = torch.empty(n // 32, dtype=torch.uint8, device=a.device)
    with torch.cuda.device(a.device):
        check("hq_mxfp4_quantize", lib.hq_mxfp4_quantize(
            a.data_ptr(), _dev(codes, torch.uint8, "codes"), _dev(scales, torch.uint8, "scales"),
            n, code, _stream()))
    return codes, scales


def mxfp4_dequantize(codes, scales, dtype=torch.float16, out=None):
    """Values of a packed MXFP4 tensor in float16 or bfloat16."""
    lib = load_library()
    n = codes.numel() * 2
    if out is None:
        out = torch.empty(n, dtype=dtype, device=codes.device)
    code = _mx_code(out)
    with torch.cuda.device(codes.device):
        check("hq_mxfp4_dequantize", lib.hq_mxfp4_dequantize(
            _dev(codes, torch.uint8, "codes"), _dev(scales, torch.uint8, "scales"), out.data_ptr(),
            n, code, _stream()))
    return out


# --------------------------------------------------------------------------
# RMSNorm -> mat-vec -> gated activation, fused
# --------------------------------------------------------------------------

ACT_NONE, ACT_SWIGLU, ACT_GEGLU = 0, 1, 2


def gemv_fused(fmt: str, x, mat, rows_out: int, *, gamma=None, eps: float = 1e-5, act: int = ACT_NONE,
               scale: float = 1.0, zero_point: float = 0.0, absmax=None, lut16=None,
               blocksize: int = 64, nibble_order: int = 0, weights_resident: bool = False,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One launch for the entry of a decode-time MLP: RMSNorm of x (skipped when
    gamma is None; rmsnorm-cuda/reference.h:4-25), the weight-only mat-vec in
    format fmt ("f16", "int8", "int4", "nf4"; layouts and parameters as gemv_fp16,
    gemv_int8_quantized, gemv_int4_quantized, gemv_nf4) and, with act = ACT_SWIGLU
    or ACT_GEGLU, the gated activation of row pairs: mat then has 2 * rows_out
    rows, row 2m the value row and row 2m + 1 the gate row of output m
    (geglu-cuda/reference.h:8-16, swish-cuda/reference.h:4).  weights_resident
    (NF4): as in gemv_nf4, the weights may be fetched while the preceding kernel
    of the stream drains."""
    lib = load_library()
    n = x.numel()
    if out is None:
        out = torch.empty(rows_out, dtype=torch.float16, device=x.device)
    xp = _dev(x, torch.float16, "x")
    gp = 0 if gamma is None else _dev(gamma, torch.float16, "gamma")
    op = _dev(out, torch.float16, "out")
    with torch.cuda.device(x.device):
        if fmt == "f16":
            st = lib.hq_gemv_fused_f16(xp, gp, float(eps), _dev(mat, torch.float16, "mat"), op,
                                       rows_out, n, act, _stream())
        elif fmt == "int8":
            st = lib.hq_gemv_fused_int8_f16(xp, gp, float(eps), _dev(mat, torch.int8, "mat"), op,
                                            rows_out, n, float(scale), float(zero_point), act,
                                            _stream())
        elif fmt == "int4":
            st = lib.hq_gemv_fused_int4_f16(xp, gp, float(eps), _dev(mat, torch.uint8, "mat"), op,
                                            rows_out, n, float(scale), float(zero_point), act,
                                            _stream())
        elif fmt == "nf4":
            st = lib.hq_gemv_fused_nf4_f16(xp, gp, float(eps), _dev(mat, torch.uint8, "mat"),
                                           _dev(absmax, torch.float32, "absmax"),
                                           _dev(lut16, torch.float32, "lut16"), op, rows_out, n,
                                           blocksize, nibble_order | (2 if weights_resident else 0),
                                           act, _stream())
        else:
            raise ValueError(f"unknown format {fmt!r}")
        check("hq_gemv_fused_" + fmt, st)
    return out


# --------------------------------------------------------------------------
# lut-gemm
# --------------------------------------------------------------------------

class nQWeight_fp16:
    """Mirror of class nQWeight_fp16 (lut-gemm-cuda/nQWeight_fp16.h:22-45,
    nQWeight_fp16.cu:22-53): holds the bit-plane weights, fp16 alphas and the
    optional fp16 q_bias on the device.  `parsing` takes the same host-side
    arrays (uint32 bit planes [K/32][nb][M], fp32 alpha [groups][nb][M], fp32
    q_bias [groups][M] or None) and converts alpha / q_bias to fp16."""

    def __init__(self, bW=None, A=None, row: int = 0, col: int = 0, num_bits: int = 0,
                 is_row_wise_quantize: bool = False, num_alpha_groups: int = 1, q_bias=None,
                 device="cuda"):
        self.bWeight = self.alpha = self.q_bias = None
        self.num_groups = self.group_size = self.mSize = self.kSize = self.nb = 0
        self.is_row_wise_quantize = False
        self._ws = None
        if bW is not None:
            self.parsing(bW, A, row, col, num_bits, is_row_wise_quantize, num_alpha_groups,
                         q_bias, device)

    def parsing(self, bW, A, row: int, col: int, num_bits: int, is_row_wise_quantize: bool,
                num_alpha_groups: int = 1, q_bias=None, device="cuda") -> None:
        self.num_groups = num_alpha_groups
        self.nb = num_bits
        self.is_row_wise_quantize = is_row_wise_quantize
        self.mSize, self.kSize = (row, col) if is_row_wise_quantize else (col, row)
        # the reference computes group_size before kSize is set
        # (nQWeight_fp16.cu:25); its launcher uses kSize/num_groups (mv_fp16.h:235)
        self.group_size = self.kSize // num_alpha_groups
        dev = torch.device(device)
        bW_t = torch.as_tensor(bW)
        if bW_t.dtype == torch.uint32:
            bW_t = bW_t.view(torch.int32)
        self.bWeight = bW_t.to(torch.int32).reshape(-1).contiguous().to(dev)
        self.alpha = torch.as_tensor(A, dtype=torch.float32).reshape(-1).to(torch.float16).to(dev)
        self.q_bias = None if q_bias is None else \
            torch.as_tensor(q_bias, dtype=torch.float32).reshape(-1).to(torch.float16).to(dev)
        need_w = self.kSize * self.mSize * self.nb // 32
        if self.bWeight.numel() != need_w:
            raise ValueError("bW has the wrong number of words")
        if self.alpha.numel() != self.num_groups * self.mSize * self.nb:
            raise ValueError("alpha has the wrong number of elements")

    def workspace(self) -> torch.Tensor:
        """Zero-initialised fp32 scratch the kernel accumulates K tiles into; it
        is left zero by every call."""
        if self._ws is None:
            nbytes = load_library().hq_lutgemm_workspace_bytes(self.mSize)
            self._ws = torch.zeros(nbytes, dtype=torch.uint8, device=self.bWeight.device)
        return self._ws


def matmul(output, input, nqW: nQWeight_fp16, m: int = 1, algo: int = 0) -> None:
    """matmul(void* output, void* input, nQWeight_fp16& nqW, int m, int algo)
    (lut-gemm-cuda/kernels.cu:27-31): overwrites output[0:mSize] with the
    mat-vec of one input row (like the reference, only batch 1 is computed)."""
    lib = load_library()
    ws = nqW.workspace()
    args = (
        _dev(output, torch.float16, "output"), _dev(input, torch.float16, "input"),
        nqW.bWeight.data_ptr(), nqW.alpha.data_ptr(),
        0 if nqW.q_bias is None else nqW.q_bias.data_ptr(),
        nqW.mSize, nqW.kSize, nqW.nb, nqW.group_size,
        ws.data_ptr(), ws.numel())
    with torch.cuda.device(nqW.bWeight.device):
        check("hq_lutgemm_nqmv", lib.hq_lutgemm_nqmv(*args, _stream()))


# --------------------------------------------------------------------------
# quantAQLM
# --------------------------------------------------------------------------

def code1x16_matvec(A, B, C_out, codebook, prob_m: int, prob_k: int,
                    codebook_a_sizes: Sequence[int], codebook_stride: int,
                    scales: Optional[torch.Tensor] = None) -> None:
    """code1x16_matvec (quantAQLM-cuda/main.cu:113-141).  A = codes (int16 or
    uint16, [prob_m][prob_k/8]), B = input half[prob_k], C_out = half[prob_m]
    (overwritten), codebook half[..][65536][8]; `scales` is an extension."""
    lib = load_library()
    if A.dtype not in (torch.int16, torch.uint16):
        raise TypeError("A: expected int16/uint16 codes")
    sizes = (C.c_int * 4)(*[int(v) for v in codebook_a_sizes])
    args = (
        _dev(A, A.dtype, "A"), _dev(B, torch.float16, "B"),
        _dev(C_out, torch.float16, "C"), _dev(codebook, torch.float16, "codebook"),
        prob_m, prob_k, sizes, codebook_stride,
        0 if scales is None else _dev(scales, torch.float16, "scales"))
    with torch.cuda.device(A.device):
        check("hq_aqlm_1x16_matvec", lib.hq_aqlm_1x16_matvec(*args, _stream()))


def code2x8_matvec(A, B, C_out, codebooks, prob_m: int, prob_k: int,
                   scales: Optional[torch.Tensor] = None) -> None:
    """AQLM 2x8 mat-vec (no counterpart in the reference tree).  A = uint8 codes
    [prob_m][prob_k/8][2], codebooks half[2][256][8]."""
    lib = load_library()
    args = (
        _dev(A, torch.uint8, "A"), _dev(B, torch.float16, "B"),
        _dev(C_out, torch.float16, "C"), _dev(codebooks, torch.float16, "codebooks"),
        prob_m, prob_k,
        0 if scales is None else _dev(scales, torch.float16, "scales"))
    with torch.cuda.device(A.device):
        check("hq_aqlm_2x8_matvec", lib.hq_aqlm_2x8_matvec(*args, _stream()))


# --------------------------------------------------------------------------
# batched dequant-GEMM (tensor cores)
# --------------------------------------------------------------------------

_qgemm_ws = {}


def _qgemm_workspace(lib, device, Mb: int, N: int):
    """Zero-initialised split-K scratch, one per (device, stream, Mb, N): calls on
    different streams may overlap on the GPU and must not share the fp32 partial
    sums and tile counters."""
    key = (device, _stream(), Mb, N)
    ws = _qgemm_ws.get(key)
    if ws is None:
        ws = torch.zeros(lib.hq_qgemm_workspace_bytes(Mb, N), dtype=torch.uint8, device=device)
        _qgemm_ws[key] = ws
    return ws.data_ptr(), ws.numel()


def qgemm_reset_workspaces() -> None:
    """Re-zero every cached split-K scratch on its device.  Call this after a
    batched product reported status 1 (a bounded in-kernel wait ran out): such a
    call may leave partial sums and tile counters behind, and the kernels rely on
    finding the scratch zero."""
    for ws in _qgemm_ws.values():
        ws.zero_()


def qgemm_q3(X, mat, scales, zeros, N: int, K: int, group_size: int = 128,
             out: Optional[torch.Tensor] = None,
             status: Optional[torch.Tensor] = None, split_k: bool = True,
             peers=None) -> Optional[torch.Tensor]:
    """Y[Mb][N] = X[Mb][K] @ dequant(mat) for the GPTQ 3-bit layout with per-group
    fp16 scales / zeros [K/group_size][N] (no counterpart in the reference tree).
    `status` (int32[1], optional) receives 1 if a bounded in-kernel wait ran out;
    call qgemm_reset_workspaces() before the next product in that case.
    With split_k a zero-initialised scratch matrix is kept per (device, stream, Mb, N).
    peers = (pointer_table, offset_elements, world): store every finished tile into
    the output slice of every GPU of the node instead of `out` (hq_qgemm_q3_f16_peers);
    returns None in that form."""
    lib = load_library()
    Mb = X.shape[0]
    head = (
        _dev(X, torch.float16, "X"), _dev(mat, torch.int32, "mat"),
        _dev(scales, torch.float16, "scales"), _dev(zeros, torch.float16, "zeros"))
    ws_ptr, ws_bytes = _qgemm_workspace(lib, X.device, Mb, N) if split_k else (0, 0)
    st = 0 if status is None else _dev(status, torch.int32, "status")
    with torch.cuda.device(X.device):
        if peers is not None:
            table, offset, world = peers
            check("hq_qgemm_q3_f16_peers", lib.hq_qgemm_q3_f16_peers(
                *head, int(table), int(offset), int(world), Mb, N, K, group_size, ws_ptr, ws_bytes,
                st, _stream()))
            return None
        if out is None:
            out = torch.empty((Mb, N), dtype=torch.float16, device=X.device)
        check("hq_qgemm_q3_f16", lib.hq_qgemm_q3_f16(
            *head, _dev(out, torch.float16, "out"), Mb, N, K, group_size, ws_ptr, ws_bytes, st,
            _stream()))
    return out


def qgemm_nf4(X, B, absmax, lut16, N: int, K: int, blocksize: int = 64, nibble_order: int = 0,
              out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
              split_k: bool = True, peers=None) -> Optional[torch.Tensor]:
    """Y[Mb][N] = X[Mb][K] @ W with W[k][n] the NF4 weight that dequantize_nf4
    gives for element n*K + k of B (uint8[N*K/2], absmax per `blocksize`
    elements); same conventions as gemv_nf4, same workspace, status and `peers`
    rules as qgemm_q3 (no counterpart in the reference tree)."""
    lib = load_library()
    Mb = X.shape[0]
    head = (
        _dev(X, torch.float16, "X"), _dev(B, torch.uint8, "B"),
        _dev(absmax, torch.float32, "absmax"), _dev(lut16, torch.float32, "lut16"))
    ws_ptr, ws_bytes = _qgemm_workspace(lib, X.device, Mb, N) if split_k else (0, 0)
    st = 0 if status is None else _dev(status, torch.int32, "status")
    with torch.cuda.device(X.device):
        if peers is not None:
            table, offset, world = peers
            check("hq_qgemm_nf4_f16_peers", lib.hq_qgemm_nf4_f16_peers(
                *head, int(table), int(offset), int(world), Mb, N, K, blocksize, nibble_order,
                ws_ptr, ws_bytes, st, _stream()))
            return None
        if out is None:
            out = torch.empty((Mb, N), dtype=torch.float16, device=X.device)
        check("hq_qgemm_nf4_f16", lib.hq_qgemm_nf4_f16(
            *head, _dev(out, torch.float16, "out"), Mb, N, K, blocksize, nibble_order, ws_ptr,
            ws_bytes, st, _stream()))
    return out
