"""hecbench_b200: B200 (sm_100a) kernels for HeCBench's weight-only quantized
matrix-vector family, behind each benchmark's own launcher signature.

The compute lives in libhq.so (hand-written CUDA, C ABI declared in
include/hq.h).  This package is the thin Python host layer over it: it mirrors
the reference launchers (`vecquant3matmul`, `vecquant3matmul_faster`,
`kQuantize`, `matmul` + `nQWeight_fp16`, `code1x16_matvec`,
`static_scaled_int8_quant`, `dynamic_scaled_int8_quant`, the `gemv` int8 / int4
kernels) on torch CUDA
tensors and adds the pieces the reference names but does not contain (NF4
dequantize / GEMV, AQLM 2x8).  There is no CPU path: importing works without a
GPU, but every compute call needs the built library and CUDA tensors.
"""
from ._lib import HqError, lib_path, load_library  # noqa: F401
from .api import (  # noqa: F401
    NF4_HIGH_NIBBLE_FIRST,
    NF4_WEIGHTS_RESIDENT,
    NF4_LOW_NIBBLE_FIRST,
    code1x16_matvec,
    code2x8_matvec,
    dequantize_nf4,
    dynamic_scaled_int8_quant,
    ACT_GEGLU,
    ACT_NONE,
    ACT_SWIGLU,
    gemv_fp16,
    gemv_fused,
    mxfp4,
    mxfp4_dequantize,
    mxfp4_quantize,
    quantize_bcq,
    quantize_nf4,
    quantize_q3,
    zero_point,
    gemv_int4_quantized,
    gemv_int8_quantized,
    gemv_nf4,
    kQuantize,
    matmul,
    nQWeight_fp16,
    qgemm_q3,
    qgemm_nf4,
    qgemm_reset_workspaces,
    static_scaled_int8_quant,
    vecquant3_dequant,
    vecquant3matmul,
    vecquant3matmul_faster,
)

__all__ = [
    "HqError", "lib_path", "load_library",
    "vecquant3matmul", "vecquant3matmul_faster", "vecquant3_dequant",
    "kQuantize", "dequantize_nf4", "gemv_nf4",
    "nQWeight_fp16", "matmul", "qgemm_q3", "qgemm_nf4", "qgemm_reset_workspaces", "code1x16_matvec", "code2x8_matvec",
    "static_scaled_int8_quant", "dynamic_scaled_int8_quant",
    "gemv_fp16", "gemv_int8_quantized", "gemv_int4_quantized",
    "gemv_fused", "ACT_NONE", "ACT_SWIGLU", "ACT_GEGLU",
    "zero_point", "mxfp4", "mxfp4_quantize", "mxfp4_dequantize", "quantize_nf4", "quantize_bcq", "quantize_q3",
    "NF4_HIGH_NIBBLE_FIRST", "NF4_LOW_NIBBLE_FIRST", "NF4_WEIGHTS_RESIDENT",
]
