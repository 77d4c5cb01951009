"""ctypes binding of libhq.so (include/hq.h).  Fails loudly when the library is
missing: there is no fallback implementation."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

_PKG = Path(__file__).resolve().parent
# HQ_LIBRARY selects another build of the same library (e.g. libhq_checked.so)
_LIB_PATH = Path(os.environ["HQ_LIBRARY"]) if os.environ.get("HQ_LIBRARY") else _PKG / "libhq.so"
_lib = None

c_void_p, c_int, c_size_t = C.c_void_p, C.c_int, C.c_size_t

# name -> (restype, argtypes); must list every symbol include/hq.h declares.
SIGNATURES = {
    "hq_version": (c_int, []),
    "hq_status_string": (C.c_char_p, [c_int]),
    "hq_last_cuda_error": (c_int, []),
    "hq_bounds_check_report": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int]),
    "hq_q3_gemv_f32": (c_int, [c_void_p] * 5 + [c_int, c_int, c_void_p]),
    "hq_q3_gemv_f16in": (c_int, [c_void_p] * 5 + [c_int, c_int, c_void_p]),
    "hq_q3_dequant_f32": (c_int, [c_void_p] * 4 + [c_int, c_int, c_void_p]),
    "hq_q3_dequant_f16": (c_int, [c_void_p] * 4 + [c_int, c_int, c_void_p]),
    "hq_bnb_quantize_u8": (c_int, [c_void_p] * 3 + [c_size_t, c_void_p]),
    "hq_nf4_dequant_f16": (c_int, [c_void_p] * 4 + [c_size_t, c_int, c_int, c_void_p]),
    "hq_nf4_gemv_f16": (c_int, [c_void_p] * 5 + [c_int, c_int, c_int, c_int, c_void_p]),
    "hq_nf4_gemv_f16_ll": (c_int, [c_void_p, c_void_p, C.c_longlong, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_int, c_int, c_int, c_int, c_void_p, C.c_longlong,
                                   c_void_p, c_int, c_int, C.c_uint, c_void_p, c_void_p]),
    "hq_ll_unpack": (c_int, [c_void_p, C.c_longlong, c_void_p, c_void_p, C.c_uint, c_void_p,
                             c_void_p]),
    "hq_gather_publish": (c_int, [c_void_p, C.c_longlong, c_int, c_void_p, c_void_p, c_int, c_int,
                                  C.c_uint, c_void_p, c_void_p]),
    "hq_gather_wait": (c_int, [c_void_p, c_void_p, c_int, C.c_uint, c_void_p, c_void_p]),
    "hq_shard_layout": (c_int, [c_int, c_int, C.c_longlong, c_int, c_int, c_int, c_void_p, c_void_p,
                                c_void_p]),
    "hq_shard_create": (c_int, [c_void_p, c_void_p, c_int, C.c_longlong, c_int, c_int, c_int]),
    "hq_shard_destroy": (None, [c_void_p]),
    "hq_shard_stream": (c_void_p, [c_void_p, c_int]),
    "hq_shard_nf4_gemv": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, C.c_longlong, c_void_p,
                                  c_void_p, c_void_p, c_int, c_int, c_int]),
    "hq_shard_unpack": (c_int, [c_void_p, c_int, c_int, c_void_p]),
    "hq_shard_local_slice": (c_void_p, [c_void_p, c_int, c_int]),
    "hq_shard_publish": (c_int, [c_void_p, c_int, c_int]),
    "hq_shard_allgather_nccl": (c_int, [c_void_p, c_int]),
    "hq_shard_gathered": (c_void_p, [c_void_p, c_int, c_int]),
    "hq_shard_status": (c_int, [c_void_p, c_int, c_void_p]),
    "hq_lutgemm_workspace_bytes": (c_size_t, [c_int]),
    "hq_lutgemm_nqmv": (c_int, [c_void_p] * 5 + [c_int] * 4 + [c_void_p, c_size_t, c_void_p]),
    "hq_lutgemm_nqmv_noalloc": (c_int, [c_void_p] * 5 + [c_int] * 4 + [c_void_p]),
    "hq_aqlm_1x16_matvec": (c_int, [c_void_p] * 4 + [c_int, c_int, C.POINTER(c_int), c_int,
                                                     c_void_p, c_void_p]),
    "hq_qgemm_workspace_bytes": (c_size_t, [c_int, c_int]),
    "hq_qgemm_q3_f16": (c_int, [c_void_p] * 5 + [c_int] * 4 + [c_void_p, c_size_t, c_void_p,
                                                               c_void_p]),
    "hq_qgemm_nf4_f16": (c_int, [c_void_p] * 5 + [c_int] * 5 + [c_void_p, c_size_t, c_void_p,
                                                                c_void_p]),
    "hq_qgemm_q3_f16_peers": (c_int, [c_void_p] * 5 + [C.c_longlong] + [c_int] * 5 +
                              [c_void_p, c_size_t, c_void_p, c_void_p]),
    "hq_qgemm_nf4_f16_peers": (c_int, [c_void_p] * 5 + [C.c_longlong] + [c_int] * 6 +
                               [c_void_p, c_size_t, c_void_p, c_void_p]),
    "hq_vllm_static_scaled_int8_quant": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, C.c_float,
                                                 C.c_int32, c_void_p]),
    "hq_vllm_dynamic_scaled_int8_quant": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int,
                                                  c_void_p, c_void_p, c_void_p]),
    "hq_gemv_f16": (c_int, [c_void_p] * 3 + [c_int, c_int, c_void_p]),
    "hq_gemv_int8_f16": (c_int, [c_void_p] * 3 + [c_int, c_int, C.c_float, C.c_float, c_void_p]),
    "hq_gemv_int4_f16": (c_int, [c_void_p] * 3 + [c_int, c_int, C.c_float, C.c_float, c_void_p]),
    "hq_gemv_fused_f16": (c_int, [c_void_p, c_void_p, C.c_float, c_void_p, c_void_p] +
                          [c_int] * 3 + [c_void_p]),
    "hq_gemv_fused_int8_f16": (c_int, [c_void_p, c_void_p, C.c_float, c_void_p, c_void_p, c_int,
                                       c_int, C.c_float, C.c_float, c_int, c_void_p]),
    "hq_gemv_fused_int4_f16": (c_int, [c_void_p, c_void_p, C.c_float, c_void_p, c_void_p, c_int,
                                       c_int, C.c_float, C.c_float, c_int, c_void_p]),
    "hq_gemv_fused_nf4_f16": (c_int, [c_void_p, c_void_p, C.c_float] + [c_void_p] * 4 +
                              [c_int] * 5 + [c_void_p]),
    "hq_zero_point": (c_int, [c_void_p, c_void_p, C.c_int32, C.c_int32, c_int, c_int, c_void_p,
                              c_void_p, c_void_p]),
    "hq_q3_quantize_workspace_bytes": (c_size_t, [c_int]),
    "hq_q3_quantize": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_size_t, c_void_p]),
    "hq_lutgemm_quantize": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                    c_void_p, c_void_p, c_void_p]),
    "hq_nf4_quantize": (c_int, [c_void_p, c_int, c_size_t, c_int, c_void_p, c_int, c_void_p,
                                c_void_p, c_void_p]),
    "hq_mxfp4_qdq": (c_int, [c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "hq_mxfp4_quantize": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "hq_mxfp4_dequantize": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "hq_aqlm_2x8_matvec": (c_int, [c_void_p] * 4 + [c_int, c_int, c_void_p, c_void_p]),
}


class HqError(RuntimeError):
    """A libhq entry point returned a negative status."""

    def __init__(self, fn: str, status: int, detail: str):
        super().__init__(f"{fn} failed: {detail} (status {status})")
        self.status = status


def lib_path() -> Path:
    return _LIB_PATH


def load_checked_library():
    """A separate handle on libhq_checked.so (the -DHQ_BOUNDS_CHECK build), with
    the same prototypes; None when it was not built."""
    path = _PKG / "libhq_checked.so"
    if not path.exists():
        return None
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


def load_library():
    """Load libhq.so once and attach the prototypes of include/hq.h."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing - build it with `python -m hecbench_b200.build` "
            "(nvcc, sm_100a).  There is no CPU or PyTorch fallback.")
    lib = C.CDLL(str(_LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(fn: str, status: int) -> None:
    if status != 0:
        lib = load_library()
        detail = lib.hq_status_string(status).decode()
        if status == -4:
            detail += f" (cudaError {lib.hq_last_cuda_error()})"
        raise HqError(fn, status, detail)
