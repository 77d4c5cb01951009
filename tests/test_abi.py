"""CPU checks of the drop-in boundary: libhq.so loads and exports exactly the
symbols include/hq.h declares (no compute call is made without a GPU)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "hq.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_family():
    names = declared_symbols()
    for needed in ["hq_q3_gemv_f32", "hq_q3_gemv_f16in", "hq_bnb_quantize_u8",
                   "hq_nf4_dequant_f16", "hq_nf4_gemv_f16", "hq_lutgemm_nqmv",
                   "hq_aqlm_1x16_matvec", "hq_aqlm_2x8_matvec"]:
        assert needed in names


def test_library_exports_every_declared_symbol(hq):
    lib = ctypes.CDLL(str(hq.lib_path()))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in hq.h but not exported"


def test_python_binding_covers_every_declared_symbol(hq):
    from hecbench_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_version_and_status_strings(hq):
    lib = hq.load_library()
    assert lib.hq_version() >= 100
    assert lib.hq_status_string(0) == b"ok"
    assert lib.hq_status_string(-1) == b"bad shape"
    assert lib.hq_lutgemm_workspace_bytes(12288) >= 12288 * 4 + 4
    assert lib.hq_lutgemm_workspace_bytes(0) == 0


def test_argument_errors_need_no_gpu(hq):
    """Shape / null checks run before any CUDA call."""
    lib = hq.load_library()
    assert lib.hq_q3_gemv_f32(None, None, None, None, None, 24, 256, None) == -2
    assert lib.hq_q3_gemv_f32(16, 16, 16, 16, 16, 25, 256, None) == -1
    assert lib.hq_q3_gemv_f32(16, 16, 16, 16, 16, 24, 254, None) == -1
    assert lib.hq_q3_gemv_f32(16, 8, 16, 16, 16, 24, 256, None) == -3
    assert lib.hq_nf4_gemv_f16(16, 16, 16, 16, 16, 8, 100, 64, 0, None) == -1
    assert lib.hq_nf4_dequant_f16(16, 16, 16, 16, 64, 48, 0, None) == -1
    assert lib.hq_lutgemm_nqmv(16, 16, 16, 16, None, 256, 128, 3, 128, None, 0, None) == -5
    assert lib.hq_lutgemm_nqmv(16, 16, 16, 16, None, 256, 128, 9, 128, 16, 1 << 20, None) == -1
    assert lib.hq_aqlm_1x16_matvec(16, 16, 16, 16, 64, 100, (ctypes.c_int * 4)(64, 64, 64, 64),
                                   0, None, None) == -1


def test_gather_and_noalloc_argument_errors_need_no_gpu(hq):
    lib = hq.load_library()
    p = 64
    # packet GEMV: exactly one input form, exactly one output form, sync words, rank < world
    assert lib.hq_nf4_gemv_f16_ll(p, p, 1, p, p, p, p, 32, 64, 64, 0, 0, 0, p, 1, 0, 0, 0,
                                  None) == -2
    assert lib.hq_nf4_gemv_f16_ll(p, 0, 1, p, p, p, p, 32, 64, 64, 0, p, 0, p, 1, 0, 0, 0,
                                  None) == -2
    assert lib.hq_nf4_gemv_f16_ll(p, 0, 1, p, p, p, p, 32, 64, 64, 0, 0, 0, 0, 1, 0, 0, 0,
                                  None) == -2
    assert lib.hq_nf4_gemv_f16_ll(p, 0, 1, p, p, p, p, 32, 64, 64, 0, 0, 0, p, 2, 2, 0, 0,
                                  None) == -1
    assert lib.hq_gather_wait(p, p, 0, 0, 0, None) == -1
    assert lib.hq_gather_publish(p, 0, -1, p, p, 1, 0, 0, 0, None) == -1
    assert lib.hq_gather_publish(p, 0, 64, p, p, 2, 2, 0, 0, None) == -1
    # batched product with the gather in its epilogue: pointer table, 1 <= world <= 32
    assert lib.hq_qgemm_q3_f16_peers(p, p, p, p, 0, 0, 2, 64, 128, 128, 128, None, 0, None,
                                     None) == -2
    assert lib.hq_qgemm_q3_f16_peers(p, p, p, p, p, 0, 0, 64, 128, 128, 128, None, 0, None,
                                     None) == -1
    assert lib.hq_qgemm_nf4_f16_peers(p, p, p, p, p, -8, 2, 64, 128, 128, 64, 0, None, 0, None,
                                      None) == -1
    assert lib.hq_qgemm_nf4_f16_peers(p, p, p, p, 0, 0, 2, 64, 128, 128, 64, 0, None, 0, None,
                                      None) == -2
    assert lib.hq_ll_unpack(p, 0, p, 0, 0, 0, None) == -1
    # allocation-free LUT-GEMM: every argument rule is checked before the shared
    # scratch array is looked up or touched (so no CUDA call is made here)
    assert lib.hq_lutgemm_nqmv_noalloc(None, p, p, p, None, 256, 128, 3, 128, None) == -2
    assert lib.hq_lutgemm_nqmv_noalloc(p, p, p, p, None, 258, 128, 3, 128, None) == -1
    assert lib.hq_lutgemm_nqmv_noalloc(p, p, p, p, None, 256, 192, 3, 96, None) == -6
    assert lib.hq_lutgemm_nqmv_noalloc(p, p, 8, p, None, 256, 128, 3, 128, None) == -3
    assert lib.hq_lutgemm_nqmv_noalloc(p, p, p, p, None, 65536 + 4, 128, 3, 128, None) == -7


def test_gemv_uniform_argument_errors_need_no_gpu(hq):
    lib = hq.load_library()
    p = 64
    assert lib.hq_gemv_int8_f16(None, p, p, 16, 16, 1.0, 0.0, None) == -2
    assert lib.hq_gemv_int4_f16(p, None, p, 16, 32, 1.0, 0.0, None) == -2
    assert lib.hq_gemv_f16(p, p, None, 16, 8, None) == -2
    assert lib.hq_gemv_int8_f16(p, p, p, 16, 24, 1.0, 0.0, None) == -1   # n % 16
    assert lib.hq_gemv_int4_f16(p, p, p, 16, 16, 1.0, 0.0, None) == -1   # n % 32
    assert lib.hq_gemv_f16(p, p, p, 0, 8, None) == -1
    assert lib.hq_gemv_int8_f16(p + 8, p, p, 16, 16, 1.0, 0.0, None) == -3


def test_shard_layout_arithmetic_and_argument_errors(hq):
    """Index arithmetic of the sharding context (no CUDA call) and the argument
    checks of hq_shard_create that come before any CUDA call."""
    lib = hq.load_library()
    pk, sl, per = (ctypes.c_longlong() for _ in range(3))
    ref = ctypes.byref
    # mat-vec: 4 ranks x 1376 features, 3 slots
    assert lib.hq_shard_layout(4, 1, 1376, 3, 2, 1, ref(pk), ref(sl), ref(per)) == 0
    assert per.value == 4 * 1376
    assert pk.value == 1 * 4 * 1376 + 2 * 1376
    assert sl.value == pk.value
    # batched: [world][rows][n_local] per slot
    assert lib.hq_shard_layout(8, 64, 3584, 2, 5, 1, ref(pk), ref(sl), ref(per)) == 0
    assert per.value == 8 * 64 * 3584
    assert sl.value == per.value + 5 * 64 * 3584
    for r in range(8):  # slices tile a slot exactly, in rank order
        lib.hq_shard_layout(8, 64, 3584, 2, r, 0, None, ref(sl), None)
        assert sl.value == r * 64 * 3584
    assert lib.hq_shard_layout(0, 1, 8, 2, 0, 0, None, None, None) == -1
    assert lib.hq_shard_layout(4, 1, 8, 2, 4, 0, None, None, None) == -1
    assert lib.hq_shard_layout(4, 1, 8, 2, 0, 2, None, None, None) == -1
    ctx = ctypes.c_void_p()
    devs = (ctypes.c_int * 2)(0, 1)
    assert lib.hq_shard_create(None, devs, 2, 128, 1, 2, 0) == -2
    assert lib.hq_shard_create(ref(ctx), devs, 0, 128, 1, 2, 0) == -1
    assert lib.hq_shard_create(ref(ctx), devs, 2, 128, 1, 1, 0) == -1  # fewer than two slots
    assert lib.hq_shard_publish(None, 0, 0) == -1
    assert lib.hq_shard_stream(None, 0) is None
    lib.hq_shard_destroy(None)


def test_python_layer_rejects_cpu_tensors(hq):
    import torch
    t = torch.zeros(256)
    with pytest.raises(TypeError):
        hq.vecquant3matmul(t, t.int(), t, t, t, 24, 256)


def test_fused_and_packer_argument_errors_need_no_gpu(hq):
    """The fused mat-vec entries and the packers reject bad arguments before any
    CUDA call: fake (aligned, never dereferenced) pointers are enough."""
    lib = hq.load_library()
    p = 64
    # fused RMSNorm -> mat-vec -> gated activation
    assert lib.hq_gemv_fused_f16(p, None, 1e-5, None, p, 8, 64, 0, None) == -2
    assert lib.hq_gemv_fused_int8_f16(p, None, 1e-5, p, p, 8, 64, 1.0, 0.0, 3, None) == -1
    assert lib.hq_gemv_fused_int4_f16(p, None, 1e-5, p, p, 8, 48, 1.0, 0.0, 0, None) == -1
    assert lib.hq_gemv_fused_int4_f16(p, p + 2, 1e-5, p, p, 8, 64, 1.0, 0.0, 0, None) == -3
    assert lib.hq_gemv_fused_nf4_f16(p, None, 1e-5, p, None, p, p, 8, 64, 64, 0, 0, None) == -2
    assert lib.hq_gemv_fused_nf4_f16(p, None, 1e-5, p, p, p, p, 8, 64, 64, 0, 5, None) == -1
    assert lib.hq_gemv_fused_nf4_f16(p, None, 1e-5, p, p, p, p, 0, 64, 64, 0, 0, None) == -1
    # zero point
    assert lib.hq_zero_point(p, p, 5, 5, 8, 1, p, p, None) == -1
    assert lib.hq_zero_point(None, p, -127, 127, 8, 1, p, p, None) == -2
    assert lib.hq_zero_point(None, None, -127, 127, 0, 1, None, None, None) == 0
    # MXFP4
    assert lib.hq_mxfp4_qdq(p, p, 48, 0, None) == -1
    assert lib.hq_mxfp4_qdq(p, p, 64, 2, None) == -6
    assert lib.hq_mxfp4_qdq(None, p, 64, 0, None) == -2
    assert lib.hq_mxfp4_qdq(p + 2, p, 32, 0, None) == -3
    assert lib.hq_mxfp4_quantize(p, p, None, 64, 0, None) == -2
    assert lib.hq_mxfp4_dequantize(p, None, p, 64, 1, None) == -2
    assert lib.hq_mxfp4_qdq(None, None, 0, 1, None) == 0
    # quantizers
    assert lib.hq_nf4_quantize(p, 0, 128, 48, p, 0, p, p, None) == -1
    assert lib.hq_nf4_quantize(p, 0, 100, 64, p, 0, p, p, None) == -1
    assert lib.hq_nf4_quantize(p, 3, 128, 64, p, 0, p, p, None) == -6
    assert lib.hq_nf4_quantize(p, 0, 128, 64, None, 0, p, p, None) == -2
    assert lib.hq_q3_quantize_workspace_bytes(16) == 128
    assert lib.hq_q3_quantize(p, 0, 48, 16, p, p, p, p, 128, None) == -1
    assert lib.hq_q3_quantize(p, 0, 64, 12, p, p, p, p, 128, None) == -1
    assert lib.hq_q3_quantize(p, 0, 64, 16, p, p, p, p, 64, None) == -5
    assert lib.hq_q3_quantize(p, 7, 64, 16, p, p, p, p, 128, None) == -6
    assert lib.hq_lutgemm_quantize(p, 0, 128, 16, 3, 48, p, p, None, None) == -1
    assert lib.hq_lutgemm_quantize(p, 0, 128, 16, 9, 128, p, p, None, None) == -1
    assert lib.hq_lutgemm_quantize(p, 0, 1024, 16, 3, 1024, p, p, None, None) == -6
    assert lib.hq_lutgemm_quantize(p, 0, 128, 16, 3, 128, None, p, None, None) == -2
