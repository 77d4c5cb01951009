"""CPU tests that pin the oracle: against the reference's own known-answer
vector (quant3MatMul), against golden vectors produced by the reference's own
CPU build (quantBnB), and against independent numpy restatements."""
from pathlib import Path

import numpy as np
import pytest

from hecbench_b200 import synth

GOLDEN = Path(__file__).resolve().parent / "golden"


# ---------- fp16 helpers ----------

def test_half_conversion_matches_numpy(oracle):
    import ctypes as C
    rng = np.random.default_rng(1)
    f = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 10,
        rng.standard_normal(20000).astype(np.float32) * 1e-5,
        np.array([0, -0.0, 65504, 65520, 65519.99, 1e-8, 6e-8, 5.96e-8, 2.98e-8, 2.9802322e-8,
                  np.inf, -np.inf, 1e10, 6.1035156e-05, 6.1e-05], dtype=np.float32)])
    out = np.empty(f.size, dtype=np.uint16)
    oracle.lib().orc_f32_to_f16(f.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p),
                                C.c_size_t(f.size))
    assert np.array_equal(out, f.astype(np.float16).view(np.uint16))
    allh = np.arange(65536, dtype=np.uint16)
    back = np.empty(65536, dtype=np.float32)
    oracle.lib().orc_f16_to_f32(allh.ctypes.data_as(C.c_void_p), back.ctypes.data_as(C.c_void_p),
                                C.c_size_t(65536))
    want = allh.view(np.float16).astype(np.float32)
    assert np.array_equal(back.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])


# ---------- quant3MatMul ----------

def test_q3_reference_known_answer(oracle):
    """quant3MatMul-cuda/main.cu:28-53,84-105: all codes 1 (pattern p1, p1<<1,
    p1<<2), vec 1, scale -1, zero 0 => every output is exactly -K; checked at a
    reduced K (multiple of 256) and at the driver's own K = 49152 on a few
    columns."""
    p1 = 0b01001001001001001001001001001001
    for K, width in [(1024, 256), (49152, 4)]:
        height = K // 32 * 3
        mat = np.empty((height, width), dtype=np.uint32)
        mat[0::3] = p1
        mat[1::3] = (p1 << 1) & 0xFFFFFFFF
        mat[2::3] = (p1 << 2) & 0xFFFFFFFF
        mat = mat.view(np.int32)
        assert np.all(oracle.q3_unpack(mat) == 1)
        vec = np.ones(K, dtype=np.float32)
        sc = -np.ones(width, dtype=np.float32)
        z = np.zeros(width, dtype=np.float32)
        zero = np.zeros(width, dtype=np.float32)
        assert np.all(oracle.q3_gemv_f32(vec, mat, zero, sc, z) == -float(K))
        assert np.all(oracle.q3_gemv_f16in(vec.astype(np.float16), mat, zero, sc, z) == -float(K))
        assert np.all(oracle.q3_gemv_f64(vec, mat, sc, z) == -float(K))


def test_q3_pack_unpack_and_bit_order(oracle):
    K, width = 256, 8
    codes = synth.q3_case(K, width, seed=3)[1]
    mat = oracle.q3_pack(codes)
    assert np.array_equal(oracle.q3_unpack(mat), codes)
    assert np.array_equal(synth.q3_pack(codes), mat)
    # independent restatement: 96-bit little-endian stream per (group, column)
    m = mat.view(np.uint32).astype(object)
    for r in range(K // 32):
        for c in range(width):
            B = int(m[3 * r, c]) | (int(m[3 * r + 1, c]) << 32) | (int(m[3 * r + 2, c]) << 64)
            got = [(B >> (3 * j)) & 7 for j in range(32)]
            assert got == list(codes[32 * r:32 * r + 32, c])
    # the extraction of the fp16 kernel: 6 bits at a time, low 3 bits = even k
    for r in range(K // 32):
        B = int(m[3 * r, 0]) | (int(m[3 * r + 1, 0]) << 32) | (int(m[3 * r + 2, 0]) << 64)
        for i in range(16):
            pair = (B >> (6 * i)) & 63
            assert pair & 7 == codes[32 * r + 2 * i, 0] and pair >> 3 == codes[32 * r + 2 * i + 1, 0]


def test_q3_dequant_rules(oracle):
    vec, codes, sc, z = synth.q3_case(64, 16, seed=4)
    mat = oracle.q3_pack(codes)
    W = oracle.q3_dequant_f32(mat, sc, z)
    want = (sc.astype(np.float64) * codes - z.astype(np.float64)).astype(np.float32)  # one rounding
    assert np.array_equal(W, want)
    W16 = oracle.q3_dequant_f16(mat, sc, z)
    s16 = sc.astype(np.float16).astype(np.float64)
    z16 = (-z).astype(np.float16).astype(np.float64)
    want16 = (codes * s16 + z16).astype(np.float16)
    assert np.array_equal(W16.view(np.uint16), want16.view(np.uint16))


def test_q3_gemv_orders_agree_with_fp64(oracle):
    vec, codes, sc, z = synth.q3_case(1024, 64, seed=5)
    mat = oracle.q3_pack(codes)
    zero = np.zeros(64, dtype=np.float32)
    y64 = oracle.q3_gemv_f64(vec, mat, sc, z)
    assert oracle.rel_err(oracle.q3_gemv_f32(vec, mat, zero, sc, z), y64) < 1e-5
    dense = oracle.q3_dequant_f32(mat, sc, z).astype(np.float64).T @ vec.astype(np.float64)
    assert np.allclose(dense, y64, rtol=1e-12, atol=1e-12)
    vh = vec.astype(np.float16)
    y64h = oracle.q3_gemv_f64(vh.astype(np.float32), mat, sc, z, f16rule=True)
    assert oracle.rel_err(oracle.q3_gemv_f16in(vh, mat, zero, sc, z), y64h) < 1e-2
    # accumulation into mul
    base = np.full(64, 3.0, dtype=np.float32)
    assert np.allclose(oracle.q3_gemv_f32(vec, mat, base, sc, z),
                       oracle.q3_gemv_f32(vec, mat, zero, sc, z) + 3.0, rtol=1e-6, atol=1e-6)


# ---------- quantBnB ----------

def test_bnb_oracle_matches_reference_golden(oracle):
    g = np.load(GOLDEN / "bnb_golden.npz")
    assert np.array_equal(oracle.bnb_quantize(g["code"], g["A"]), g["out"])


def test_bnb_table_properties_and_nearest_neighbour(oracle):
    g = np.load(GOLDEN / "bnb_golden.npz")
    code = g["code"]
    assert code.size == 256 and np.all(np.diff(code) > 0) and code[127] == 0.0 and code[255] == 1.0
    rng = np.random.default_rng(7)
    x = rng.uniform(-1.2, 1.2, 50000).astype(np.float32)
    q = oracle.bnb_quantize(code, x)
    # away from exact ties the selected entry is the nearest table entry
    d = np.abs(x[:, None].astype(np.float64) - code[None, :].astype(np.float64))
    nearest = d.argmin(axis=1)
    best = d.min(axis=1)
    second = np.partition(d, 1, axis=1)[:, 1]
    clear = (second - best) > 1e-6
    assert np.array_equal(q[clear], nearest[clear].astype(np.uint8))


def test_bnb_reference_build_when_present(oracle):
    if oracle.ref_cpu() is None:
        pytest.skip("reference CPU build not present")
    g = np.load(GOLDEN / "bnb_golden.npz")
    assert np.array_equal(oracle.ref_bnb_code_table(), g["code"])
    x = np.random.default_rng(9).standard_normal(200000).astype(np.float32)
    assert np.array_equal(oracle.ref_bnb_quantize(x), oracle.bnb_quantize(g["code"], x))


# ---------- NF4 (parity unpinned: checked against an independent numpy restatement) ----------

@pytest.mark.parametrize("low_first", [0, 1])
def test_nf4_dequant_and_gemv(oracle, low_first):
    N, K, bs = 12, 256, 64
    A, B, absmax, lut = synth.nf4_case(N, K, bs, seed=6)
    hi, lo = B >> 4, B & 15
    codes = np.stack([lo, hi] if low_first else [hi, lo], axis=1).reshape(-1)
    w32 = (lut[codes] * np.repeat(absmax, bs)[:codes.size]).astype(np.float32)
    deq = oracle.nf4_dequant_f16(B, absmax, lut, N * K, bs, low_first)
    assert np.array_equal(deq.view(np.uint16), w32.astype(np.float16).view(np.uint16))
    y = oracle.nf4_gemv_f64(A, B, absmax, lut, N, K, bs, low_first)
    want = w32.reshape(N, K).astype(np.float64) @ A.astype(np.float64)
    assert np.allclose(y, want, rtol=1e-12, atol=1e-12)
    y32 = oracle.nf4_gemv_f32(A, B, absmax, lut, N, K, bs, low_first)
    assert oracle.rel_err(y32.astype(np.float64), y) < 2e-3


# ---------- LUT-GEMM ----------

@pytest.mark.parametrize("bias", [True, False])
def test_lutgemm_oracle(oracle, bias):
    M, K, nb, gs = 32, 256, 3, 128
    x, bW, alpha, qb = synth.lutgemm_case(M, K, nb, gs, seed=8, bias=bias)
    W = oracle.lutgemm_dequant_f32(bW, alpha, qb, M, K, nb, gs)
    # independent restatement (lut-gemm-cuda/main.cu:118-146 with the [K][M] layout)
    bits = ((bW[:, :, None, :] >> np.arange(32, dtype=np.uint32)[None, None, :, None]) & 1)
    signs = (2.0 * bits - 1.0).transpose(0, 2, 1, 3).reshape(K, nb, M)
    a = np.repeat(alpha.astype(np.float64), gs, axis=0)
    want = (signs * a).sum(axis=1)
    if bias:
        want = want + np.repeat(qb.astype(np.float64), gs, axis=0)
    assert np.allclose(W, want, rtol=1e-6, atol=1e-7)
    y = oracle.lutgemm_gemv_f64(x, bW, alpha, qb, M, K, nb, gs)
    assert np.allclose(y, want.T @ x.astype(np.float64), rtol=1e-10, atol=1e-10)
    y32 = oracle.lutgemm_gemv_f32(x, bW, alpha, qb, M, K, nb, gs)
    assert oracle.rel_err(y32.astype(np.float64), y) < 2e-3


# ---------- AQLM ----------

def test_aqlm_1x16_oracle(oracle):
    m, k = 24, 512
    codes, x, cb, scales = synth.aqlm_1x16_case(m, k, n_codebooks=3, seed=9)
    sizes = [8, 16, 24, 1 << 30]
    stride = 65536 * 8 * 2 // 16
    y64 = oracle.aqlm_1x16_f64(codes, x, cb, m, k, sizes, stride)
    want = np.empty(m)
    for r in range(m):
        book = cb[r // 8].astype(np.float64)
        want[r] = (book[codes[r]].reshape(-1) * x.astype(np.float64)).sum()
    assert np.allclose(y64, want, rtol=1e-12, atol=1e-12)
    yref = oracle.aqlm_1x16_ref(codes, x, cb, m, k, sizes, stride)
    assert oracle.rel_err(yref.astype(np.float64), y64) < 1e-2
    ys = oracle.aqlm_1x16_f64(codes, x, cb, m, k, sizes, stride, scales)
    assert np.allclose(ys, want * scales.astype(np.float64), rtol=1e-12)


def test_aqlm_2x8_oracle(oracle):
    m, k = 16, 256
    codes, x, cbs, scales = synth.aqlm_2x8_case(m, k, seed=10)
    y = oracle.aqlm_2x8_f64(codes, x, cbs, m, k, scales)
    w = cbs[0].astype(np.float64)[codes[:, :, 0]] + cbs[1].astype(np.float64)[codes[:, :, 1]]
    want = (w.reshape(m, k) @ x.astype(np.float64)) * scales.astype(np.float64)
    assert np.allclose(y, want, rtol=1e-12, atol=1e-12)


# ---------- batched ----------

def test_gemm_oracles(oracle):
    rng = np.random.default_rng(11)
    X = rng.standard_normal((5, 96)).astype(np.float16)
    W = rng.standard_normal((96, 40)).astype(np.float16)
    assert np.allclose(oracle.gemm_f16_f64(X, W), X.astype(np.float64) @ W.astype(np.float64))
    assert np.allclose(oracle.gemm_f16_nk_f64(X, np.ascontiguousarray(W.T)),
                       X.astype(np.float64) @ W.astype(np.float64))


def test_batched_nf4_oracle_agrees_with_gemv_oracle(oracle):
    """The batched path's checker (bit-exact dequantised weights, then an fp64
    product) gives, row by row, what the mat-vec oracle gives for that input."""
    from hecbench_b200 import synth
    Mb, K, N, bs = 3, 256, 40, 64
    X, B, absmax, lut = synth.qgemm_nf4_case(Mb, K, N, bs, seed=4)
    for low_first in (0, 1):
        W = oracle.nf4_dequant_f16(B, absmax, lut, N * K, bs, low_first).reshape(N, K)
        Y = oracle.gemm_f16_nk_f64(X, W)
        for j in range(Mb):
            y = oracle.nf4_gemv_f64(X[j], B, absmax, lut, N, K, bs, low_first)
            # the mat-vec oracle multiplies lut*absmax in fp64; the batched one rounds
            # each weight to fp16 first, as the kernel under test does
            assert np.allclose(Y[j], y, rtol=2e-3, atol=2e-3 * np.abs(y).max())


def test_bnb_pivot_only_rule_equals_dquantize(oracle):
    """The GPU kernel tracks only the pivot through the search and derives the
    bracket from the final pivot P (upper_pivot = P + 1, lower_pivot = max(P - 1, 0)).
    This numpy restatement of that rule must agree with the restated dQuantize<0>
    (quantBnB-cuda/main.cu:13-66) for ANY table - sorted, unsorted, with NaN
    entries - and any input, and with the reference-generated golden file."""
    def pivot_only(code, A):
        x = A.astype(np.float32)
        with np.errstate(invalid="ignore", over="ignore"):
            P = np.where(x > code[127], 191, 63)
            val = code[P]
            i = 32
            while i > 0:
                P = P + np.where(x > val, i, -i)
                val = code[P]
                i >>= 1
            gt = x > val
            nb = np.maximum(P + np.where(gt, 1, -1), 0)
            mid = (code[nb] + val) * np.float32(0.5)
            return np.where(np.where(gt, x > mid, x < mid), nb, P).astype(np.uint8)

    g = np.load(GOLDEN / "bnb_golden.npz")
    assert np.array_equal(pivot_only(g["code"], g["A"]), g["out"])
    rng = np.random.default_rng(1)
    for t in range(8):
        code = rng.standard_normal(256).astype(np.float32)
        if t % 3 == 0:
            code = np.sort(code)
        if t % 4 == 1:
            code[rng.integers(0, 256, 5)] = np.nan
        A = (rng.standard_normal(50000) * 2).astype(np.float32)
        A[:50] = np.nan
        A[50:100] = np.inf
        A[100:150] = -np.inf
        A[200:456] = code
        assert np.array_equal(pivot_only(code, A), oracle.bnb_quantize(code, A)), t


VLLM_DTYPES = ["float16", "bfloat16", "float32"]


@pytest.mark.parametrize("dtype", VLLM_DTYPES)
def test_vllm_quant_oracle_matches_reference_golden(oracle, dtype):
    """The C restatement of quantVLLM-cuda/reference.h against the golden file
    produced by the reference's own host functions (tests/golden/make_golden_vllm.py)."""
    g = np.load(GOLDEN / "vllm_golden.npz")
    x = g[f"x_{dtype}"]
    assert np.array_equal(oracle.vllm_static_quant(x, dtype, 0.1, 0), g[f"static_{dtype}"])
    assert np.array_equal(oracle.vllm_static_quant(x, dtype, 0.1, 54), g[f"static_azp_{dtype}"])
    q, s, _ = oracle.vllm_dynamic_quant(x, dtype, False)
    assert np.array_equal(q, g[f"dyn_{dtype}"])
    assert np.array_equal(s.view(np.uint32), g[f"dyn_scale_{dtype}"].view(np.uint32))
    q, s, z = oracle.vllm_dynamic_quant(x, dtype, True)
    assert np.array_equal(q, g[f"dynazp_{dtype}"])
    assert np.array_equal(s.view(np.uint32), g[f"dynazp_scale_{dtype}"].view(np.uint32))
    assert np.array_equal(z, g[f"dynazp_azp_{dtype}"])


def test_gemv_uniform_oracle_against_numpy(oracle):
    """The C restatement of gemv-cuda's device-side checks (gemv.cu:83-141)
    against the same arithmetic written in numpy: fp32 dequantisation with the
    fp16-rounded scale and zero point, element 2j in the low nibble."""
    from hecbench_b200 import synth
    for bits in (8, 4, 16):
        mat, vec = synth.gemv_uniform_case(33, 96, bits, seed=bits)
        y = oracle.gemv_uniform_f64(mat, vec, bits, 0.0625, 0.01)
        s = np.float32(np.float16(0.0625))
        z = np.float32(np.float16(0.01))
        if bits == 8:
            w = (mat.astype(np.float32) - z) * s
        elif bits == 4:
            w = np.empty((33, 96), np.float32)
            w[:, 0::2] = mat & 15
            w[:, 1::2] = mat >> 4
            w = (w - z) * s
        else:
            w = mat.astype(np.float32)
        assert np.array_equal(y, w.astype(np.float64) @ vec.astype(np.float64)) or \
            np.allclose(y, w.astype(np.float64) @ vec.astype(np.float64), rtol=1e-13, atol=0)


def _fused_dequant(fmt, mat, kw, rows, n):
    """fp32 weights of a fused-case matrix, in numpy."""
    if fmt == "f16":
        return mat.astype(np.float32)
    if fmt == "nf4":
        codes = np.empty(rows * n, np.uint8)
        flat = mat.reshape(-1)
        codes[0::2], codes[1::2] = flat >> 4, flat & 15   # element 2j in the high nibble
        return (kw["lut16"][codes] * np.repeat(kw["absmax"], kw["blocksize"])).reshape(rows, n)
    s, z = np.float32(np.float16(kw["scale"])), np.float32(np.float16(kw["zero_point"]))
    if fmt == "int8":
        return (mat.astype(np.float32) - z) * s
    w = np.empty((rows, n), np.float32)
    w[:, 0::2], w[:, 1::2] = mat & 15, mat >> 4
    return (w - z) * s


@pytest.mark.parametrize("fmt", ["f16", "int8", "int4", "nf4"])
@pytest.mark.parametrize("act", [0, 1, 2])
@pytest.mark.parametrize("norm", [True, False])
def test_gemv_fused_oracle_against_reference_operators(oracle, fmt, act, norm):
    """The C restatement of RMSNorm -> mat-vec -> SwiGLU / GeGLU (fp64) against
    (a) the same arithmetic in numpy fp64 and (b) the reference's own host checks
    of the three operators (rmsnorm-cuda, geglu-cuda, swish-cuda; fp32) around a
    numpy product, when the reference build is present."""
    from math import erf
    from hecbench_b200 import synth
    rows_out, n = 24, 128
    rows = rows_out * (2 if act else 1)
    rng = np.random.default_rng(11 + act)
    x = rng.standard_normal(n).astype(np.float16)
    gamma = rng.uniform(0.5, 1.5, n).astype(np.float16) if norm else None
    kw = {}
    if fmt == "nf4":
        _, B, absmax, lut = synth.nf4_case(rows, n, 64, 5)
        mat, kw = B.reshape(rows, n // 2), dict(absmax=absmax, lut16=lut, blocksize=64)
    else:
        mat, _ = synth.gemv_uniform_case(rows, n, {"f16": 16, "int8": 8, "int4": 4}[fmt], 5)
        if fmt != "f16":
            kw = dict(scale=0.05, zero_point=3.5)
    y = oracle.gemv_fused_f64(fmt, mat, x, gamma, 1e-5, rows_out, act, **kw)
    W = _fused_dequant(fmt, mat, kw, rows, n)
    xd = x.astype(np.float64)
    if norm:
        xd = xd / np.sqrt(np.mean(xd * xd) + 1e-5) * gamma.astype(np.float64)
    t = W.astype(np.float64) @ xd
    if act == 1:
        t = t[0::2] * t[1::2] / (1.0 + np.exp(-t[1::2]))
    elif act == 2:
        t = t[0::2] * 0.5 * t[1::2] * (1.0 + np.array([erf(g / np.sqrt(2.0)) for g in t[1::2]]))
    assert np.allclose(y, t, rtol=1e-12, atol=1e-12)
    ref = oracle.ref_fused_f32(W, x, gamma, rows_out, act)
    if ref is None:
        pytest.skip("reference host operators not built")
    assert np.allclose(y, ref.astype(np.float64), rtol=2e-5, atol=2e-5 * np.abs(y).max())


# ---------------- MXFP4 ----------------

# the values the reference driver draws from (mxfp4-cuda/main.cu:178-182) and what
# its own check expects of each (verify.h:3-85) when the group's scale is 1
MXFP4_KNOWN = {0.0: 0.0, 0.5: 0.5, 1.0: 1.0, 1.5: 1.5, 2.0: 2.0, 3.0: 3.0, 4.0: 4.0,
               0.25: 0.0, 0.75: 1.0, 1.25: 1.0, 1.75: 2.0, 2.5: 2.0, 3.5: 4.0, 5.0: 4.0,
               0.1: 0.0, 0.3: 0.5, 0.4: 0.5, 0.6: 0.5, 0.9: 1.0}


def mxfp4_driver_case(numel: int, seed: int, dtype):
    """Inputs drawn like the reference driver's (main.cu:184-190): every group of 32
    holds values of the list above, either sign, and one +-6 that fixes its scale at 1."""
    rng = np.random.default_rng(seed)
    vals = np.array(list(MXFP4_KNOWN) + [-v for v in MXFP4_KNOWN if v != 0.0] + [-0.0])
    x = rng.choice(vals, size=numel).reshape(-1, 32)
    pos = rng.integers(0, 32, size=x.shape[0])
    x[np.arange(x.shape[0]), pos] = np.where(pos < 16, 6.0, -6.0)
    return x.reshape(-1).astype(dtype)


def _bf16_bits(x32: np.ndarray) -> np.ndarray:
    u = x32.astype(np.float32).view(np.uint32)
    return ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def _bf16_vals(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize("bf16", [False, True])
def test_mxfp4_oracle_known_answers(oracle, bf16):
    x = mxfp4_driver_case(32 * 4096, 3, np.float32)
    bits = _bf16_bits(x) if bf16 else x.astype(np.float16).view(np.uint16)
    xin = _bf16_vals(bits) if bf16 else bits.view(np.float16).astype(np.float32)
    y_bits = oracle.mxfp4_qdq(bits, bf16)
    y = _bf16_vals(y_bits) if bf16 else y_bits.view(np.float16).astype(np.float32)
    # expectations are keyed by the value as T holds it (0.1, 0.3 ... are inexact)
    conv = (lambda v: float(_bf16_vals(_bf16_bits(np.array([v], np.float32)))[0])) if bf16 else \
        (lambda v: float(np.float16(v)))
    want = {conv(k): v for k, v in MXFP4_KNOWN.items()}
    want[conv(6.0)] = 6.0
    exp = np.array([np.copysign(want[abs(float(v))], v) for v in xin], dtype=np.float32)
    assert np.array_equal(y, exp)
    assert np.array_equal(np.signbit(y), np.signbit(xin))
    # the packed form decodes to the same values, scale byte 127 (2^0) everywhere
    codes, scales = oracle.mxfp4_quantize(bits, bf16)
    assert np.all(scales == 127)
    assert np.array_equal(oracle.mxfp4_dequantize(codes, scales, bf16), y_bits)


@pytest.mark.parametrize("bf16", [False, True])
def test_mxfp4_scale_exponent_is_the_references_where_that_is_defined(oracle, bf16):
    """floor(log2(rounded maximum)) - 2 from the fp32 form of the maximum equals
    the reference's expression on T's own bits for every finite maximum whose
    rounded value is a normal number of T."""
    top = 0x7f80 if bf16 else 0x7c00
    defined = 0
    for bits in range(0, top, 7 if bf16 else 3):
        ours, ref = oracle.mxfp4_scale_exponents(bits, bf16)
        if ref is not None:
            defined += 1
            assert ours == ref, hex(bits)
    assert defined > 1000


def test_mxfp4_oracle_random_groups(oracle):
    """Scaled groups: the result is the nearest grid value times the scale, ties
    to the even mantissa, computed here in numpy on exact binary fractions."""
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(32 * 2048) * np.repeat(2.0 ** rng.integers(-8, 9, 2048), 32))
    x = x.astype(np.float16)
    y = oracle.mxfp4_qdq(x.view(np.uint16)).view(np.float16).astype(np.float64)
    g = x.astype(np.float64).reshape(-1, 32)
    m = np.abs(g).max(axis=1)
    e = np.floor(np.log2(m))
    e = np.where(m / 2.0 ** e >= 1.75, e + 1, e)
    s = 2.0 ** (e - 2)
    a = np.abs(g) / s[:, None]
    step = np.where(a < 2, 0.5, np.where(a < 4, 1.0, 2.0))
    q = np.minimum(np.round(a / step) * step, 6.0)   # np.round: ties to even
    assert np.array_equal(y.reshape(-1, 32), np.copysign(q * s[:, None], g))


# ---------------- zero point ----------------

ZP_CONFIGS = [(-127, 127), (-128, 127), (0, 255), (0, 15), (-8, 7)]


@pytest.mark.parametrize("qmin,qmax", ZP_CONFIGS)
@pytest.mark.parametrize("preserve", [0, 1])
def test_zero_point_oracle_matches_reference_golden(oracle, qmin, qmax, preserve):
    """The C restatement against vectors recorded from the reference's own host
    function (zeropoint-cuda/reference.h): scales bit for bit, zero points equal."""
    g = np.load(GOLDEN / "zeropoint_golden.npz")
    scale, zp = oracle.zero_point(g["x_min"], g["x_max"], qmin, qmax, bool(preserve))
    assert np.array_equal(scale.view(np.uint32), g[f"scale_{qmin}_{qmax}_{preserve}"].view(np.uint32))
    assert np.array_equal(zp, g[f"zp_{qmin}_{qmax}_{preserve}"])
    ref = oracle.ref_zero_point(g["x_min"], g["x_max"], qmin, qmax, bool(preserve))
    if ref is not None:  # the reference build itself, where it is present
        assert np.array_equal(ref[0].view(np.uint32), scale.view(np.uint32))
        assert np.array_equal(ref[1], zp)


# ---------------- blockwise 4-bit quantizer ----------------

def spaced_levels(seed: int) -> np.ndarray:
    """16 ascending levels from -1 to 1, neighbours at least 0.05 apart (so that an
    fp16 rounding of level * absmax cannot cross a midpoint)."""
    rng = np.random.default_rng(seed)
    gaps = 0.05 + rng.uniform(0, 1, 15)
    lv = np.concatenate([[0.0], np.cumsum(gaps)])
    return (lv / lv[-1] * 2 - 1).astype(np.float32)


def test_nf4_quantize_oracle_against_numpy(oracle):
    rng = np.random.default_rng(2)
    lut = spaced_levels(1)
    w = (rng.standard_normal(64 * 300) * np.repeat(10.0 ** rng.integers(-3, 3, 300), 64)).astype(np.float32)
    w[128:192] = 0.0
    mids = (0.5 * (lut[:-1] + lut[1:])).astype(np.float32)
    w[200] = 0.0
    for order in (0, 1):
        B, absmax = oracle.nf4_quantize(w, 64, lut, order)
        g = w.reshape(-1, 64)
        m = np.abs(g).max(axis=1)
        assert np.array_equal(absmax, m)
        inv = np.where(m > 0, np.float32(1) / np.where(m > 0, m, 1), 0).astype(np.float32)
        x = (g * inv[:, None]).astype(np.float32)
        codes = (x[..., None] > mids).sum(axis=-1).astype(np.uint8).reshape(-1)
        first, second = (codes[0::2], codes[1::2])
        want = (second << 4 | first) if order else (first << 4 | second)
        assert np.array_equal(B, want)
        # dequantising and quantising again returns the same codes
        deq = oracle.nf4_dequant_f16(B, absmax, lut, w.size, 64, order).astype(np.float32)
        B2, _ = oracle.nf4_quantize(deq, 64, lut, order)
        assert np.array_equal(B2, B)


def test_q3_quantize_oracle_against_numpy(oracle):
    """The C restatement of the per-column min / max 3-bit quantizer against numpy,
    and its packed matrix through the unpacker and the dequantiser."""
    rng = np.random.default_rng(8)
    K, N = 96, 40
    W = (rng.standard_normal((K, N)) * rng.uniform(0.01, 2, N)).astype(np.float32)
    W[:, 0] = 0.0
    W[:, 1] = np.abs(W[:, 1]) + 0.5
    mat, scales, zeros = oracle.q3_quantize(W)
    lo, hi = np.minimum(W.min(axis=0), 0), np.maximum(W.max(axis=0), 0)
    lo[0], hi[0] = -1.0, 1.0
    sc = ((hi - lo) / np.float32(7)).astype(np.float32)
    z = np.rint((-lo / sc).astype(np.float32))
    q = np.clip(np.rint((W / sc).astype(np.float32)) + z, 0, 7).astype(np.uint8)
    assert np.array_equal(scales, sc) and np.array_equal(zeros, (sc * z).astype(np.float32))
    assert np.array_equal(oracle.q3_unpack(mat), q)
    Wq = oracle.q3_dequant_f32(mat, scales, zeros)
    assert np.all(np.abs(Wq - W) <= sc / 2 * (1 + 1e-5) + 1e-7)
