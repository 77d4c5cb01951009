"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (host-side numpy arrays).

These stand in for real checkpoints: codes are drawn uniformly, no quantiser is
run.  One generator per tensor family so that the tests, the smoke entry and
the bench all see the same data for a given seed.
"""
from __future__ import annotations

import numpy as np


def _rng(seed: int, stream: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64([int(seed), int(stream)]))


def q3_case(K: int, width: int, seed: int = 0):
    """GPTQ 3-bit: fp32 vec~N(0,1), codes U{0..7} (unpacked uint8[K][width]),
    scales~U(0.001,0.01), zeros = scale*U{0..7}."""
    codes = _rng(seed, 1).integers(0, 8, size=(K, width), dtype=np.uint8)
    vec = _rng(seed, 2).standard_normal(K).astype(np.float32)
    scales = _rng(seed, 3).uniform(0.001, 0.01, width).astype(np.float32)
    zeros = (scales * _rng(seed, 4).integers(0, 8, width).astype(np.float32)).astype(np.float32)
    return vec, codes, scales, zeros


def q3_pack(codes: np.ndarray) -> np.ndarray:
    """Pack 3-bit codes uint8[K][width] into the quant3MatMul layout
    int32[K*3/32][width]: per column and group of 32 inputs a 96-bit
    little-endian stream over three consecutive rows, code j at bits 3j..3j+2
    (quant3MatMul-cuda/kernels.h:41-87)."""
    K, width = codes.shape
    assert K % 32 == 0
    q = (codes.reshape(K // 32, 32, width) & 7).astype(np.uint64)
    w = np.zeros((K // 32, 3, width), dtype=np.uint64)
    for j in range(32):
        bit = 3 * j
        word, off = divmod(bit, 32)
        w[:, word] |= q[:, j] << np.uint64(off)
        if off > 29:
            w[:, word + 1] |= q[:, j] >> np.uint64(32 - off)
    w &= np.uint64(0xFFFFFFFF)
    return w.astype(np.uint32).view(np.int32).reshape(K // 32 * 3, width)


def q3_words(K: int, width: int, seed: int = 0) -> np.ndarray:
    """Packed quant3MatMul words int32[K*3/32][width] drawn directly: 32 uniform
    3-bit codes fill 96 bits exactly, so uniform codes and uniform words are the
    same distribution.  For large shapes where the unpacked codes are not needed."""
    assert K % 32 == 0
    w = _rng(seed, 5).integers(0, 2**32, size=(K // 32 * 3, width), dtype=np.uint32)
    return w.view(np.int32)


def nf4_levels(seed: int = 0) -> np.ndarray:
    """A 16-entry sorted level table in [-1, 1] with exact -1, 0 and 1 (the
    shape of a normal-float table; the values are seeded, not a published
    table)."""
    r = _rng(seed, 10)
    neg = -np.sort(r.uniform(0.05, 0.95, 6))[::-1]
    pos = np.sort(r.uniform(0.05, 0.95, 7))
    return np.concatenate([[-1.0], neg, [0.0], pos, [1.0]]).astype(np.float32)


def nf4_case(N: int, K: int, blocksize: int = 64, seed: int = 0):
    """NF4: fp16 A~N(0,1), codes uniform over 16 levels packed 2 per byte,
    fp32 absmax~U(0.01,0.1) per block."""
    n = N * K
    B = _rng(seed, 11).integers(0, 256, size=n // 2, dtype=np.uint8)
    absmax = _rng(seed, 12).uniform(0.01, 0.1, (n + blocksize - 1) // blocksize).astype(np.float32)
    A = _rng(seed, 13).standard_normal(K).astype(np.float16)
    return A, B, absmax, nf4_levels(seed)


def gemv_uniform_case(rows: int, n: int, bits: int, seed: int = 0):
    """gemv-cuda's inputs (simple_tensor.h:63-87): fp16 vec~U(0,1); mat int8
    uniform over -128..127, or two uniform 4-bit codes per byte, or fp16~U(0,1)."""
    vec = _rng(seed, 71).uniform(0.0, 1.0, n).astype(np.float16)
    if bits == 8:
        mat = _rng(seed, 72).integers(-128, 128, size=(rows, n), dtype=np.int8)
    elif bits == 4:
        mat = _rng(seed, 73).integers(0, 256, size=(rows, n // 2), dtype=np.uint8)
    else:
        mat = _rng(seed, 74).uniform(0.0, 1.0, (rows, n)).astype(np.float16)
    return mat, vec


def qgemm_nf4_case(Mb: int, K: int, N: int, blocksize: int = 64, seed: int = 0):
    """Batched NF4 path: fp16 X~N(0,1) plus the weights of nf4_case(N, K)."""
    _, B, absmax, lut16 = nf4_case(N, K, blocksize, seed)
    X = _rng(seed, 55).standard_normal((Mb, K)).astype(np.float16)
    return X, B, absmax, lut16


def lutgemm_case(M: int, K: int, nb: int = 3, group_size: int = 128, seed: int = 0,
                 bias: bool = True):
    """LUT-GEMM: fp16 x~N(0,1), Bernoulli(1/2) sign planes uint32[K/32][nb][M],
    fp16 alpha~U(0.001,0.05), fp16 q_bias~N(0,0.01)."""
    G = K // group_size
    bW = _rng(seed, 21).integers(0, 2**32, size=(K // 32, nb, M), dtype=np.uint32)
    alpha = _rng(seed, 22).uniform(0.001, 0.05, (G, nb, M)).astype(np.float16)
    q_bias = (_rng(seed, 23).standard_normal((G, M)) * 0.01).astype(np.float16) if bias else None
    x = _rng(seed, 24).standard_normal(K).astype(np.float16)
    return x, bW, alpha, q_bias


def aqlm_1x16_case(prob_m: int, prob_k: int, n_codebooks: int = 1, seed: int = 0):
    """AQLM 1x16: uint16 codes uniform over 65536, fp16 codebook[65536][8]~N(0,0.02),
    fp16 per-output scale~U(0.5,2)."""
    codes = _rng(seed, 31).integers(0, 65536, size=(prob_m, prob_k // 8), dtype=np.uint16)
    codebook = (_rng(seed, 32).standard_normal((n_codebooks, 65536, 8)) * 0.02).astype(np.float16)
    x = _rng(seed, 33).standard_normal(prob_k).astype(np.float16)
    scales = _rng(seed, 34).uniform(0.5, 2.0, prob_m).astype(np.float16)
    return codes, x, codebook, scales


def aqlm_2x8_case(prob_m: int, prob_k: int, seed: int = 0):
    codes = _rng(seed, 41).integers(0, 256, size=(prob_m, prob_k // 8, 2), dtype=np.uint8)
    codebooks = (_rng(seed, 42).standard_normal((2, 256, 8)) * 0.02).astype(np.float16)
    x = _rng(seed, 43).standard_normal(prob_k).astype(np.float16)
    scales = _rng(seed, 44).uniform(0.5, 2.0, prob_m).astype(np.float16)
    return codes, x, codebooks, scales


def qgemm_q3_case(Mb: int, K: int, N: int, group_size: int = 128, seed: int = 0):
    """Batched path: fp16 X~N(0,1), 3-bit codes uniform, per-group fp16
    scales~U(0.001,0.01) and zeros = scale*U{0..7}."""
    codes = _rng(seed, 51).integers(0, 8, size=(K, N), dtype=np.uint8)
    X = _rng(seed, 52).standard_normal((Mb, K)).astype(np.float16)
    G = K // group_size
    scales = _rng(seed, 53).uniform(0.001, 0.01, (G, N)).astype(np.float16)
    zeros = (scales.astype(np.float32) * _rng(seed, 54).integers(0, 8, (G, N))).astype(np.float16)
    return X, codes, scales, zeros
