"""Batched dequant-GEMM on the tensor cores (tcgen05 / tensor memory), 3-bit
and NF4 weights, against the oracle: bit-exact fp16 dequantised weights
(oracle rule) times X in fp64.
No reference implementation exists for this path (parity unpinned); tolerance
1e-2 on |y - ref| / max(|ref|, rms(ref)) for the fp16 output."""
import numpy as np
import pytest

from hecbench_b200 import synth
from conftest import to_dev

pytestmark = pytest.mark.gpu
TOL_F16 = 1e-2


def _run(hq, oracle, dev, Mb, K, N, group, seed):
    import torch
    X, codes, scales, zeros = synth.qgemm_q3_case(Mb, K, N, group, seed)
    mat = synth.q3_pack(codes)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    Y = hq.qgemm_q3(to_dev(X, dev), to_dev(mat, dev), to_dev(scales, dev), to_dev(zeros, dev), N, K,
                    group, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded in-kernel wait ran out"
    W16 = oracle.q3g_dequant_f16(mat, scales, zeros, K, N, group)
    ref = oracle.gemm_f16_f64(X, W16)
    return oracle.rel_err(Y.cpu().numpy().astype(np.float64), ref)


@pytest.mark.parametrize("Mb,K,N,group", [(64, 256, 128, 128), (16, 128, 256, 128),
                                          (64, 1024, 512, 128), (128, 512, 256, 64),
                                          (37, 256, 128, 128), (1, 128, 128, 64)])
def test_qgemm_q3_small(hq, oracle, dev, Mb, K, N, group):
    assert _run(hq, oracle, dev, Mb, K, N, group, seed=Mb + K + N) < TOL_F16


def _run_nf4(hq, oracle, dev, Mb, K, N, blocksize, low_first, seed):
    import torch
    X, B, absmax, lut16 = synth.qgemm_nf4_case(Mb, K, N, blocksize, seed)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    Y = hq.qgemm_nf4(to_dev(X, dev), to_dev(B, dev), to_dev(absmax, dev), to_dev(lut16, dev), N, K,
                     blocksize, low_first, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded in-kernel wait ran out"
    W16 = oracle.nf4_dequant_f16(B, absmax, lut16, N * K, blocksize, low_first).reshape(N, K)
    ref = oracle.gemm_f16_nk_f64(X, W16)
    return oracle.rel_err(Y.cpu().numpy().astype(np.float64), ref)


@pytest.mark.parametrize("Mb,K,N,blocksize,low_first", [
    (64, 256, 128, 64, 0), (16, 128, 256, 64, 1), (64, 1024, 512, 64, 0), (128, 512, 256, 128, 0),
    (37, 768, 128, 256, 1), (1, 128, 128, 64, 0), (64, 4096, 1024, 64, 0), (32, 576, 384, 192, 0)])
def test_qgemm_nf4_small(hq, oracle, dev, Mb, K, N, blocksize, low_first):
    assert _run_nf4(hq, oracle, dev, Mb, K, N, blocksize, low_first, seed=Mb + K + N) < TOL_F16


def test_qgemm_nf4_matches_dequant_then_gemm(hq, dev):
    """Llama-2-7B MLP shape (11008 x 4096): the fused kernel against the library's
    own NF4 dequantisation followed by a dense fp32 product in torch (checker only)."""
    import torch
    Mb, K, N = 64, 4096, 11008
    X, B, absmax, lut16 = synth.qgemm_nf4_case(Mb, K, N, 64, 5)
    dX, dB, dA, dL = (to_dev(a, dev) for a in (X, B, absmax, lut16))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    Y = hq.qgemm_nf4(dX, dB, dA, dL, N, K, 64, 0, status=status)
    W = hq.dequantize_nf4(dB, dA, dL, N * K, 64, 0).view(N, K)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = dX.float() @ W.float().t()
    err = (Y.float() - ref).abs() / torch.maximum(ref.abs(), ref.pow(2).mean().sqrt())
    assert float(err.max()) < TOL_F16


LLAMA3_70B_MLP = [(8192, 28672), (28672, 8192)]  # (K, N): up/gate and down projections


def _feature_subset(N, tiles=4, width=128):
    """`tiles` whole 128-feature tiles spread over [0, N): first, last and evenly between."""
    starts = np.unique(np.linspace(0, N - width, tiles).astype(np.int64) // width * width)
    return np.concatenate([np.arange(s0, s0 + width) for s0 in starts])


@pytest.mark.parametrize("K,N", LLAMA3_70B_MLP)
def test_qgemm_q3_llama3_70b_mlp(hq, oracle, dev, K, N):
    """Batch 64 at the full Llama-3-70B MLP shapes (the second one takes the K-split
    path): 512 output features against the CPU oracle (bit-exact fp16 dequantised
    weights times X in fp64), then every output against a dense fp32 product of
    the dequantised weights computed by torch on the same GPU."""
    import torch
    Mb, group = 64, 128
    X, codes, scales, zeros = synth.qgemm_q3_case(Mb, K, N, group, seed=K % 97)
    mat = synth.q3_pack(codes)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    dX, dS, dZ = to_dev(X, dev), to_dev(scales, dev), to_dev(zeros, dev)
    Y = hq.qgemm_q3(dX, to_dev(mat, dev), dS, dZ, N, K, group, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded in-kernel wait ran out"
    cols = _feature_subset(N)
    W16 = oracle.q3g_dequant_f16(np.ascontiguousarray(mat[:, cols]),
                                 np.ascontiguousarray(scales[:, cols]),
                                 np.ascontiguousarray(zeros[:, cols]), K, cols.size, group)
    ref = oracle.gemm_f16_f64(X, W16)
    got = Y[:, torch.from_numpy(cols).to(dev)].cpu().numpy().astype(np.float64)
    assert oracle.rel_err(got, ref) < TOL_F16
    assert oracle.rel_err_above_floor(got, ref) < TOL_F16
    s = dS.float().repeat_interleave(group, dim=0)
    z = dZ.float().repeat_interleave(group, dim=0)
    W = torch.addcmul(-z, torch.from_numpy(codes).to(dev).float(), s).half().float()
    del s, z
    full = dX.float() @ W
    err = (Y.float() - full).abs() / torch.maximum(full.abs(), full.pow(2).mean().sqrt())
    assert float(err.max()) < TOL_F16


@pytest.mark.parametrize("K,N", LLAMA3_70B_MLP)
def test_qgemm_nf4_llama3_70b_mlp(hq, oracle, dev, K, N):
    """The NF4 operand at the same two shapes: 512 output features against the CPU
    oracle, every output against the library's own bit-exact dequantisation
    followed by a dense fp32 product in torch."""
    import torch
    Mb, bs = 64, 64
    X, B, absmax, lut16 = synth.qgemm_nf4_case(Mb, K, N, bs, seed=K % 89)
    dX, dB, dA, dL = (to_dev(a, dev) for a in (X, B, absmax, lut16))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    Y = hq.qgemm_nf4(dX, dB, dA, dL, N, K, bs, 0, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded in-kernel wait ran out"
    rows = _feature_subset(N)
    Brows = np.ascontiguousarray(B.reshape(N, K // 2)[rows]).reshape(-1)
    Arows = np.ascontiguousarray(absmax.reshape(N, K // bs)[rows]).reshape(-1)
    W16 = oracle.nf4_dequant_f16(Brows, Arows, lut16, rows.size * K, bs, 0).reshape(rows.size, K)
    ref = oracle.gemm_f16_nk_f64(X, W16)
    got = Y[:, torch.from_numpy(rows).to(dev)].cpu().numpy().astype(np.float64)
    assert oracle.rel_err(got, ref) < TOL_F16
    assert oracle.rel_err_above_floor(got, ref) < TOL_F16
    W = hq.dequantize_nf4(dB, dA, dL, N * K, bs, 0).view(N, K)
    full = dX.float() @ W.float().t()
    err = (Y.float() - full).abs() / torch.maximum(full.abs(), full.pow(2).mean().sqrt())
    assert float(err.max()) < TOL_F16
