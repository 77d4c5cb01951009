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


def test_qgemm_q3_llama_shapes_property(hq, dev):
    """Full Llama-3-70B MLP shapes: compare with a dense fp32 product of the
    dequantised weights computed by torch on the same GPU (checker only)."""
    import torch
    for (K, N) in [(8192, 28672), (28672, 8192)]:
        Mb, group = 64, 128
        g = torch.Generator(device="cpu").manual_seed(K)
        codes = torch.randint(0, 8, (K, N), generator=g, dtype=torch.uint8)
        mat = torch.from_numpy(synth.q3_pack(codes.numpy())).to(dev)
        scales = (torch.rand(K // group, N, generator=g) * 0.009 + 0.001).half()
        zeros = (scales.float() * torch.randint(0, 8, (K // group, N), generator=g)).half()
        X = torch.randn(Mb, K, generator=g).half()
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        Y = hq.qgemm_q3(X.to(dev), mat, scales.to(dev), zeros.to(dev), N, K, group, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        s = scales.to(dev).float().repeat_interleave(group, dim=0)
        z = zeros.to(dev).float().repeat_interleave(group, dim=0)
        W = (codes.to(dev).float() * s - z).half().float()
        ref = X.to(dev).float() @ W
        err = (Y.float() - ref).abs() / torch.maximum(ref.abs(), ref.pow(2).mean().sqrt())
        assert float(err.max()) < TOL_F16
        del W, s, z, ref
