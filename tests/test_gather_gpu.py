"""One-GPU tests of the gather protocols through the C ABI, on ordinary device
memory with world = 1 (a rank is then its own only peer): the low-latency
packet form of the NF4 GEMV (packet output, packet input, epochs across
rounds), the copy + flag form, and the give-up path of every bounded wait - a
wait for something nobody will ever write must return within milliseconds with
status 1 and leave the GPU usable.  Nothing here faults or hangs the GPU: the
waits are counted loops that end on their own.

The same protocols across real peers are exercised by tests/multi_gpu_gather.py
(one process per GPU under torchrun)."""
import time

import numpy as np
import pytest

from hecbench_b200 import synth
from conftest import to_dev

pytestmark = pytest.mark.gpu
TOL_F16 = 1e-2


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def _ll_call(lib, *, A=None, A_ll=0, a_stride=1, B, absmax, lut, out=None, N, K, bs=64, flags=0,
             peer_ll=None, offset=0, sync, world=1, rank=0, max_polls=0, status):
    return lib.hq_nf4_gemv_f16_ll(
        0 if A is None else A.data_ptr(), A_ll, a_stride, B.data_ptr(), absmax.data_ptr(),
        lut.data_ptr(), 0 if out is None else out.data_ptr(), N, K, bs, flags,
        0 if peer_ll is None else peer_ll.data_ptr(), offset, sync.data_ptr(), world, rank,
        max_polls, status.data_ptr(), _stream())


@pytest.mark.parametrize("pairs", [False, True])
def test_ll_packets_chain_two_layers(hq, oracle, dev, monkeypatch, pairs):
    """Layer 1 (4096 x 4096) writes packets; layer 2 (512 x 4096) reads its input
    from those packets; three rounds over two alternating packet vectors, so later
    rounds meet the packets of earlier ones.  pairs: the opt-in form that sends two
    neighbouring rows in one 16-byte store."""
    import torch
    if pairs:
        monkeypatch.setenv("HQ_LL_PAIRS", "1")
    lib = hq.load_library()
    N1, K1, N2, bs = 4096, 4096, 512, 64
    A, B1, a1, lut = synth.nf4_case(N1, K1, bs, seed=21)
    _, B2, a2, _ = synth.nf4_case(N2, N1, bs, seed=22)
    dA, dB1, da1, dl = (to_dev(v, dev) for v in (A, B1, a1, lut))
    dB2, da2 = to_dev(B2, dev), to_dev(a2, dev)
    slots = [torch.zeros((N1, 2), dtype=torch.int32, device=dev) for _ in range(2)]
    peers = [torch.tensor([s.data_ptr()], dtype=torch.int64, device=dev) for s in slots]
    sync = torch.zeros(2, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    y1_ref = oracle.nf4_gemv_f64(A, B1, a1, lut, N1, K1, bs)
    for rnd in range(3):
        s = rnd % 2
        y2 = torch.full((N2,), 9.0, dtype=torch.float16, device=dev)
        assert _ll_call(lib, A=dA, B=dB1, absmax=da1, lut=dl, N=N1, K=K1, peer_ll=peers[s],
                        sync=sync, status=status) == 0
        assert _ll_call(lib, A_ll=slots[s].data_ptr(), B=dB2, absmax=da2, lut=dl, out=y2, N=N2,
                        K=N1, sync=sync, status=status) == 0
        y1 = torch.empty(N1, dtype=torch.float16, device=dev)
        assert lib.hq_ll_unpack(slots[s].data_ptr(), N1, y1.data_ptr(), sync.data_ptr(), 0,
                                status.data_ptr(), _stream()) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert sync.cpu().tolist() == [0, rnd + 1]
        pk = slots[s].cpu().numpy()
        assert np.all(pk[:, 1] == rnd + 1), "every packet carries the round's epoch"
        y1h = y1.cpu().numpy()
        assert oracle.rel_err(y1h.astype(np.float64), y1_ref) < TOL_F16
        y2_ref = oracle.nf4_gemv_f64(y1h, B2, a2, lut, N2, N1, bs)
        assert oracle.rel_err(y2.cpu().numpy().astype(np.float64), y2_ref) < TOL_F16


def test_ll_strided_input_matches_plain_input(hq, oracle, dev):
    """Packet input with a stride (element k = packet k * stride) gives bit for bit
    what the plain fp16 input gives."""
    import torch
    lib = hq.load_library()
    N, K, bs, stride = 256, 1024, 64, 3
    A, B, absmax, lut = synth.nf4_case(N, K, bs, seed=23)
    dA, dB, da, dl = (to_dev(v, dev) for v in (A, B, absmax, lut))
    pk = np.zeros((K * stride, 2), dtype=np.int32)
    pk[::stride, 0] = A.view(np.uint16).astype(np.int32)
    pk[::stride, 1] = 4
    dpk = to_dev(pk, dev)
    sync = torch.tensor([0, 4], dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    y_ll = torch.empty(N, dtype=torch.float16, device=dev)
    assert _ll_call(lib, A_ll=dpk.data_ptr(), a_stride=stride, B=dB, absmax=da, lut=dl, out=y_ll,
                    N=N, K=K, sync=sync, status=status) == 0
    y = hq.gemv_nf4(dA, dB, da, dl, N, K, bs)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(y_ll.view(torch.int16), y.view(torch.int16))


def test_ll_wait_for_missing_packets_gives_up(hq, oracle, dev):
    """Input packets that never reach the expected epoch: the kernel returns on its
    own with status 1; an ordinary GEMV afterwards is correct."""
    import torch
    lib = hq.load_library()
    N, K, bs = 256, 1024, 64
    A, B, absmax, lut = synth.nf4_case(N, K, bs, seed=24)
    dA, dB, da, dl = (to_dev(v, dev) for v in (A, B, absmax, lut))
    stale = torch.zeros((K, 2), dtype=torch.int32, device=dev)  # epoch 0 everywhere
    sync = torch.tensor([0, 5], dtype=torch.int32, device=dev)  # epoch 5 expected
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    y = torch.empty(N, dtype=torch.float16, device=dev)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    assert _ll_call(lib, A_ll=stale.data_ptr(), B=dB, absmax=da, lut=dl, out=y, N=N, K=K,
                    sync=sync, max_polls=2000, status=status) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0
    assert int(status.item()) == 1
    status.zero_()
    plain = torch.empty(K, dtype=torch.float16, device=dev)
    assert lib.hq_ll_unpack(stale.data_ptr(), K, plain.data_ptr(), sync.data_ptr(), 500,
                            status.data_ptr(), _stream()) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    good = hq.gemv_nf4(dA, dB, da, dl, N, K, bs)
    ref = oracle.nf4_gemv_f64(A, B, absmax, lut, N, K, bs)
    assert oracle.rel_err(good.cpu().numpy().astype(np.float64), ref) < TOL_F16


def test_gather_wait_gives_up_and_succeeds(hq, dev):
    """hq_gather_wait: a flag nobody raises -> status 1 within milliseconds; once
    the flag has the round's value the same wait leaves a fresh status word 0."""
    import torch
    lib = hq.load_library()
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    sync = torch.tensor([0, 1], dtype=torch.int32, device=dev)  # round 1 expected
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    t0 = time.perf_counter()
    assert lib.hq_gather_wait(flags.data_ptr(), sync.data_ptr(), 2, 4000, status.data_ptr(),
                              _stream()) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0
    assert int(status.item()) == 1
    flags[:2] = 1
    status.zero_()
    assert lib.hq_gather_wait(flags.data_ptr(), sync.data_ptr(), 2, 4000, status.data_ptr(),
                              _stream()) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0


def test_gather_publish_single_rank(hq, dev):
    """Copy + flag form with world = 1: the rank flags itself, the wait passes, the
    round counter advances and the slice is untouched."""
    import torch
    lib = hq.load_library()
    n = 1024
    data = torch.arange(n, dtype=torch.float16, device=dev)
    want = data.clone()
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    peer_out = torch.tensor([data.data_ptr()], dtype=torch.int64, device=dev)
    peer_flags = torch.tensor([flags.data_ptr()], dtype=torch.int64, device=dev)
    sync = torch.zeros(2, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for rnd in range(3):
        assert lib.hq_gather_publish(peer_out.data_ptr(), 0, n, peer_flags.data_ptr(),
                                     sync.data_ptr(), 1, 0, 0, status.data_ptr(), _stream()) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert sync.cpu().tolist() == [0, rnd + 1]
        assert int(flags[0].item()) == rnd + 1
    assert torch.equal(data, want)


@pytest.mark.parametrize("n,offset", [(100_000, 8), (24_000, 0), (1001, 3), (0, 0)])
def test_gather_publish_spreads_the_copy_over_ctas(hq, dev, n, offset):
    """world = 3, rank 1, with the two "peers" as further buffers of this GPU and
    their flags raised by the host beforehand, so the launch waits for no other
    kernel: the slice (several 16 KB pieces per peer, i.e. several CTAs; an
    unaligned one; an empty one = signal only) must arrive in both peer buffers,
    nothing outside it may change, and the flags and the round counter advance."""
    import torch
    lib = hq.load_library()
    total = offset + n + 64
    bufs = [torch.full((total,), float(r + 1), dtype=torch.float16, device=dev) for r in range(3)]
    bufs[1][offset:offset + n] = torch.arange(n, device=dev).remainder(2039).to(torch.float16)
    want = bufs[1][offset:offset + n].clone()
    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(3)]
    flags[1][0] = 1  # ranks 0 and 2 have "already published" round 1 here
    flags[1][2] = 1
    peer_out = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
    peer_flags = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=dev)
    sync = torch.zeros(2, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.hq_gather_publish(peer_out.data_ptr(), offset, n, peer_flags.data_ptr(),
                                 sync.data_ptr(), 3, 1, 0, status.data_ptr(), _stream()) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert sync.cpu().tolist() == [0, 1]
    for r in (0, 2):
        assert int(flags[r][1].item()) == 1            # this rank's flag on GPU r
        if n:
            assert torch.equal(bufs[r][offset:offset + n], want)
        assert bool((bufs[r][:offset] == r + 1).all()) and bool((bufs[r][offset + n:] == r + 1).all())
    assert int(flags[1][1].item()) == 1


@pytest.mark.parametrize("fmt", ["q3", "nf4"])
@pytest.mark.parametrize("Mb,N,K", [(64, 512, 1024), (37, 256, 4096)])
def test_qgemm_peer_epilogue_equals_plain(hq, dev, fmt, Mb, N, K):
    """The sharded form of the batched product (tiles stored to every GPU's slice by
    the epilogue) with two local buffers standing in for two GPUs: both must hold
    the plain product, at the given offset, and nothing around it changes; the
    narrow shape runs with the K split."""
    import torch
    offset = 128
    if fmt == "q3":
        X, codes, scales, zeros = synth.qgemm_q3_case(Mb, K, N, 128, seed=N + K)
        args = (to_dev(X, dev), to_dev(synth.q3_pack(codes), dev), to_dev(scales, dev),
                to_dev(zeros, dev), N, K, 128)
        fn = hq.qgemm_q3
    else:
        X, B, absmax, lut = synth.qgemm_nf4_case(Mb, K, N, 64, seed=N + K)
        args = (to_dev(X, dev), to_dev(B, dev), to_dev(absmax, dev), to_dev(lut, dev), N, K, 64, 0)
        fn = hq.qgemm_nf4
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    plain = fn(*args, status=status)
    bufs = [torch.full((offset + Mb * N + 64,), 3.0, dtype=torch.float16, device=dev) for _ in range(2)]
    table = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
    assert fn(*args, status=status, peers=(table.data_ptr(), offset, 2)) is None
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got = [b[offset:offset + Mb * N].view(Mb, N) for b in bufs]
    assert torch.equal(got[0], got[1])
    if N >= 512:
        assert torch.equal(got[0], plain)
    else:
        # K split: the partial sums meet in fp32 atomics, whose order differs from
        # launch to launch, so two launches agree only to fp32 rounding
        assert torch.allclose(got[0].float(), plain.float(), rtol=2e-3, atol=2e-3)
    for b in bufs:
        assert bool((b[:offset] == 3).all()) and bool((b[offset + Mb * N:] == 3).all())
