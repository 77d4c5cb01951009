"""Two-or-more-GPU check of the sharded path, run as
  python -m torch.distributed.run --nproc-per-node G --master-addr 127.0.0.1 tests/multi_gpu_gather.py
(not collected by pytest: it needs one process per GPU).  Every rank owns a
slice of the output features; each rank compares ITS copy of every gathered
result with the CPU oracle of the whole layer.

  1. NF4 GEMV, low-latency packet gather (PacketGather): a chain of layers in
     which every layer's input is read from the previous layer's gathered
     packets, first step by step (each layer unpacked and checked), then back
     to back with no host synchronisation in between;
  2. NF4 GEMV, copy + flag gather (PeerGather.publish);
  3. NF4 GEMV, NCCL all-gather;
  4. batched dequant-GEMM (3-bit and NF4 weights), column-sharded, gathered by
     PeerGather.publish (rows = batch) and by NCCL.
"""
import datetime
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    rank, world = dist.get_rank(), dist.get_world_size()
    import hecbench_b200 as hq
    from hecbench_b200 import synth
    from hecbench_b200.shard import FeatureShard, PacketGather, PeerGather, gather_features
    from oracle import oracle as O

    t = lambda a: torch.from_numpy(np.ascontiguousarray(
        a.view(np.int32) if a.dtype == np.uint32 else a)).to(dev)
    f64 = lambda x: x.cpu().numpy().astype(np.float64)
    report = {}

    # ---- 1-3: NF4 GEMV --------------------------------------------------------
    n_local, K, bs = 1376, 1024, 64
    N = n_local * world
    stride = N // K  # the next layer's input: every stride-th element of the gathered output
    A, B, absmax, lut = synth.nf4_case(N, K, bs, seed=7)
    sh = FeatureShard(rank, world, N)
    Bl = t(sh.rows(B.reshape(N, K // 2)).reshape(-1))
    al = t(sh.nf4_absmax(absmax, K, bs))
    dA, dl = t(A), t(lut)

    layers, slots = 6, 3
    # the same chain once more through the NVSwitch multicast mapping, where there is one
    pm = PacketGather(sh, slots=slots, device=dev, multicast=None)
    if pm.multicast:
        x_host, worst = A, 0.0
        for l in range(layers):
            if l == 0:
                pm.gemv_nf4(0, dA, Bl, al, dl, K, bs, weights_resident=True)
            else:
                pm.gemv_nf4(l % slots, None, Bl, al, dl, K, bs, weights_resident=True,
                            a_slot=(l - 1) % slots, a_stride=stride)
            y = pm.unpack(l % slots)
            torch.cuda.synchronize()
            yh = y.cpu().numpy()
            worst = max(worst, O.rel_err(yh.astype(np.float64),
                                         O.nf4_gemv_f64(x_host, B, absmax, lut, N, K, bs)))
            x_host = np.ascontiguousarray(yh[::stride][:K])
            dist.barrier()
        report["packets by multicast"] = worst
        if int(pm.status.item()) != 0:
            report["packets by multicast"] = 1.0
    pg = PacketGather(sh, slots=slots, device=dev, multicast=False)
    worst = 0.0
    x_host = A
    finals = []
    for l in range(layers):  # step by step
        if l == 0:
            pg.gemv_nf4(0, dA, Bl, al, dl, K, bs, weights_resident=True)
        else:
            pg.gemv_nf4(l % slots, None, Bl, al, dl, K, bs, weights_resident=True,
                        a_slot=(l - 1) % slots, a_stride=stride)
        y = pg.unpack(l % slots)
        torch.cuda.synchronize()
        yh = y.cpu().numpy()
        worst = max(worst, O.rel_err(yh.astype(np.float64),
                                     O.nf4_gemv_f64(x_host, B, absmax, lut, N, K, bs)))
        finals.append(yh.copy())
        x_host = np.ascontiguousarray(yh[::stride][:K])
        dist.barrier()
    report["packets step by step"] = worst
    # the same chain twice more, back to back; packets of older rounds are in the slots
    same = True
    for _ in range(2):
        for l in range(layers):
            if l == 0:
                pg.gemv_nf4(0, dA, Bl, al, dl, K, bs, weights_resident=True)
            else:
                pg.gemv_nf4(l % slots, None, Bl, al, dl, K, bs, weights_resident=True,
                            a_slot=(l - 1) % slots, a_stride=stride)
        y = pg.unpack((layers - 1) % slots)
        torch.cuda.synchronize()
        same = same and np.array_equal(y.cpu().numpy().view(np.uint16), finals[-1].view(np.uint16))
        dist.barrier()
    report["packets back to back == step by step"] = 0.0 if same else 1.0
    status = int(pg.status.item())

    ref = O.nf4_gemv_f64(A, B, absmax, lut, N, K, bs)
    pp = PeerGather(sh, slots=3, device=dev)
    worst = 0.0
    for it in range(6):
        i = it % 3
        hq.gemv_nf4(dA, Bl, al, dl, n_local, K, bs, 0, pp.local_slice(i))
        pp.publish(i)
    torch.cuda.synchronize()
    for i in range(3):
        worst = max(worst, O.rel_err(f64(pp.slot(i)), ref))
    report["publish"] = worst
    status |= int(pp.status.item())
    y = hq.gemv_nf4(dA, Bl, al, dl, n_local, K, bs)
    report["nccl"] = O.rel_err(f64(gather_features(y, sh)), ref)

    # ---- 4: batched dequant-GEMM, column-sharded -------------------------------
    Mb, Kg, ng_local, group = 64, 1024, 256, 128
    Ng = ng_local * world
    shg = FeatureShard(rank, world, Ng, multiple=128)
    X, codes, scales, zeros = synth.qgemm_q3_case(Mb, Kg, Ng, group, seed=9)
    mat = synth.q3_pack(codes)
    ref_q3 = O.gemm_f16_f64(X, O.q3g_dequant_f16(mat, scales, zeros, Kg, Ng, group))
    dX = t(X)
    stq = torch.zeros(1, dtype=torch.int32, device=dev)
    pq = PeerGather(shg, slots=2, device=dev, rows=Mb)
    args_q3 = (dX, t(shg.cols(mat)), t(shg.cols(scales)), t(shg.cols(zeros)), ng_local, Kg, group)
    worst = 0.0
    for it in range(4):
        i = it % 2
        hq.qgemm_q3(*args_q3, out=pq.local_slice(i), status=stq)
        pq.publish(i)
    torch.cuda.synchronize()
    for i in range(2):
        got = pq.slot(i).permute(1, 0, 2).reshape(Mb, Ng)  # [G][Mb][n] -> [Mb][G*n]
        worst = max(worst, O.rel_err(f64(got), ref_q3))
    report["qgemm q3 publish"] = worst
    Yl = hq.qgemm_q3(*args_q3, status=stq)
    report["qgemm q3 nccl"] = O.rel_err(f64(gather_features(Yl, shg)), ref_q3)

    Xn, Bn, an, ln = synth.qgemm_nf4_case(Mb, Kg, Ng, 64, seed=10)
    Wn = O.nf4_dequant_f16(Bn, an, ln, Ng * Kg, 64).reshape(Ng, Kg)
    ref_nf4 = O.gemm_f16_nk_f64(Xn, Wn)
    args_nf4 = (t(Xn), t(shg.rows(Bn.reshape(Ng, Kg // 2)).reshape(-1)),
                t(shg.nf4_absmax(an, Kg, 64)), t(ln), ng_local, Kg, 64, 0)
    hq.qgemm_nf4(*args_nf4, out=pq.local_slice(0), status=stq)
    pq.publish(0)
    torch.cuda.synchronize()
    report["qgemm nf4 publish"] = O.rel_err(
        f64(pq.slot(0).permute(1, 0, 2).reshape(Mb, Ng)), ref_nf4)

    # fused form: the product's epilogue stores every tile into all GPUs' buffers and
    # publish only signals; the buffers are cleared first so that nothing stale passes
    def clear_slots():
        torch.cuda.synchronize(); dist.barrier()
        for i in range(2):
            pq.slot(i).zero_()
        torch.cuda.synchronize(); dist.barrier()
    clear_slots()
    for it in range(4):
        i = it % 2
        hq.qgemm_q3(*args_q3, status=stq, peers=pq.peers(i))
        pq.publish(i, stored=True)
    torch.cuda.synchronize()
    report["qgemm q3 fused"] = max(
        O.rel_err(f64(pq.slot(i).permute(1, 0, 2).reshape(Mb, Ng)), ref_q3) for i in range(2))
    clear_slots()
    hq.qgemm_nf4(*args_nf4, status=stq, peers=pq.peers(1))
    pq.publish(1, stored=True)
    torch.cuda.synchronize()
    report["qgemm nf4 fused"] = O.rel_err(
        f64(pq.slot(1).permute(1, 0, 2).reshape(Mb, Ng)), ref_nf4)
    # fused with the K split (narrow shard, workspace in use) and a ragged batch
    clear_slots()
    Xr = dX[:37].contiguous()
    hq.qgemm_q3(Xr, *args_q3[1:], status=stq, peers=pq.peers(0))
    pq.publish(0, stored=True)
    torch.cuda.synchronize()
    got = pq.slot(0)[:, :37, :]  # rows 37 .. 63 of every slice stay zero
    report["qgemm q3 fused ragged"] = O.rel_err(
        f64(got.permute(1, 0, 2).reshape(37, Ng)), ref_q3[:37])
    if float(pq.slot(0)[:, 37:, :].abs().max()) != 0.0:
        status |= 2
    status |= int(pq.status.item()) | int(stq.item())

    ok = status == 0 and all(v < 1e-2 for v in report.values())
    print(f"[rank {rank}/{world}] " + ", ".join(f"{k}: {v:.2e}" for k, v in report.items()) +
          f", wait status {status}: {'PASS' if ok else 'FAIL'}", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    main()
