"""Two-or-more-GPU check of the fused NF4 GEMV + peer-store gather, run as
  python -m torch.distributed.run --nproc-per-node G --master-addr 127.0.0.1 tests/multi_gpu_gather.py
(not collected by pytest: it needs one process per GPU).  Every rank computes
its rows, the kernel stores them into all ranks' gathered vectors, and each
rank compares its gathered copy with the CPU oracle of the whole layer; the
NCCL all-gather of the plain kernel's output is checked the same way."""
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
    from hecbench_b200.shard import FeatureShard, PeerGather, gather_features
    from oracle import oracle as O

    n_local, K, bs = 1376, 4096, 64
    N = n_local * world
    A, B, absmax, lut = synth.nf4_case(N, K, bs, seed=7)
    sh = FeatureShard(rank, world, N)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    Bl = t(sh.rows(B.reshape(N, K // 2)).reshape(-1))
    al = t(sh.nf4_absmax(absmax, K, bs))
    dA, dl = t(A), t(lut)
    ref = O.nf4_gemv_f64(A, B, absmax, lut, N, K, bs)

    pg = PeerGather(sh, slots=3, device=dev)
    worst = 0.0
    for it in range(6):  # slots are reused: later rounds meet old contents and old flags
        i = it % 3
        pg.slot(i).zero_()
        torch.cuda.synchronize()
        dist.barrier()
        pg.gemv_nf4(i, dA, Bl, al, dl, K, bs)
        torch.cuda.synchronize()
        got = pg.slot(i).cpu().numpy().astype(np.float64)
        worst = max(worst, O.rel_err(got, ref))
    # chained form: each call waits inside the kernel for the previous gather
    for it in range(6):
        pg.gemv_nf4(it % 3, dA, Bl, al, dl, K, bs, wait=False, wait_previous=True)
    pg.wait_all()
    torch.cuda.synchronize()
    for i in range(3):
        worst = max(worst, O.rel_err(pg.slot(i).cpu().numpy().astype(np.float64), ref))
    # split form: ordinary kernel into the local slice, then the publish kernel
    for it in range(6):
        i = it % 3
        hq.gemv_nf4(dA, Bl, al, dl, n_local, K, bs, 0, pg.local_slice(i))
        pg.publish(i)
    torch.cuda.synchronize()
    for i in range(3):
        worst = max(worst, O.rel_err(pg.slot(i).cpu().numpy().astype(np.float64), ref))
    status = int(pg.status.item())
    y = hq.gemv_nf4(dA, Bl, al, dl, n_local, K, bs)
    full = gather_features(y, sh)
    err_nccl = O.rel_err(full.cpu().numpy().astype(np.float64), ref)
    ok = worst < 1e-2 and err_nccl < 1e-2 and status == 0
    print(f"[rank {rank}] fused gather rel err {worst:.2e}, nccl gather rel err {err_nccl:.2e}, "
          f"wait status {status}: {'PASS' if ok else 'FAIL'}", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    main()
