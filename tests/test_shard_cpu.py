"""World-size-2 gloo test of the output-feature sharding: each CPU rank computes
its slice with the oracle (the GPU launchers are injected in production) and
the gathered result must equal the unsharded oracle result."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hecbench_b200 import synth
        from hecbench_b200.shard import FeatureShard, gather_features
        from oracle import oracle as O
        # NF4 (row-major [N][K]) ------------------------------------------------
        N, K, bs = 64, 256, 64
        A, B, absmax, lut = synth.nf4_case(N, K, bs, seed=3)
        sh = FeatureShard(rank, world, N)
        Bl = sh.rows(B.reshape(N, K // 2)).reshape(-1)
        al = sh.nf4_absmax(absmax, K, bs)
        y_local = torch.from_numpy(O.nf4_gemv_f32(A, Bl, al, lut, sh.n_local, K, bs))
        y = gather_features(y_local, sh)
        full = O.nf4_gemv_f32(A, B, absmax, lut, N, K, bs)
        ok1 = np.array_equal(y.numpy().view(np.uint16), full.view(np.uint16))
        # q3 (column-major [rows][N]) batched: [Mb][N] outputs ------------------
        Kq, Nq = 128, 32
        vec, codes, sc, z = synth.q3_case(Kq, Nq, seed=4)
        mat = synth.q3_pack(codes)
        shq = FeatureShard(rank, world, Nq, multiple=4)
        ml = np.ascontiguousarray(shq.cols(mat))
        yl = O.q3_gemv_f32(vec, ml, np.zeros(shq.n_local, np.float32), shq.cols(sc), shq.cols(z))
        two = torch.from_numpy(np.stack([yl, 2 * yl]))  # a [2][n_local] "batch"
        yq = gather_features(two, shq)
        fullq = O.q3_gemv_f32(vec, mat, np.zeros(Nq, np.float32), sc, z)
        ok2 = np.array_equal(yq[0].numpy(), fullq) and np.array_equal(yq[1].numpy(), 2 * fullq)
        q.put((rank, bool(ok1), bool(ok2)))
    finally:
        dist.destroy_process_group()


def test_feature_sharding_world2_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    res = sorted(q.get(timeout=5) for _ in range(2))
    assert res == [(0, True, True), (1, True, True)]


def test_shard_arithmetic():
    from hecbench_b200.shard import FeatureShard
    s = FeatureShard(3, 8, 28672, multiple=128)
    assert (s.n_local, s.begin, s.end) == (3584, 10752, 14336)
    with pytest.raises(ValueError):
        FeatureShard(0, 8, 11008, multiple=128)  # 1376 is not a multiple of 128
    assert FeatureShard(1, 2, 11008).n_local == 5504
