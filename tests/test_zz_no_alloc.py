"""The allocation-free LUT-GEMM entry point (hq_lutgemm_nqmv_noalloc).

Meant for hosts that cannot allocate device memory where they call the
mat-vec - a plugin living inside another framework's memory pool, a serving
loop where cudaMalloc's device synchronisation is forbidden, a process whose
memory budget was fixed at start-up.  Its scratch row is a fixed array inside
the library's device image, shared by all calls on a device.

The test calls it through the C ABI twice in a row (the second call meets the
scratch contents the first one left behind) and compares each result with the
workspace-taking entry point hq_lutgemm_nqmv on the same inputs, within the
tolerance the other fp16-output tests use; it also checks that sizes beyond the
fixed maximum are rejected before anything is launched.  The file sorts last so
that a run stopping at the first failure has already run every other test.
"""

import numpy as np
import pytest

from hecbench_b200 import synth
from conftest import to_dev

pytestmark = pytest.mark.gpu

TOL_F16 = 1e-2


def test_noalloc_matches_workspace_entry_twice(hq, oracle, dev):
    import torch
    lib = hq.load_library()
    M, K, nb, gs = 4096, 1024, 3, 128
    x, bW, alpha, qb = synth.lutgemm_case(M, K, nb, gs, seed=11)
    w = hq.nQWeight_fp16(bW, alpha.astype(np.float32), K, M, nb, False, K // gs,
                         qb.astype(np.float32), device=dev)
    dx = to_dev(x.view(np.uint16), dev).view(torch.float16)
    ref_out = torch.empty(M, dtype=torch.float16, device=dev)
    hq.matmul(ref_out, dx, w)  # existing entry point, caller-provided workspace
    torch.cuda.synchronize()
    want = ref_out.cpu().numpy().astype(np.float64)
    truth = oracle.lutgemm_gemv_f64(x, bW, alpha, qb, M, K, nb, gs)
    stream = torch.cuda.current_stream().cuda_stream
    with torch.cuda.device(dev):
        for call in range(2):
            out = torch.full((M,), 3.0, dtype=torch.float16, device=dev)
            st = lib.hq_lutgemm_nqmv_noalloc(
                out.data_ptr(), dx.data_ptr(), w.bWeight.data_ptr(), w.alpha.data_ptr(),
                w.q_bias.data_ptr(), M, K, nb, gs, stream)
            assert st == 0, lib.hq_status_string(st)
            torch.cuda.synchronize()
            got = out.cpu().numpy().astype(np.float64)
            assert oracle.rel_err(got, want) < TOL_F16, f"call {call}"
            assert oracle.rel_err(got, truth) < TOL_F16, f"call {call}"


def test_noalloc_rejects_sizes_beyond_the_maximum(hq, dev):
    import torch
    lib = hq.load_library()
    t = torch.zeros(64, dtype=torch.float16, device=dev)
    p = t.data_ptr()
    with torch.cuda.device(dev):
        st = lib.hq_lutgemm_nqmv_noalloc(p, p, p, p, None, 65536 + 4, 128, 3, 128, None)
    assert st == -7  # HQ_ERR_TOO_LARGE
    assert lib.hq_status_string(st) == b"size beyond supported maximum"
