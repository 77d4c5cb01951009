"""Per-token int8 activation quantization (quantVLLM) on the GPU, through the
mirrored launchers, byte for byte against (1) the golden file produced by the
reference's own host functions (quantVLLM-cuda/reference.h) and (2) the CPU
oracle on fresh inputs, including the reference run's own shape
(hidden_size = 5137: rows that start at odd addresses) and rows longer than
the register cache."""
import numpy as np
import pytest

from conftest import GOLDEN

pytestmark = pytest.mark.gpu
DTYPES = ["float16", "bfloat16", "float32"]


def _to_dev(x, dtype, dev):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x.view(np.int16) if dtype == "bfloat16" else x))
    t = t.to(dev)
    return t.view(torch.bfloat16) if dtype == "bfloat16" else t


def _run_all(hq, x, dtype, dev):
    import torch
    tokens, hidden = x.shape
    dx = _to_dev(x, dtype, dev)
    res = {}
    for azp in (0, 54):
        out = torch.full((tokens, hidden), 99, dtype=torch.int8, device=dev)
        hq.static_scaled_int8_quant(out, dx, hidden, tokens, 0.1, azp)
        res["static" if azp == 0 else "static_azp"] = out.cpu().numpy()
    out = torch.full((tokens, hidden), 99, dtype=torch.int8, device=dev)
    sc = torch.zeros(tokens, dtype=torch.float32, device=dev)
    hq.dynamic_scaled_int8_quant(out, dx, hidden, tokens, sc, None)
    res["dyn"], res["dyn_scale"] = out.cpu().numpy(), sc.cpu().numpy()
    out = torch.full((tokens, hidden), 99, dtype=torch.int8, device=dev)
    sc = torch.zeros(tokens, dtype=torch.float32, device=dev)
    zp = torch.zeros(tokens, dtype=torch.int32, device=dev)
    hq.dynamic_scaled_int8_quant(out, dx, hidden, tokens, sc, zp)
    res["dynazp"], res["dynazp_scale"], res["dynazp_azp"] = (out.cpu().numpy(), sc.cpu().numpy(),
                                                            zp.cpu().numpy())
    return res


def _same(a, b):
    if a.dtype == np.float32:
        return np.array_equal(a.view(np.uint32), b.view(np.uint32))
    return np.array_equal(a, b)


@pytest.mark.parametrize("dtype", DTYPES)
def test_vllm_quant_matches_reference_golden(hq, dev, dtype):
    g = np.load(GOLDEN / "vllm_golden.npz")
    res = _run_all(hq, g[f"x_{dtype}"], dtype, dev)
    for key, got in res.items():
        assert _same(got, g[f"{key}_{dtype}"]), key


def _bf16_bits(a):
    u = a.astype(np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,hidden", [(64, 5137), (3, 1), (5, 4096), (2, 9001), (7, 16)])
def test_vllm_quant_matches_oracle(hq, oracle, dev, dtype, tokens, hidden):
    rng = np.random.default_rng(tokens * 100003 + hidden)
    base = (rng.integers(0, 1000, (tokens, hidden)) - 300).astype(np.float32)
    base[0] = rng.standard_normal(hidden) * 3
    x = {"float16": lambda a: a.astype(np.float16), "bfloat16": _bf16_bits,
         "float32": lambda a: a.astype(np.float32)}[dtype](base)
    res = _run_all(hq, x, dtype, dev)
    assert _same(res["static"], oracle.vllm_static_quant(x, dtype, 0.1, 0))
    assert _same(res["static_azp"], oracle.vllm_static_quant(x, dtype, 0.1, 54))
    q, s, _ = oracle.vllm_dynamic_quant(x, dtype, False)
    assert _same(res["dyn"], q) and _same(res["dyn_scale"], s)
    q, s, z = oracle.vllm_dynamic_quant(x, dtype, True)
    assert _same(res["dynazp"], q) and _same(res["dynazp_scale"], s) and _same(res["dynazp_azp"], z)


def test_vllm_quant_rejects_bad_arguments(hq, dev):
    import torch
    t = torch.zeros((4, 8), dtype=torch.float64, device=dev)
    o = torch.zeros((4, 8), dtype=torch.int8, device=dev)
    with pytest.raises(TypeError):
        hq.static_scaled_int8_quant(o, t, 8, 4, 0.1)
    with pytest.raises(TypeError):
        hq.static_scaled_int8_quant(o, torch.zeros(4, 8), 8, 4, 0.1)
