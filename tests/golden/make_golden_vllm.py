"""Generates tests/golden/vllm_golden.npz from the reference's own host code.

Run where the HeCBench tree is available (REFERENCE_ROOT, or a directory
`reference` beside this repository): `python tests/golden/make_golden_vllm.py`.
It builds oracle/_ref/libref_cpu.so (which includes quantVLLM-cuda/reference.h
and utils.h from where they lie) and records, for fp16 / bf16 / fp32 inputs,

  x_<dtype>        [24][517] inputs: rows drawn like the reference driver does
                   (integers rand() % 1000 - 300, quantVLLM-cuda/main.cu:189-192),
                   N(0,1) rows, rows of negative values only (the reference
                   starts its running maximum at FLT_MIN), rows with ties at
                   .5 after scaling, values beyond the int8 range, one huge value
  static_<dtype>, static_azp_<dtype>          int8 outputs, scale 0.1, azp 0 / 54
  dyn_<dtype>, dyn_scale_<dtype>              dynamic form without zero point
  dynazp_<dtype>, dynazp_scale_, dynazp_azp_  dynamic form with zero point
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

from oracle import build, oracle as O  # noqa: E402

TOKENS, HIDDEN = 24, 517


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns."""
    u = a.astype(np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def inputs() -> np.ndarray:
    rng = np.random.default_rng(20240607)
    x = np.empty((TOKENS, HIDDEN), dtype=np.float32)
    x[:8] = rng.integers(0, 1000, (8, HIDDEN)) - 300
    x[8:12] = rng.standard_normal((4, HIDDEN))
    x[12:14] = -np.abs(rng.standard_normal((2, HIDDEN))) - 0.25       # negative only
    x[14:16] = (rng.integers(-260, 260, (2, HIDDEN)) + 0.5) * 0.1      # ties at .5 for scale 0.1
    x[16:18] = rng.standard_normal((2, HIDDEN)) * 40.0                 # saturates with scale 0.1
    x[18] = rng.standard_normal(HIDDEN) * 1e-3
    x[19] = rng.standard_normal(HIDDEN); x[19, 7] = 60000.0
    x[20] = np.abs(rng.standard_normal(HIDDEN)) + 0.5                  # positive only
    x[21:24] = rng.integers(-128, 128, (3, HIDDEN)) * 0.5
    return x


def main():
    build.build_ref_cpu(force=True)
    base = inputs()
    out = {}
    for dtype, conv in [("float16", lambda a: a.astype(np.float16)), ("bfloat16", to_bf16_bits),
                        ("float32", lambda a: a.astype(np.float32))]:
        x = conv(base)
        out[f"x_{dtype}"] = x
        out[f"static_{dtype}"] = O.ref_vllm_static_quant(x, dtype, 0.1, 0)
        out[f"static_azp_{dtype}"] = O.ref_vllm_static_quant(x, dtype, 0.1, 54)
        q, s, _ = O.ref_vllm_dynamic_quant(x, dtype, False)
        out[f"dyn_{dtype}"], out[f"dyn_scale_{dtype}"] = q, s
        q, s, z = O.ref_vllm_dynamic_quant(x, dtype, True)
        out[f"dynazp_{dtype}"], out[f"dynazp_scale_{dtype}"], out[f"dynazp_azp_{dtype}"] = q, s, z
    path = Path(__file__).resolve().parent / "vllm_golden.npz"
    np.savez_compressed(path, **out)
    print(path, {k: v.shape for k, v in out.items() if k.startswith("x_")})


if __name__ == "__main__":
    main()
