"""Generates tests/golden/zeropoint_golden.npz from the reference's own host code.

Run where the HeCBench tree is available (REFERENCE_ROOT, or a directory
`reference` beside this repository): `python tests/golden/make_golden_zeropoint.py`.
It builds oracle/_ref/libref_cpu.so (which includes zeropoint-cuda/reference.h
from where it lies) and records

  x_min, x_max     4096 channel ranges: drawn like the reference driver's
                   (uniform in (-1, 1), zeropoint-cuda/main.cu:104-109, so min may
                   exceed max), ordered pairs at several magnitudes, ranges on one
                   side of zero, ranges touching zero, empty ranges, huge and
                   denormal bounds, exact ties of the zero point at .5
  scale_<c>, zp_<c>  the reference's outputs for configuration c =
                   "<qmin>_<qmax>_<preserve_sparsity>" over int8 symmetric
                   (-127, 127: the driver's), int8 (-128, 127), uint8 (0, 255),
                   uint4 (0, 15), int4 (-8, 7), each with and without
                   preserve_sparsity
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

from oracle import build, oracle as O  # noqa: E402

CONFIGS = [(-127, 127), (-128, 127), (0, 255), (0, 15), (-8, 7)]


def inputs():
    rng = np.random.default_rng(20240611)
    lo = np.empty(4096, dtype=np.float32)
    hi = np.empty(4096, dtype=np.float32)
    lo[:1024] = rng.uniform(-1, 1, 1024)                    # as the driver: unordered
    hi[:1024] = rng.uniform(-1, 1, 1024)
    a = rng.standard_normal(1024) * 10.0 ** rng.integers(-6, 6, 1024)
    b = rng.standard_normal(1024) * 10.0 ** rng.integers(-6, 6, 1024)
    lo[1024:2048], hi[1024:2048] = np.minimum(a, b), np.maximum(a, b)
    lo[2048:2304] = rng.uniform(0.1, 5, 256)                # positive only
    hi[2048:2304] = lo[2048:2304] + rng.uniform(0, 5, 256)
    hi[2304:2560] = -rng.uniform(0.1, 5, 256)               # negative only
    lo[2304:2560] = hi[2304:2560] - rng.uniform(0, 5, 256)
    lo[2560:2688], hi[2560:2688] = 0.0, rng.uniform(0, 3, 128)
    lo[2688:2816], hi[2688:2816] = -rng.uniform(0, 3, 128), 0.0
    lo[2816:2880] = hi[2816:2880] = rng.standard_normal(64)  # empty ranges
    lo[2880:2944] = hi[2880:2944] = 0.0
    lo[2944:3008] = -rng.uniform(0, 1, 64) * 1e-42           # denormal bounds
    hi[2944:3008] = rng.uniform(0, 1, 64) * 1e-42
    lo[3008:3072] = -rng.uniform(0.5, 1, 64) * 3e38          # huge bounds
    hi[3008:3072] = rng.uniform(0.5, 1, 64) * 3e38
    # zero points that land on .5 before rounding: min = -(k + .5) * s, max = (255 - k - .5) * s
    k = rng.integers(0, 255, 512).astype(np.float64)
    s = 2.0 ** rng.integers(-6, 3, 512)
    lo[3072:3584] = -(k + 0.5) * s
    hi[3072:3584] = (255 - k - 0.5) * s
    a = rng.uniform(-4, 0, 512)
    lo[3584:], hi[3584:] = a, a + rng.uniform(0, 8, 512)
    return lo, hi


def main():
    build.build_ref_cpu()
    lo, hi = inputs()
    out = {"x_min": lo, "x_max": hi}
    for qmin, qmax in CONFIGS:
        for ps in (0, 1):
            r = O.ref_zero_point(lo, hi, qmin, qmax, bool(ps))
            if r is None:
                raise SystemExit("oracle/_ref/libref_cpu.so is missing ref_zero_point")
            out[f"scale_{qmin}_{qmax}_{ps}"], out[f"zp_{qmin}_{qmax}_{ps}"] = r
    np.savez_compressed(Path(__file__).resolve().parent / "zeropoint_golden.npz", **out)
    print("wrote zeropoint_golden.npz:", {k: v.shape for k, v in out.items() if k.startswith("x_")})


if __name__ == "__main__":
    main()
