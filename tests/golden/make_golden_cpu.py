"""Generates tests/golden/bnb_golden.npz from the reference's own CPU code.

Run where the HeCBench tree is available (REFERENCE_ROOT, or a directory
`reference` beside this repository): `python tests/golden/make_golden_cpu.py`.  It builds
oracle/_ref/libref_cpu.so from quantBnB-omp/main.cpp and records

  code  the 256-entry table of quantBnB-cuda/code.h
  A     inputs: N(0,1) samples plus edge values (every table entry, every
        midpoint of neighbouring entries and its fp32 neighbours, +-inf, NaN,
        values outside [-1, 1], denormals, +-0)
  out   dQuantize<0>(code, 0, A[i]) computed by the reference build
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

from oracle import build, oracle as O  # noqa: E402


def main():
    build.build_ref_cpu(force=True)
    code = O.ref_bnb_code_table()
    assert code is not None, "reference tree not found"
    rng = np.random.Generator(np.random.PCG64(19937))
    normal = rng.standard_normal(24576).astype(np.float32)
    mids = ((code[1:] + code[:-1]) * np.float32(0.5)).astype(np.float32)
    edge = np.concatenate([
        code, mids, np.nextafter(mids, np.float32(np.inf)), np.nextafter(mids, np.float32(-np.inf)),
        np.nextafter(code, np.float32(np.inf)), np.nextafter(code, np.float32(-np.inf)),
        np.array([np.inf, -np.inf, np.nan, 0.0, -0.0, 1e-45, -1e-45, 1.5, -1.5, 1e30, -1e30,
                  0.99999994, -0.99999994], dtype=np.float32),
    ]).astype(np.float32)
    A = np.concatenate([normal, edge]).astype(np.float32)
    out = O.ref_bnb_quantize(A)
    np.savez_compressed(Path(__file__).parent / "bnb_golden.npz", code=code, A=A, out=out)
    print("bnb_golden.npz:", A.size, "samples; histogram head", np.bincount(out, minlength=256)[:4])


if __name__ == "__main__":
    main()
