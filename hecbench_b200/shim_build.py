"""Builds the C++ host-side drop-ins against libhq.so when the HeCBench tree is
present (the directory named by REFERENCE_ROOT, else a directory `reference`
beside this repository); used by the GPU drop-in tests.  Outputs (binaries
only) go to hecbench_b200/build/dropin/:

  dropin_quant3MatMul  reference main.cu + shim/quant3MatMul/kernels.h
  dropin_lutgemm       reference main.cu, nQWeight_fp16.cu + shim/lut-gemm/kernels.cu
  dropin_quantBnB      shim/quantBnB/main.cu (reference code.h on the include path)
  dropin_quantAQLM     shim/quantAQLM/main.cu
  dropin_quantVLLM     shim/quantVLLM/main.cu (reference reference.h, utils.h on the include path)
  dropin_gemv          reference main.cu + shim/gemv/gemv.cu (reference kernels.h, simple_tensor.h on the include path)
  dropin_zeropoint     shim/zeropoint/main.cu (reference reference.h on the include path)
  dropin_mxfp4         shim/mxfp4/main.cu (reference verify.h on the include path)
  shard_demo           shim/shard/main.cu: one-process host of the hq_shard_* context

The reference sources are compiled from where they lie; for quant3MatMul the
driver is copied into a temporary directory first, because `#include
"kernels.h"` resolves in the including file's own directory before any -I.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import tempfile
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
SHIM = PKG / "shim"
OUT = PKG / "build" / "dropin"
REF = Path(os.environ["REFERENCE_ROOT"]) if os.environ.get("REFERENCE_ROOT") else \
    ROOT.parent / "reference"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
COMMON = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-w",
          f"-I{ROOT / 'include'}", f"-L{PKG}", "-lhq", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../.."]


def _run(cmd, cwd=None):
    r = subprocess.run(list(map(str, cmd)), capture_output=True, text=True, cwd=cwd)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(map(str, cmd)) + "\n" + r.stderr)


def build(force: bool = False):
    """Returns the list of binaries built (only shard_demo when the reference
    tree is absent)."""
    src = REF / "src"
    OUT.mkdir(parents=True, exist_ok=True)
    lib = PKG / "libhq.so"
    built = []

    def stale(target: Path, deps):
        if force or not target.exists():
            return True
        t = target.stat().st_mtime
        return any(Path(d).exists() and Path(d).stat().st_mtime > t for d in [lib, *deps])

    # our own multi-GPU host for the hq_shard_* context (no reference source involved)
    tgt = OUT / "shard_demo"
    drv = SHIM / "shard" / "main.cu"
    if stale(tgt, [drv]):
        _run([NVCC, *COMMON, drv, "-o", tgt])
    built.append(tgt)
    if not (src / "quant3MatMul-cuda" / "main.cu").exists():
        return built

    # quant3MatMul: reference driver + our kernels.h
    tgt = OUT / "dropin_quant3MatMul"
    shim_h = SHIM / "quant3MatMul" / "kernels.h"
    if stale(tgt, [shim_h]):
        with tempfile.TemporaryDirectory() as tmp:
            shutil.copy(src / "quant3MatMul-cuda" / "main.cu", Path(tmp) / "main.cu")
            shutil.copy(shim_h, Path(tmp) / "kernels.h")
            _run([NVCC, *COMMON, "main.cu", "-o", tgt], cwd=tmp)
    built.append(tgt)

    # lut-gemm: reference driver and weight container + our kernels.cu
    tgt = OUT / "dropin_lutgemm"
    shim_cu = SHIM / "lut-gemm" / "kernels.cu"
    if stale(tgt, [shim_cu]):
        d = src / "lut-gemm-cuda"
        _run([NVCC, *COMMON, f"-I{d}", d / "main.cu", d / "nQWeight_fp16.cu", shim_cu, "-lcublas",
              "-o", tgt])
    built.append(tgt)

    tgt = OUT / "dropin_quantBnB"
    drv = SHIM / "quantBnB" / "main.cu"
    if stale(tgt, [drv]):
        _run([NVCC, *COMMON, f"-I{src / 'quantBnB-cuda'}", drv, "-o", tgt])
    built.append(tgt)

    tgt = OUT / "dropin_quantAQLM"
    drv = SHIM / "quantAQLM" / "main.cu"
    if stale(tgt, [drv]):
        _run([NVCC, *COMMON, drv, "-o", tgt])
    built.append(tgt)

    tgt = OUT / "dropin_quantVLLM"
    drv = SHIM / "quantVLLM" / "main.cu"
    if stale(tgt, [drv]):
        _run([NVCC, *COMMON, "--expt-relaxed-constexpr", f"-I{src / 'quantVLLM-cuda'}", drv,
              "-o", tgt])
    built.append(tgt)

    # gemv: reference driver (option parsing) + our gemv.cu in place of the reference's
    tgt = OUT / "dropin_gemv"
    shim_cu = SHIM / "gemv" / "gemv.cu"
    if stale(tgt, [shim_cu]):
        d = src / "gemv-cuda"
        _run([NVCC, *COMMON, f"-I{d}", d / "main.cu", shim_cu, "-o", tgt])
    built.append(tgt)

    for name, extra in (("zeropoint", []), ("mxfp4", ["--expt-relaxed-constexpr"])):
        tgt = OUT / f"dropin_{name}"
        drv = SHIM / name / "main.cu"
        if stale(tgt, [drv]):
            _run([NVCC, *COMMON, *extra, f"-I{src / (name + '-cuda')}", drv, "-o", tgt])
        built.append(tgt)
    return built


if __name__ == "__main__":
    for b in build(force=True):
        print(b)
