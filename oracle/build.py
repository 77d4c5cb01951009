"""Builds the test oracles.  TEST INFRASTRUCTURE ONLY.

  oracle/liboracle.so          plain-C restatement (hq_oracle.c), gcc -fopenmp
  oracle/_ref/libref_cpu.so    the reference's own CPU quantBnB code, g++
  oracle/_ref/libref_gpu.so    the reference's own CUDA kernels for sm_100a, nvcc
  oracle/_ref/ref_gpu_bench    the same kernels plus ref_gpu_bench.cu: the timing
                               program behind `bench.py --impl refgpu`

The _ref outputs are compiled from the reference sources where they lie: the
HeCBench tree named by REFERENCE_ROOT, or else a directory `reference` beside
this repository.  They are only (re)built when that tree is present, and never
needed by the shipped library.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = Path(os.environ["REFERENCE_ROOT"]) if os.environ.get("REFERENCE_ROOT") else \
    HERE.parent.parent / "reference"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def _run(cmd):
    r = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(map(str, cmd)) + "\n" + r.stderr)


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).exists() and Path(d).stat().st_mtime > t for d in deps)


def build_oracle(force: bool = False) -> Path:
    out = HERE / "liboracle.so"
    src = HERE / "hq_oracle.c"
    if force or _stale(out, [src]):
        _run(["gcc", "-O3", "-march=native", "-fopenmp", "-fPIC", "-shared", "-std=c11",
              "-fno-fast-math", "-ffp-contract=off", src, "-o", out, "-lm"])
    return out


def build_ref_cpu(force: bool = False):
    """The reference's CPU code of the path: quantBnB-omp/main.cpp, the host
    reference loops of quantVLLM-cuda/reference.h, and those of rmsnorm-cuda,
    geglu-cuda and swish-cuda (the operators fused around the mat-vec) and of
    zeropoint-cuda."""
    out = HERE / "_ref" / "libref_cpu.so"
    if not (REF / "src" / "quantBnB-omp" / "main.cpp").exists():
        return out if out.exists() else None
    # each harness sees only its own benchmark's directory (both have a utils.h)
    parts = {"ref_cpu.cpp": ["quantBnB-omp", "quantBnB-cuda"], "ref_cpu_vllm.cpp": ["quantVLLM-cuda"],
             "ref_cpu_fused.cpp": ["."],  # rmsnorm-cuda, geglu-cuda, swish-cuda by path
             "ref_cpu_zeropoint.cpp": ["zeropoint-cuda"]}
    if force or _stale(out, [HERE / p for p in parts]):
        out.parent.mkdir(exist_ok=True)
        cuda_inc = Path(NVCC).resolve().parent.parent / "include"
        objs = []
        for name, dirs in parts.items():
            obj = out.parent / (Path(name).stem + ".o")
            _run(["g++", "-O2", "-std=c++17", "-pthread", "-fPIC", "-w", "-fno-fast-math",
                  "-ffp-contract=off", *[f"-I{REF / 'src' / d}" for d in dirs], f"-I{cuda_inc}",
                  "-c", HERE / name, "-o", obj])
            objs.append(obj)
        _run(["g++", "-shared", "-pthread", *objs, "-o", out])
    return out


def build_ref_gpu(force: bool = False):
    out = HERE / "_ref" / "libref_gpu.so"
    if not (REF / "src" / "quant3MatMul-cuda" / "kernels.h").exists():
        return out if out.exists() else None
    parts = REF_GPU_PARTS
    srcs = [HERE / p for p in parts]
    if not (force or _stale(out, srcs)):
        return out
    out.parent.mkdir(exist_ok=True)
    objs = []
    for name, dirs in parts.items():
        obj = out.parent / (Path(name).stem + ".o")
        inc = [f"-I{REF / 'src' / d}" for d in dirs]
        _run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-w",
              "-Xcompiler", "-fPIC", *inc, "-c", HERE / name, "-o", obj])
        objs.append(obj)
    _run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", out, *objs,
          "-lcudart"])
    return out


REF_GPU_PARTS = {
    "ref_gpu_q3.cu": ["quant3MatMul-cuda"],
    "ref_gpu_bnb.cu": ["quantBnB-cuda"],
    "ref_gpu_lut.cu": ["lut-gemm-cuda"],
    "ref_gpu_aqlm.cu": ["quantAQLM-cuda"],
    "ref_gpu_gemv.cu": ["gemv-cuda"],
    "ref_gpu_mxfp4.cu": ["mxfp4-cuda"],
    "ref_gpu_zeropoint.cu": ["zeropoint-cuda"],
}


def build_ref_gpu_bench(force: bool = False):
    """The reference kernels again, with the default stream made per-thread so
    that their launches can be captured in a CUDA graph, linked with the timing
    program ref_gpu_bench.cu."""
    out = HERE / "_ref" / "ref_gpu_bench"
    if not (REF / "src" / "quant3MatMul-cuda" / "kernels.h").exists():
        return out if out.exists() else None
    srcs = [HERE / p for p in REF_GPU_PARTS] + [HERE / "ref_gpu_bench.cu"]
    if not (force or _stale(out, srcs)):
        return out
    out.parent.mkdir(exist_ok=True)
    common = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-w",
              "--default-stream", "per-thread"]
    objs = []
    for name, dirs in REF_GPU_PARTS.items():
        obj = out.parent / (Path(name).stem + "_pt.o")
        _run([*common, *[f"-I{REF / 'src' / d}" for d in dirs], "-c", HERE / name, "-o", obj])
        objs.append(obj)
    _run([*common, HERE / "ref_gpu_bench.cu", *objs, "-o", out, "-lcudart"])
    return out


def build_all(force: bool = False):
    return (build_oracle(force), build_ref_cpu(force), build_ref_gpu(force),
            build_ref_gpu_bench(force))


if __name__ == "__main__":
    for p in build_all(force="-f" in sys.argv):
        print(p)
