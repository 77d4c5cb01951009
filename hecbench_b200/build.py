"""In-tree build of libhq.so (the C-ABI launcher library) for sm_100a.

`python -m hecbench_b200.build` compiles every .cu under csrc/ with nvcc
(cross-compiles without a GPU) into hecbench_b200/libhq.so, and the
streaming-read probe of bench.py (csrc/probe/) into hecbench_b200/libhq_probe.so.  The objects are
cached under hecbench_b200/build/ and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libhq.so"
PROBE_LIB = PKG / "libhq_probe.so"
CHECKED_LIB = PKG / "libhq_checked.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
         f"-I{ROOT / 'include'}", f"-I{CSRC}"]
# extra nvcc flags, e.g. HQ_NVCC_FLAGS="-DHQ_BOUNDS_CHECK" for the index-checked build
FLAGS += os.environ.get("HQ_NVCC_FLAGS", "").split()


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((ROOT / "include").glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if force or _newer(obj, [src, *headers]):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [NVCC, *ARCH, *FLAGS, "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        (OBJ / (src.stem + ".ptxas.log")).write_text(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stderr}")
        if verbose:
            print(r.stderr, file=sys.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))

    objs = [OBJ / (s.stem + ".o") for s in sources]
    if force or jobs or _newer(LIB, objs):
        cmd = [NVCC, *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stderr}")
    # measurement aid of bench.py, kept out of the product library
    probe_src = CSRC / "probe" / "stream_read.cu"
    if force or _newer(PROBE_LIB, [probe_src, *headers]):
        cmd = [NVCC, *ARCH, *FLAGS, "-shared", str(probe_src), "-o", str(PROBE_LIB), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {probe_src.name}:\n{r.stderr}")
    return LIB


def build_checked(force: bool = False) -> Path:
    """The same sources with -DHQ_BOUNDS_CHECK into hecbench_b200/libhq_checked.so:
    every global access of the instrumented kernels is tested against its
    buffer's extent, violations are recorded and skipped (never trapped), and
    hq_bounds_check_report returns them.  The GPU tests run their small parity
    cases through this library as well."""
    global OBJ, LIB, PROBE_LIB, FLAGS
    saved = (OBJ, LIB, PROBE_LIB, FLAGS)
    try:
        OBJ = PKG / "build" / "checked"
        OBJ.parent.mkdir(exist_ok=True)
        LIB = CHECKED_LIB
        PROBE_LIB = OBJ / "probe_unused.so"
        FLAGS = FLAGS + ["-DHQ_BOUNDS_CHECK"]
        return build(force=force)
    finally:
        OBJ, LIB, PROBE_LIB, FLAGS = saved


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
    if "--checked" in sys.argv:
        print(build_checked(force="-f" in sys.argv))
