"""Drop-in tests: the reference's own host drivers (quant3MatMul, lut-gemm),
compiled unmodified against this library's shim headers / objects, and the two
replacement drivers (quantBnB, quantAQLM), run on the GPU and judged by the
drivers' own PASS / FAIL lines.  The binaries are built where the HeCBench tree
is available (hecbench_b200/shim_build.py) and travel as build outputs."""
import re
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
BIN = Path(__file__).resolve().parent.parent / "hecbench_b200" / "build" / "dropin"


def run(name, *args, timeout=600):
    exe = BIN / name
    if not exe.exists():
        pytest.skip(f"{name} not built (reference tree absent at build time)")
    r = subprocess.run([str(exe), *map(str, args)], capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def test_quant3matmul_reference_driver_passes():
    out = run("dropin_quant3MatMul", 20)
    lines = out.strip().splitlines()
    assert lines[0] == "PASS" and lines[1] == "PASS", out  # main.cu:91,105
    assert re.search(r"Average execution time of the kernel: [\d.]+ \(us\)", out)
    assert re.search(r"Average execution time of the faster kernel: [\d.]+ \(us\)", out)


def test_lutgemm_reference_driver_runs():
    out = run("dropin_lutgemm", 0, 5)
    assert out.count("mean Error") == 3 and out.count("latency min") == 3, out
    assert "status" not in out  # the shim prints a status line only on failure


def test_quantbnb_driver_passes():
    out = run("dropin_quantBnB", 1 << 20, 10)
    assert "Average execution time of kQuantize kernel with block size 256" in out
    assert out.strip().splitlines()[-1] == "PASS", out


def test_quantaqlm_driver_passes():
    out = run("dropin_quantAQLM")
    assert out.count("kernel execution time") == 4
    assert out.strip().splitlines()[-1] == "PASS", out


def test_quantvllm_driver_passes():
    """The reference run's own shape (4096 tokens x 5137), fewer repetitions."""
    out = run("dropin_quantVLLM", 4096, 5137, 20)
    assert out.count("Average execution time of") == 12
    assert out.count("PASS") == 3 and "FAIL" not in out, out
