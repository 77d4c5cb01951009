"""Drop-in tests: the reference's own host drivers (quant3MatMul, lut-gemm),
compiled unmodified against this library's shim headers / objects, and the two
replacement drivers (quantBnB, quantAQLM), run on the GPU and judged by the
drivers' own PASS / FAIL lines.  The binaries are built where the HeCBench tree
is available (hecbench_b200/shim_build.py) and travel as build outputs."""
import math
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


def test_zeropoint_driver_passes():
    """The reference run's own size (10^7 channels, zeropoint-cuda/Makefile), fewer
    repetitions: the driver's comparison with the reference's host function."""
    out = run("dropin_zeropoint", 10000000, 20)
    assert "Average execution time of zero-point kernel" in out
    assert out.count("PASS") == 1 and "FAIL" not in out and "status" not in out, out


def test_mxfp4_driver_passes():
    """fp16 and bf16 sections with the reference's own verify.h; 2^24 elements (the
    reference run has 2^29)."""
    out = run("dropin_mxfp4", 1 << 24, 20)
    assert "Simulate conversion between FP16 and FP4" in out
    assert "Simulate conversion between BF16 and FP4" in out
    assert out.count("PASS") == 2 and "FAIL" not in out and "status" not in out, out


@pytest.mark.parametrize("size", [512, 4096])
def test_gemv_reference_driver_runs_clean(size):
    """The reference's own main.cu (option parsing, prints) linked with this
    library's gemv.cu: both quantized sections run and the device-side check
    (one '!!!' line per element outside 0.125 * n / 512) reports nothing but
    fp16 output rounding.  512 is the driver's default size (main.cu:31)."""
    out = run("dropin_gemv", "-s", size, "-i", 10)
    assert f"size={size}, iter=10" in out
    assert "GEMV int8 quantized..." in out and "GEMV int4 quantized..." in out
    assert out.count("Average kernel execution time") == 2
    assert out.count("Check correctness on the device") == 2
    assert "status" not in out, out
    # The reference's check allows 0.125 * n / 512 absolute, less than half an fp16
    # spacing of the largest results (its tensors are all drawn from the same
    # generator state, so row 0 correlates with the input vector and is large): a
    # correctly rounded fp16 result can be reported.  Every reported element must
    # be explained by that rounding alone.
    for m in re.finditer(r"!!!\[idx=(\d+)\] (\S+) != (\S+), diff=(\S+)", out):
        want, diff = float(m.group(3)), float(m.group(4))
        half_spacing = 2.0 ** (math.floor(math.log2(abs(want))) - 10) / 2
        assert abs(diff) <= half_spacing * 1.001, m.group(0)
