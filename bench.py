#!/usr/bin/env python
"""Benchmark of the quantized mat-vec hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one pass of the workload's kernel over R independent packed
weight replicas (R layers of a decoder, back to back, as one CUDA graph); R is
chosen so that R x bytes is several times the 126 MB L2, so every launch
streams its weights from HBM.  Rank 0 prints ONE JSON line:

  value      effective weight GB/s over all ranks = algorithmic bytes / time,
             inputs resident in HBM, CUDA-event timed, max over ranks
  e2e        same metric through the C ABI with HOST activations: every launch
             copies its input vector from pinned host memory and its output
             back (weights are model state and stay resident)
  roofline   achieved GB/s of the kernel (algorithmic bytes per launch / mean
             launch duration inside the timed region) against the measured HBM
             copy bandwidth of MEASURED_PEAKS.json
  cpu_baseline  the CPU oracle port of the same workload timed on a bounded
             sample on this box's host cores (rank 0, N = 1 only)

`--impl reference` times the reference algorithm's CPU implementation (the
reference's own build for kQuantize, the oracle port otherwise) on the same
workload with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_BF16_TFLOPS = 1590.0
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peak():
    """Dense bf16 cuBLAS throughput measured on this pool (burst figure: the
    kernel is timed in a short graph, not inside a seconds-long step)."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"]), "measured"
        except Exception:
            pass
    return FALLBACK_BF16_TFLOPS, "fallback"


def ncu_traffic(workload: str):
    """DRAM bytes per launch from the committed ncu summary, or None."""
    p = ROOT / "profiles" / "traffic.json"
    if p.exists():
        try:
            return json.loads(p.read_text()).get(workload, {}).get("dram_bytes_per_launch")
        except Exception:
            return None
    return None


# --------------------------------------------------------------------------
# workloads: name -> builder(seed) returning a dict of host arrays + metadata
# --------------------------------------------------------------------------

def _host_case(name: str, seed: int):
    from hecbench_b200 import synth
    if name == "nf4_gemv":
        N, K, bs = 11008, 4096, 64
        A, B, absmax, lut = synth.nf4_case(N, K, bs, seed)
        return dict(N=N, K=K, bs=bs, A=A, B=B, absmax=absmax, lut=lut,
                    bytes=B.nbytes + absmax.nbytes + K * 2 + N * 2 + 64,
                    desc="NF4 blockwise 4-bit GEMV 11008x4096, blocksize 64, fp16 in/out")
    if name == "nf4_dequant":
        N, K, bs = 11008, 4096, 64
        A, B, absmax, lut = synth.nf4_case(N, K, bs, seed)
        return dict(N=N, K=K, bs=bs, B=B, absmax=absmax, lut=lut,
                    bytes=B.nbytes + absmax.nbytes + N * K * 2,
                    desc="NF4 blockwise dequantize 11008x4096 -> fp16")
    if name in ("q3_gemv_f32", "q3_gemv_f16"):
        K, W = (4096, 4096)
        if os.environ.get("HQ_BENCH_Q3_SHAPE") == "opt175b":
            K, W = 49152, 12288
        vec, codes, sc, z = synth.q3_case(K, W, seed)
        return dict(K=K, W=W, vec=vec, codes=codes, sc=sc, z=z,
                    bytes=K * 3 // 32 * W * 4 + 3 * 4 * W + 4 * K,
                    desc=f"GPTQ 3-bit GEMV {K}x{W}")
    if name == "bnb_quantize":
        n = 1 << 24
        A = np.random.Generator(np.random.PCG64([seed, 50])).standard_normal(n).astype(np.float32)
        return dict(n=n, A=A, bytes=n * 5, desc="bitsandbytes 8-bit kQuantize, 16777216 fp32")
    if name == "lutgemm":
        M = K = 12288
        x, bW, alpha, qb = synth.lutgemm_case(M, K, 3, 128, seed)
        return dict(M=M, K=K, x=x, bW=bW, alpha=alpha, qb=qb,
                    bytes=bW.nbytes + alpha.nbytes + qb.nbytes + 2 * K + 2 * M,
                    desc="LUT-GEMM nqmv 12288x12288, 3 bit planes, group 128")
    if name == "aqlm_1x16":
        m = k = 4096
        codes, x, cb, scales = synth.aqlm_1x16_case(m, k, 1, seed)
        return dict(m=m, k=k, codes=codes, x=x, cb=cb, scales=scales,
                    bytes=codes.nbytes + cb.nbytes + 3 * 8192,
                    desc="AQLM 1x16 mat-vec 4096x4096 (packed bytes; 16-byte gathers go through L2)")
    if name == "aqlm_2x8":
        m = k = 4096
        codes, x, cbs, scales = synth.aqlm_2x8_case(m, k, seed)
        return dict(m=m, k=k, codes=codes, x=x, cbs=cbs, scales=scales,
                    bytes=codes.nbytes + 4 * 8192, desc="AQLM 2x8 mat-vec 4096x4096")
    if name == "qgemm_q3":
        Mb, K, N = 64, 8192, 28672
        if os.environ.get("HQ_BENCH_QGEMM_SHAPE") == "down":
            K, N = 28672, 8192
        X, codes, scales, zeros = synth.qgemm_q3_case(Mb, K, N, 128, seed)
        return dict(Mb=Mb, K=K, N=N, X=X, codes=codes, scales=scales, zeros=zeros,
                    bytes=K * 3 // 32 * N * 4 + 2 * (K // 128) * N * 2 + Mb * K * 2 + Mb * N * 2,
                    flops=2.0 * Mb * K * N,
                    desc=f"batched dequant-GEMM, 3-bit g128, X[{Mb}x{K}] x W[{K}x{N}] (Llama-3-70B MLP)")
    if name == "qgemm_nf4":
        Mb, K, N, bs = 64, 8192, 28672, 64
        if os.environ.get("HQ_BENCH_QGEMM_SHAPE") == "down":
            K, N = 28672, 8192
        X, B, absmax, lut = synth.qgemm_nf4_case(Mb, K, N, bs, seed)
        return dict(Mb=Mb, K=K, N=N, bs=bs, X=X, B=B, absmax=absmax, lut=lut,
                    bytes=B.nbytes + absmax.nbytes + Mb * K * 2 + Mb * N * 2 + 64,
                    flops=2.0 * Mb * K * N,
                    desc=f"batched dequant-GEMM, NF4 blocksize 64, X[{Mb}x{K}] x W[{K}x{N}] "
                         "(Llama-3-70B MLP)")
    raise SystemExit(f"unknown workload {name}")


# Weights are resident model state: the NF4 GEMV may fetch them while the preceding
# launch of the stream is finishing (HQ_BENCH_NO_PDL=1 turns that off).
PDL = os.environ.get("HQ_BENCH_NO_PDL") != "1"

WORKLOADS = ["nf4_gemv", "nf4_dequant", "q3_gemv_f32", "q3_gemv_f16", "bnb_quantize", "lutgemm",
             "aqlm_1x16", "aqlm_2x8", "qgemm_q3", "qgemm_nf4"]
DTYPE = {"nf4_gemv": "f16", "nf4_dequant": "f16", "q3_gemv_f32": "f32", "q3_gemv_f16": "f16",
         "bnb_quantize": "u8", "lutgemm": "f16", "aqlm_1x16": "f16", "aqlm_2x8": "f16",
         "qgemm_q3": "f16", "qgemm_nf4": "f16"}


class DeviceWorkload:
    """R replicas of one workload on one GPU, launched through the C ABI."""

    def __init__(self, name: str, dev, seed: int, target_bytes: float):
        import torch
        import hecbench_b200 as hq
        self.hq, self.torch, self.name, self.dev = hq, torch, name, dev
        c = _host_case(name, seed)
        self.case = c
        self.bytes = int(c["bytes"])
        self.R = max(2, int(np.ceil(target_bytes / self.bytes)))
        t = lambda a: torch.from_numpy(np.ascontiguousarray(
            a.view(np.int32) if a.dtype == np.uint32 else a)).to(dev)
        R = self.R
        rot = lambda a, i: np.roll(a.reshape(-1), 4099 * i).reshape(a.shape) if i else a
        if name in ("nf4_gemv", "nf4_dequant"):
            self.B = [t(rot(c["B"], i)) for i in range(R)]
            self.absmax = [t(rot(c["absmax"], i)) for i in range(R)]
            self.lut = t(c["lut"])
            if name == "nf4_gemv":
                self.x = [t(c["A"]) for _ in range(R)]
                self.out = [torch.empty(c["N"], dtype=torch.float16, device=dev) for _ in range(R)]
            else:
                self.W = torch.empty(c["N"] * c["K"], dtype=torch.float16, device=dev)
        elif name.startswith("q3_gemv"):
            from hecbench_b200 import synth
            mat = synth.q3_pack(c["codes"])
            self.height = mat.shape[0]
            self.mat = [t(rot(mat, i)) for i in range(R)]
            self.sc, self.z = t(c["sc"]), t(c["z"])
            v = c["vec"] if name == "q3_gemv_f32" else c["vec"].astype(np.float16)
            self.x = [t(v) for _ in range(R)]
            self.out = [torch.zeros(c["W"], dtype=torch.float32, device=dev) for _ in range(R)]
        elif name == "bnb_quantize":
            g = np.load(ROOT / "tests" / "golden" / "bnb_golden.npz")
            self.code = t(g["code"])
            self.A = [t(rot(c["A"], i)) for i in range(R)]
            self.outq = torch.empty(c["n"], dtype=torch.uint8, device=dev)
        elif name == "lutgemm":
            self.w = [hq.nQWeight_fp16(rot(c["bW"], i), c["alpha"].astype(np.float32), c["K"],
                                       c["M"], 3, False, c["K"] // 128,
                                       c["qb"].astype(np.float32), device=dev) for i in range(R)]
            self.x = [t(c["x"]) for _ in range(R)]
            self.out = [torch.empty(c["M"], dtype=torch.float16, device=dev) for _ in range(R)]
        elif name == "aqlm_1x16":
            self.codes = [t(rot(c["codes"], i).view(np.int16)) for i in range(R)]
            self.cb = t(c["cb"])
            self.x = [t(c["x"]) for _ in range(R)]
            self.out = [torch.empty(c["m"], dtype=torch.float16, device=dev) for _ in range(R)]
        elif name == "qgemm_q3":
            from hecbench_b200 import synth
            mat = synth.q3_pack(c["codes"])
            self.mat = [t(rot(mat, i)) for i in range(R)]
            self.sc, self.z = t(c["scales"]), t(c["zeros"])
            self.x = [t(c["X"]) for _ in range(R)]
            self.out = [torch.empty((c["Mb"], c["N"]), dtype=torch.float16, device=dev)
                        for _ in range(R)]
        elif name == "qgemm_nf4":
            self.B = [t(rot(c["B"], i)) for i in range(R)]
            self.absmax, self.lut = t(c["absmax"]), t(c["lut"])
            self.x = [t(c["X"]) for _ in range(R)]
            self.out = [torch.empty((c["Mb"], c["N"]), dtype=torch.float16, device=dev)
                        for _ in range(R)]
        elif name == "aqlm_2x8":
            self.codes = [t(rot(c["codes"], i)) for i in range(R)]
            self.cbs = t(c["cbs"])
            self.x = [t(c["x"]) for _ in range(R)]
            self.out = [torch.empty(c["m"], dtype=torch.float16, device=dev) for _ in range(R)]

    def launch(self, i: int):
        hq, c, n = self.hq, self.case, self.name
        if n == "nf4_gemv":
            hq.gemv_nf4(self.x[i], self.B[i], self.absmax[i], self.lut, c["N"], c["K"], c["bs"], 0,
                        self.out[i], weights_resident=PDL)
        elif n == "nf4_dequant":
            hq.dequantize_nf4(self.B[i], self.absmax[i], self.lut, c["N"] * c["K"], c["bs"], 0,
                              self.W)
        elif n == "q3_gemv_f32":
            hq.vecquant3matmul(self.x[i], self.mat[i], self.out[i], self.sc, self.z, self.height,
                               c["W"])
        elif n == "q3_gemv_f16":
            hq.vecquant3matmul_faster(self.x[i], self.mat[i], self.out[i], self.sc, self.z,
                                      self.height, c["W"])
        elif n == "bnb_quantize":
            hq.kQuantize(self.code, self.A[i], self.outq, c["n"])
        elif n == "lutgemm":
            hq.matmul(self.out[i], self.x[i], self.w[i])
        elif n == "aqlm_1x16":
            m = c["m"]
            hq.code1x16_matvec(self.codes[i], self.x[i], self.out[i], self.cb, m, c["k"],
                               [m, m, m, 1 << 30], 65536)
        elif n == "aqlm_2x8":
            hq.code2x8_matvec(self.codes[i], self.x[i], self.out[i], self.cbs, c["m"], c["k"])
        elif n == "qgemm_q3":
            hq.qgemm_q3(self.x[i], self.mat[i], self.sc, self.z, c["N"], c["K"], 128,
                        out=self.out[i])
        elif n == "qgemm_nf4":
            hq.qgemm_nf4(self.x[i], self.B[i], self.absmax, self.lut, c["N"], c["K"], c["bs"], 0,
                         out=self.out[i])

    # host <-> device traffic of one launch on the end-to-end path
    def host_io(self):
        """(pinned host input, device input list, device output list) or None."""
        torch = self.torch
        if not hasattr(self, "x") or not hasattr(self, "out"):
            return None
        hin = [torch.empty_like(self.x[i], device="cpu").pin_memory().copy_(self.x[i])
               for i in range(self.R)]
        hout = [torch.empty_like(self.out[i], device="cpu").pin_memory() for i in range(self.R)]
        return hin, hout

    def check_one(self):
        """One replica against the CPU oracle (cheap sanity guard before timing)."""
        from oracle import oracle as O
        c = self.case
        if self.name != "nf4_gemv":
            return None
        self.launch(0)
        self.torch.cuda.synchronize()
        y = self.out[0].cpu().numpy().astype(np.float64)
        rows = 512
        ref = O.nf4_gemv_f64(c["A"], c["B"][:rows * c["K"] // 2], c["absmax"], c["lut"], rows,
                             c["K"], c["bs"], 0)
        return O.rel_err(y[:rows], ref)


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([f.strip() for f in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
                for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                    "sw_power_cap"], r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_baseline(name: str, budget_s: float = 12.0):
    """Oracle port (or the reference's own CPU build for kQuantize) on a bounded
    sample of the workload, all host threads."""
    from oracle import oracle as O
    c = _host_case(name, 0)
    threads = O.num_threads()
    kind = "port"
    if name == "nf4_gemv":
        rows = c["N"]
        fn = lambda: O.nf4_gemv_f32(c["A"], c["B"], c["absmax"], c["lut"], rows, c["K"], c["bs"], 0)
        sample = f"full {c['N']}x{c['K']} GEMV, fp32 accumulate"
    elif name == "nf4_dequant":
        fn = lambda: O.nf4_dequant_f16(c["B"], c["absmax"], c["lut"], c["N"] * c["K"], c["bs"], 0)
        sample = "full dequantize"
    elif name.startswith("q3_gemv"):
        mat = O.q3_pack(c["codes"])
        zero = np.zeros(c["W"], dtype=np.float32)
        fn = lambda: O.q3_gemv_f32(c["vec"], mat, zero, c["sc"], c["z"])
        sample = "full GEMV, reference fp32 order"
    elif name == "bnb_quantize":
        g = np.load(ROOT / "tests" / "golden" / "bnb_golden.npz")
        if O.ref_cpu() is not None:
            kind = "reference"
            threads = os.cpu_count() or 1
            fn = lambda: O.ref_bnb_quantize(c["A"])
        else:
            fn = lambda: O.bnb_quantize(g["code"], c["A"])
        sample = "full 16777216 elements"
    elif name == "lutgemm":
        cols = 1536
        bW = np.ascontiguousarray(c["bW"][:, :, :cols])
        al = np.ascontiguousarray(c["alpha"][:, :, :cols])
        qb = np.ascontiguousarray(c["qb"][:, :cols])
        fn = lambda: O.lutgemm_gemv_f32(c["x"], bW, al, qb, cols, c["K"], 3, 128)
        sample = f"{cols} of {c['M']} output columns"
        c = dict(c, bytes=c["bytes"] * cols / c["M"])
    elif name == "aqlm_1x16":
        m = c["m"]
        fn = lambda: O.aqlm_1x16_f32(c["codes"], c["x"], c["cb"], m, c["k"], [m, m, m, 1 << 30],
                                     65536)
        sample = "full mat-vec"
    elif name == "aqlm_2x8":
        m = c["m"]
        fn = lambda: O.aqlm_2x8_f64(c["codes"], c["x"], c["cbs"], m, c["k"])
        sample = "full mat-vec (fp64 oracle)"
    elif name == "qgemm_q3":
        cols = 128
        mat = np.ascontiguousarray(O.q3_pack(c["codes"])[:, :cols])
        sc, z = (np.ascontiguousarray(c[k][:, :cols]) for k in ("scales", "zeros"))
        fn = lambda: O.gemm_f16_f64(c["X"], O.q3g_dequant_f16(mat, sc, z, c["K"], cols, 128))
        sample = f"{cols} of {c['N']} output features (dequantise + fp64 product), one thread"
        threads = 1
        c = dict(c, bytes=c["bytes"] * cols / c["N"])
    elif name == "qgemm_nf4":
        cols = 128
        B = c["B"][:cols * c["K"] // 2]
        fn = lambda: O.gemm_f16_nk_f64(
            c["X"], O.nf4_dequant_f16(B, c["absmax"], c["lut"], cols * c["K"], c["bs"],
                                      0).reshape(cols, c["K"]))
        sample = f"{cols} of {c['N']} output features (dequantise + fp64 product), one thread"
        threads = 1
        c = dict(c, bytes=c["bytes"] * cols / c["N"])
    else:
        raise SystemExit(f"no CPU baseline for {name}")
    fn()
    t0 = time.perf_counter(); reps = 0
    while True:
        fn(); reps += 1
        el = time.perf_counter() - t0
        if el > budget_s or reps >= 20000:
            break
    per = el / reps
    return {"value": c["bytes"] / per / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
            "sample": f"{sample}; {reps} repetitions in {el:.1f} s", "us_per_call": per * 1e6}


def cpu_baseline_clean(name: str):
    """cpu_baseline in a fresh interpreter (no CUDA context, no helper threads of
    this process competing for the host cores), all host threads."""
    env = dict(os.environ, OMP_NUM_THREADS=str(os.cpu_count() or 1))
    code = ("import json, sys; sys.path.insert(0, %r); import bench; "
            "print(json.dumps(bench.cpu_baseline(%r)))" % (str(ROOT), name))
    try:
        out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True,
                             text=True, timeout=300, check=True).stdout
        return json.loads(out.strip().splitlines()[-1])
    except Exception:
        return cpu_baseline(name)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1; the CPU arm uses every host thread
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    name = args.workload
    c = _host_case(name, 0)
    # each step = one bounded CPU sample (a few repetitions of the workload)
    per_step_budget = max(0.5, min(6.0, 60.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_baseline(name, budget_s=per_step_budget / 4)
    vals, t0 = [], time.perf_counter()
    last = None
    for _ in range(args.steps):
        last = cpu_baseline(name, budget_s=per_step_budget)
        vals.append(last["value"])
    el = time.perf_counter() - t0
    v = float(np.mean(vals))
    line = {
        "impl": "reference", "metric": "effective_weight_bandwidth", "value": v, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": el / max(1, args.steps) * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": DTYPE[name], "data": "synthetic",
        "config": {"workload": c["desc"], "host_threads": last["cores"]},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": last["cores"], "kind": last["kind"],
                         "sample": last["sample"]},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="nf4_gemv", choices=WORKLOADS)
    ap.add_argument("--replica-bytes", type=float, default=640e6,
                    help="bytes of packed weights resident per GPU (>> L2)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly (for profilers)")
    ap.add_argument("--gather", default="publish", choices=["publish", "fused", "nccl"],
                    help="N > 1: how the output slices of a layer are gathered")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    import hecbench_b200 as hq

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU: there is no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    hq.load_library()

    wl = DeviceWorkload(args.workload, dev, seed=rank, target_bytes=args.replica_bytes)
    R = wl.R
    err = wl.check_one()
    if err is not None and err > 1e-2:
        raise SystemExit(f"parity guard failed before timing: rel err {err}")

    # N > 1: every rank holds its output-feature shard of each of the R layers
    # (weak scaling: the layer grows with N) and the slices of every layer are
    # all-gathered over NCCL right after its kernel, as a decoder needs them.
    gathered = None
    peer = None
    if world > 1 and args.workload == "nf4_gemv" and args.gather in ("publish", "fused"):
        # fused GEMV + gather: the kernel stores its slice into every GPU's
        # gathered vector over NVLink and flags it; a bounded wait follows
        from hecbench_b200.shard import FeatureShard, PeerGather
        c = wl.case
        peer = PeerGather(FeatureShard(rank, world, world * c["N"]), slots=R, device=dev)
    elif world > 1 and hasattr(wl, "out"):
        gathered = [torch.empty(world * wl.out[i].numel(), dtype=wl.out[i].dtype, device=dev)
                    for i in range(R)]

    def layer(i):
        if peer is not None:
            c = wl.case
            if args.gather == "fused":
                # the GEMV's last CTA sends the slice itself; bounded wait after it
                peer.gemv_nf4(i, wl.x[i], wl.B[i], wl.absmax[i], wl.lut, c["K"], c["bs"])
            else:
                # ordinary GEMV into this rank's slice of its own gathered vector,
                # then one small kernel: peer stores over NVLink, flags, bounded wait
                hq.gemv_nf4(wl.x[i], wl.B[i], wl.absmax[i], wl.lut, c["N"], c["K"], c["bs"], 0,
                            peer.local_slice(i), weights_resident=PDL)
                peer.publish(i)
            return
        wl.launch(i)
        if gathered is not None:
            dist.all_gather_into_tensor(gathered[i], wl.out[i].view(-1))

    stream = torch.cuda.Stream()
    graph = None
    with torch.cuda.stream(stream):
        for i in range(R):
            layer(i)
        stream.synchronize()
        if not args.no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for i in range(R):
                        layer(i)
            except Exception as exc:  # NCCL capture not available: launch eagerly
                print(f"[bench] graph capture failed ({exc}); running eagerly", file=sys.stderr)
                graph = None
                torch.cuda.synchronize()

    def step():
        if graph is not None:
            graph.replay()
        else:
            for i in range(R):
                layer(i)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    with torch.cuda.stream(stream):
        for _ in range(max(3, args.warmup)):
            step()
        barrier()
        if sampler:
            sampler.start()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    if world > 1:
        tt = torch.tensor([ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())

    # ceiling of a kernel with this footprint: pure streaming read of the same
    # number of bytes per launch over the same rotating buffers, same graph setup
    read_us = None
    if args.workload == "nf4_gemv" and world == 1:
        lib = hq.load_library()
        sink = torch.zeros(1, dtype=torch.int32, device=dev)
        nbytes = wl.B[0].numel()
        with torch.cuda.stream(stream):
            def reads():
                for i in range(R):
                    lib.hq_probe_stream_read(wl.B[i].data_ptr(), nbytes, sink.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream)
            reads()
            stream.synchronize()
            rg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(rg, stream=stream):
                reads()
            for _ in range(3):
                rg.replay()
            ra = torch.cuda.Event(enable_timing=True); rb = torch.cuda.Event(enable_timing=True)
            ra.record(stream)
            for _ in range(min(args.steps, 100)):
                rg.replay()
            rb.record(stream)
            stream.synchronize()
            read_us = ra.elapsed_time(rb) * 1e3 / (R * min(args.steps, 100))

    launches = R * args.steps
    us_per_launch = ms * 1e3 / launches
    total_bytes = wl.bytes * launches * world
    value = total_bytes / (ms * 1e-3) / 1e9

    # ---- end to end: host activations in, host results out, every launch ----
    e2e = None
    io = wl.host_io()
    if io is not None:
        hin, hout = io
        with torch.cuda.stream(stream):
            # The R launches of a pass are independent requests (own input, weights
            # and output), so they run as a few parallel chains: one request's copies
            # overlap another's kernel, as in a serving loop with requests in flight.
            chains = [torch.cuda.Stream() for _ in range(min(4, R))] if world == 1 else []

            def e2e_one(i):
                wl.x[i].copy_(hin[i], non_blocking=True)
                layer(i)
                if peer is not None:  # this rank's slice of the gathered vector
                    c = wl.case
                    hout[i].copy_(peer.slot(i)[rank * c["N"]:(rank + 1) * c["N"]],
                                  non_blocking=True)
                else:
                    hout[i].copy_(wl.out[i], non_blocking=True)

            def e2e_pass():
                if not chains:
                    for i in range(R):
                        e2e_one(i)
                    return
                for cs in chains:
                    cs.wait_stream(stream)
                for i in range(R):
                    with torch.cuda.stream(chains[i % len(chains)]):
                        e2e_one(i)
                for cs in chains:
                    stream.wait_stream(cs)
            # the whole pass (pinned-host -> device copy, kernel, device -> pinned-host
            # copy, per launch) as one CUDA graph, like the device-only leg
            e2e_graph = None
            e2e_pass()
            stream.synchronize()
            if graph is not None:
                try:
                    e2e_graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(e2e_graph, stream=stream):
                        e2e_pass()
                except Exception as exc:
                    print(f"[bench] e2e graph capture failed ({exc}); running eagerly",
                          file=sys.stderr)
                    e2e_graph = None
                    torch.cuda.synchronize()

            def e2e_step():
                if e2e_graph is not None:
                    e2e_graph.replay()
                else:
                    e2e_pass()
            for _ in range(3):
                e2e_step()
            barrier()
            a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(args.steps):
                e2e_step()
            b.record(stream)
            barrier()
            ems = a.elapsed_time(b)
        if world > 1:
            tt = torch.tensor([ems], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ems = float(tt.item())
        e2e = {"value": total_bytes / (ems * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": int(sum(h.numel() * h.element_size() for h in hin)),
               "d2h_bytes_per_step": int(sum(h.numel() * h.element_size() for h in hout)),
               "us_per_call": ems * 1e3 / launches,
               "launch": ("cuda graph of R x (H2D copy, kernel, D2H copy)" if e2e_graph is not None
                          else "eager") + (f", {len(chains)} requests in flight" if chains else "")}

    if peer is not None and int(peer.status.item()) != 0:
        raise SystemExit("a bounded gather wait ran out")
    if rank == 0:
        peak, peak_src = measured_peak()
        achieved = wl.bytes / (us_per_launch * 1e-6) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": f"of {peak_src}",
                "traffic": ncu_traffic(args.workload), "same_size_pure_read_us": read_us}
        if "flops" in wl.case:
            # batch 64: 14.7 us of HBM time against 18.2 us of tensor time -> tensor bound
            tpeak, tsrc = measured_tensor_peak()
            tf = wl.case["flops"] / (us_per_launch * 1e-6) / 1e12
            roof = {"bound": "tensor", "achieved": tf, "peak": tpeak, "unit": "TFLOP/s",
                    "frac": tf / tpeak, "peak_source": f"of {tsrc}",
                    "traffic": ncu_traffic(args.workload), "hbm_frac": achieved / peak}
        line = {
            "metric": "effective_weight_bandwidth", "value": value, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": DTYPE[args.workload], "data": "synthetic",
            "config": {"workload": wl.case["desc"], "replicas_per_gpu": R,
                       "resident_weight_bytes_per_gpu": wl.bytes * R,
                       "l2": "inputs larger than L2 (replicas rotate, R x bytes >> 126 MB)",
                       "algorithmic_bytes_per_launch": wl.bytes,
                       "launch": ("cuda graph of R launches" if graph is not None else "eager") +
                                 ("; weights flagged resident: a launch fetches its weights while "
                                  "the previous launch's tail drains (programmatic dependent launch)"
                                  if PDL and args.workload == "nf4_gemv" else ""),
                       "parallelism": ("single GPU" if world == 1 else
                                       f"output features sharded over {world} GPUs, " +
                                       (f"gather '{args.gather}': slices stored into every GPU's "
                                        "gathered vector by our own kernel (peer stores over "
                                        "NVLink + flags), bounded wait after every layer"
                                        if peer is not None else
                                        "NCCL all-gather of the slices after every layer"))},
            "us_per_gemv": us_per_launch,
            "roofline": roof,
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_clean(args.workload)
        print(json.dumps(line), flush=True)
    if world > 1:
        # Tearing the NCCL communicator down after its collectives were captured in
        # a CUDA graph blocked forever on this stack; the ranks agree that they are
        # done and leave without the teardown.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
