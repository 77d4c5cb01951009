#!/usr/bin/env python
"""Benchmark of the quantized mat-vec hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME]
                  [--impl ours|reference|refgpu] [--scaling weak|strong] [--gather FORM]

One "step" is P passes of the workload's kernel over R independent packed
weight replicas (R layers of a decoder, back to back, one CUDA graph per pass);
R is chosen so that R x bytes is several times the 126 MB L2, so every launch
streams its weights from HBM, and P so that a step lasts about 10 ms.  Rank 0
prints ONE JSON line:

  value      effective weight GB/s over all ranks = algorithmic bytes / time,
             inputs resident in HBM, CUDA-event timed, max over ranks
  e2e        same metric through the C ABI with HOST activations: every launch
             copies its input vector from pinned host memory and its output
             back (weights are model state and stay resident)
  roofline   achieved GB/s of the kernel (algorithmic bytes per launch / mean
             launch duration inside the timed region) against the measured HBM
             copy bandwidth of MEASURED_PEAKS.json (and against the 8 TB/s
             spec figure)
  workloads  N = 1, headline workload only: every other workload of the family,
             each timed the same way in a short loop, with the reference's own
             CUDA kernel compiled for sm_100a beside it (`ref_kernel_us`, from
             a separate process: `--impl refgpu`) and the CPU oracle time
  cpu_baseline  the CPU oracle port of the same workload timed on a bounded
             sample on this box's host cores (rank 0, N = 1 only)

N > 1 (one process per GPU under torchrun): `--scaling weak` (default) gives
every rank its own shard of a layer N times wider and gathers the output
slices after every layer; `--scaling strong` (batched workloads) splits the
one layer's output features over the ranks.  After the timed loops every rank
checks its gathered results against the CPU oracle (`gather_check`).

`--impl reference` times the reference algorithm's CPU implementation (the
reference's own build for kQuantize, the oracle port otherwise) on the same
workload with all host threads.  `--impl refgpu` times the reference's CUDA
kernels (oracle/_ref/ref_gpu_bench).
"""
from __future__ import annotations

import argparse
import ctypes
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
SPEC_HBM_GBS = 8000.0


def _peak(key, fallback):
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())[key]), "measured"
        except Exception:
            pass
    return fallback, "fallback"


def measured_peak():
    return _peak("hbm_gbs", FALLBACK_HBM_GBS)


def measured_tensor_peak():
    """Dense bf16 cuBLAS throughput measured on this pool (burst figure: the
    kernel is timed in a short graph, not inside a seconds-long step)."""
    return _peak("bf16_tflops", FALLBACK_BF16_TFLOPS)


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
# workloads: name -> host arrays + metadata
# --------------------------------------------------------------------------

def _host_case(name: str, seed: int, Mb: int = 64):
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
    if name in ("q3_gemv_f32", "q3_gemv_f16", "q3_gemv_f32_opt175b", "q3_gemv_f16_opt175b"):
        K, W = (49152, 12288) if name.endswith("opt175b") else (4096, 4096)
        vec, _, sc, z = synth.q3_case(32, W, seed)
        vec = synth._rng(seed, 2).standard_normal(K).astype(np.float32)
        mat = synth.q3_words(K, W, seed)
        return dict(K=K, W=W, vec=vec, mat=mat, sc=sc, z=z,
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
                    bytes=codes.nbytes + cb.nbytes + 3 * 8192, gather_bytes=m * k // 8 * 16,
                    desc="AQLM 1x16 mat-vec 4096x4096 (packed bytes; 16-byte gathers go through L2)")
    if name == "aqlm_2x8":
        m = k = 4096
        codes, x, cbs, scales = synth.aqlm_2x8_case(m, k, seed)
        return dict(m=m, k=k, codes=codes, x=x, cbs=cbs, scales=scales,
                    bytes=codes.nbytes + 4 * 8192, desc="AQLM 2x8 mat-vec 4096x4096")
    if name in ("vllm_static_f16", "vllm_dynamic_f16", "vllm_dynamic_azp_f16"):
        tokens, hidden = 4096, 5137  # the reference's own run (quantVLLM-cuda/Makefile:57)
        x = (synth._rng(seed, 60).integers(0, 1000, (tokens, hidden)) - 300).astype(np.float16)
        return dict(tokens=tokens, hidden=hidden, x=x, bytes=tokens * hidden * 3 + tokens * 8,
                    desc=f"per-token int8 activation quantization {tokens}x{hidden} fp16 "
                         f"({name[5:-4].replace('_', ' ')})")
    if name in ("gemv_int8", "gemv_int4"):
        size = 8192  # square, as in the reference driver (its default 512 is 256 KB: all launch)
        bits = 8 if name == "gemv_int8" else 4
        mat, vec = synth.gemv_uniform_case(size, size, bits, seed)
        return dict(size=size, bits=bits, mat=mat, vec=vec, scale=0.0625, zp=0.01,
                    bytes=mat.nbytes + 4 * size,
                    desc=f"uniform int{bits} weight-only GEMV {size}x{size} (gemv-cuda), fp16 in/out")
    if name in ("fused_nf4_swiglu", "fused_int8_swiglu", "fused_int4_swiglu"):
        # entry of a Llama-3-8B MLP at batch 1: RMSNorm(4096) -> interleaved up/gate
        # rows [2 * 14336][4096] -> SwiGLU, one launch
        n, rows_out = 4096, 14336
        rng = synth._rng(seed, 70)
        x = (rng.standard_normal(n) * 2).astype(np.float16)
        gamma = rng.uniform(0.5, 1.5, n).astype(np.float16)
        fmt = name.split("_")[1]
        if fmt == "nf4":
            _, B, absmax, lut = synth.nf4_case(2 * rows_out, n, 64, seed)
            extra = dict(mat=B.reshape(2 * rows_out, n // 2), absmax=absmax, lut=lut)
            nbytes = B.nbytes + absmax.nbytes + 64
        else:
            mat, _ = synth.gemv_uniform_case(2 * rows_out, n, int(fmt[3:]), seed)
            extra = dict(mat=mat, scale=0.02, zp=0.5)
            nbytes = mat.nbytes
        return dict(n=n, rows_out=rows_out, fmt=fmt, x=x, gamma=gamma, **extra,
                    bytes=nbytes + 4 * n + 2 * rows_out,
                    desc=f"RMSNorm -> {fmt} up/gate mat-vec [{2 * rows_out}x{n}] -> SwiGLU, one "
                         "launch (Llama-3-8B MLP entry, batch 1)")
    if name in ("mxfp4_qdq_f16", "mxfp4_quantize_f16"):
        numel = 1 << 26  # 128 MB of fp16 per launch (the reference's own run has 2^29 elements)
        x = (synth._rng(seed, 80).standard_normal(numel, dtype=np.float32) * 3).astype(np.float16)
        pack = name == "mxfp4_quantize_f16"
        return dict(numel=numel, x=x, pack=pack,
                    bytes=numel * 2 + (numel // 2 + numel // 32 if pack else numel * 2),
                    desc=f"MXFP4 {'packer' if pack else 'quantize-dequantize'} of {numel} fp16 values "
                         "(mxfp4-cuda)")
    if name in ("q3_quantize", "bcq_quantize"):
        K, N = 12288, 12288  # the LUT-GEMM workload's layer; one square projection of the 3-bit one
        W = (synth._rng(seed, 84).standard_normal((K, N), dtype=np.float32) * 0.02).astype(np.float16)
        if name == "bcq_quantize":
            return dict(K=K, N=N, W=W,
                        bytes=K * N * 2 + K // 32 * 3 * N * 4 + K // 128 * 4 * N * 2,
                        desc=f"greedy binary-coding quantizer, {K}x{N} fp16 weights, 3 planes, "
                             "groups of 128")
        return dict(K=K, N=N, W=W, bytes=2 * K * N * 2 + K * 3 // 32 * N * 4 + 8 * N,
                    desc=f"3-bit round-to-nearest quantizer and packer, {K}x{N} fp16 weights "
                         "(two passes over the weights)")
    if name == "nf4_quantize":
        N, K, bs = 11008, 4096, 64
        W = (synth._rng(seed, 83).standard_normal(N * K, dtype=np.float32) * 0.02).astype(np.float16)
        return dict(n=N * K, bs=bs, W=W, lut=synth.nf4_levels(seed),
                    bytes=N * K * 2 + N * K // 2 + N * K // bs * 4,
                    desc="blockwise 4-bit quantizer, 11008x4096 fp16 weights, blocksize 64")
    if name == "zero_point":
        size = 1 << 24  # the reference's own run has 10^7 channels
        lo = synth._rng(seed, 81).uniform(-1, 1, size).astype(np.float32)
        hi = synth._rng(seed, 82).uniform(-1, 1, size).astype(np.float32)
        return dict(size=size, lo=lo, hi=hi, bytes=size * 16,
                    desc=f"scale / zero point of {size} channels from min / max, int8 symmetric "
                         "(zeropoint-cuda)")
    if name in ("qgemm_q3", "qgemm_q3_down"):
        K, N = (28672, 8192) if name.endswith("down") else (8192, 28672)
        G = K // 128
        X = synth._rng(seed, 52).standard_normal((Mb, K)).astype(np.float16)
        scales = synth._rng(seed, 53).uniform(0.001, 0.01, (G, N)).astype(np.float16)
        zeros = (scales.astype(np.float32) *
                 synth._rng(seed, 54).integers(0, 8, (G, N))).astype(np.float16)
        mat = synth.q3_words(K, N, seed)
        return dict(Mb=Mb, K=K, N=N, X=X, mat=mat, scales=scales, zeros=zeros,
                    bytes=K * 3 // 32 * N * 4 + 2 * G * N * 2 + Mb * K * 2 + Mb * N * 2,
                    flops=2.0 * Mb * K * N,
                    desc=f"batched dequant-GEMM, 3-bit g128, X[{Mb}x{K}] x W[{K}x{N}] (Llama-3-70B MLP)")
    if name in ("qgemm_nf4", "qgemm_nf4_down"):
        bs = 64
        K, N = (28672, 8192) if name.endswith("down") else (8192, 28672)
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

WORKLOADS = ["nf4_gemv", "nf4_dequant", "q3_gemv_f32", "q3_gemv_f16", "q3_gemv_f32_opt175b",
             "q3_gemv_f16_opt175b", "bnb_quantize", "lutgemm", "aqlm_1x16", "aqlm_2x8",
             "qgemm_q3", "qgemm_nf4", "qgemm_q3_down", "qgemm_nf4_down",
             "vllm_static_f16", "vllm_dynamic_f16", "vllm_dynamic_azp_f16",
             "gemv_int8", "gemv_int4", "fused_nf4_swiglu", "fused_int8_swiglu",
             "fused_int4_swiglu", "mxfp4_qdq_f16", "mxfp4_quantize_f16", "zero_point",
             "nf4_quantize", "q3_quantize", "bcq_quantize"]


def dtype_of(name: str) -> str:
    if name.startswith("vllm"):
        return "i8"
    if name.startswith("mxfp4"):
        return "fp4"
    if name == "zero_point":
        return "f64"
    return "f32" if name.startswith("q3_gemv_f32") else ("u8" if name == "bnb_quantize" else "f16")


class DeviceWorkload:
    """R replicas of one workload on one GPU, launched through the C ABI.
    `shard` (FeatureShard) keeps only this rank's output features of each
    replica (strong scaling)."""

    def __init__(self, name: str, dev, seed: int, target_bytes: float, Mb: int = 64, shard=None):
        import torch
        import hecbench_b200 as hq
        self.hq, self.torch, self.name, self.dev, self.shard = hq, torch, name, dev, shard
        c = _host_case(name, seed, Mb)
        self.case = c
        self.bytes = int(c["bytes"])
        local_bytes = self.bytes / (shard.world if shard else 1)
        self.R = max(2, int(np.ceil(target_bytes / local_bytes)))
        t = lambda a: torch.from_numpy(np.ascontiguousarray(
            a.view(np.int32) if a.dtype == np.uint32 else a)).to(dev)
        R = self.R
        rot = lambda a, i: np.roll(a.reshape(-1), 4099 * i).reshape(a.shape) if i else a
        rows = (lambda a: shard.rows(a)) if shard else (lambda a: a)
        cols = (lambda a: shard.cols(a)) if shard else (lambda a: a)
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
            self.height = c["mat"].shape[0]
            self.mat = [t(rot(c["mat"], i)) for i in range(R)]
            self.sc, self.z = t(c["sc"]), t(c["z"])
            v = c["vec"] if name.startswith("q3_gemv_f32") else c["vec"].astype(np.float16)
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
        elif name.startswith("qgemm_q3"):
            self.n_local = c["N"] // (shard.world if shard else 1)
            self.mat = [t(cols(rot(c["mat"], i))) for i in range(R)]
            self.sc, self.z = t(cols(c["scales"])), t(cols(c["zeros"]))
            self.x = [t(c["X"]) for _ in range(R)]
            self.out = [torch.empty((c["Mb"], self.n_local), dtype=torch.float16, device=dev)
                        for _ in range(R)]
        elif name.startswith("qgemm_nf4"):
            self.n_local = c["N"] // (shard.world if shard else 1)
            Bm = c["B"].reshape(c["N"], c["K"] // 2)
            am = c["absmax"].reshape(c["N"], c["K"] // c["bs"])
            self.B = [t(rows(rot(Bm, i)).reshape(-1)) for i in range(R)]
            self.absmax, self.lut = t(rows(am).reshape(-1)), t(c["lut"])
            self.x = [t(c["X"]) for _ in range(R)]
            self.out = [torch.empty((c["Mb"], self.n_local), dtype=torch.float16, device=dev)
                        for _ in range(R)]
        elif name.startswith("gemv_int"):
            self.mat = [t(rot(c["mat"], i)) for i in range(R)]
            self.x = [t(c["vec"]) for _ in range(R)]
            self.out = [torch.empty(c["size"], dtype=torch.float16, device=dev) for _ in range(R)]
        elif name.startswith("fused_"):
            self.mat = [t(rot(c["mat"], i)) for i in range(R)]
            self.gamma = t(c["gamma"])
            if c["fmt"] == "nf4":
                self.absmax = [t(rot(c["absmax"], i)) for i in range(R)]
                self.lut = t(c["lut"])
            self.x = [t(c["x"]) for _ in range(R)]
            self.out = [torch.empty(c["rows_out"], dtype=torch.float16, device=dev)
                        for _ in range(R)]
        elif name.startswith("mxfp4"):
            self.xin = [t(rot(c["x"], i)) for i in range(R)]
            self.y = torch.empty(c["numel"], dtype=torch.float16, device=dev)
            self.codes = torch.empty(c["numel"] // 2, dtype=torch.uint8, device=dev)
            self.scales8 = torch.empty(c["numel"] // 32, dtype=torch.uint8, device=dev)
        elif name == "bcq_quantize":
            self.W = [t(rot(c["W"], i)) for i in range(R)]
        elif name == "q3_quantize":
            self.W = [t(rot(c["W"], i)) for i in range(R)]
            self.mat3 = torch.empty((c["K"] * 3 // 32, c["N"]), dtype=torch.int32, device=dev)
            self.sc3 = torch.empty(c["N"], dtype=torch.float32, device=dev)
            self.z3 = torch.empty(c["N"], dtype=torch.float32, device=dev)
        elif name == "nf4_quantize":
            self.W = [t(rot(c["W"], i)) for i in range(R)]
            self.lut = t(c["lut"])
            self.B = torch.empty(c["n"] // 2, dtype=torch.uint8, device=dev)
            self.absmax = torch.empty(c["n"] // c["bs"], dtype=torch.float32, device=dev)
        elif name == "zero_point":
            self.lo = [t(rot(c["lo"], i)) for i in range(R)]
            self.hi = [t(rot(c["hi"], i)) for i in range(R)]
            self.sc = torch.empty(c["size"], dtype=torch.float32, device=dev)
            self.zp = torch.empty(c["size"], dtype=torch.int32, device=dev)
        elif name.startswith("vllm"):
            self.xin = [t(rot(c["x"], i)) for i in range(R)]
            self.q = torch.empty((c["tokens"], c["hidden"]), dtype=torch.int8, device=dev)
            self.scales = torch.empty(c["tokens"], dtype=torch.float32, device=dev)
            self.azp = torch.empty(c["tokens"], dtype=torch.int32, device=dev)
        elif name == "aqlm_2x8":
            self.codes = [t(rot(c["codes"], i)) for i in range(R)]
            self.cbs = t(c["cbs"])
            self.x = [t(c["x"]) for _ in range(R)]
            self.out = [torch.empty(c["m"], dtype=torch.float16, device=dev) for _ in range(R)]

    def launch(self, i: int, out=None, pdl: bool = PDL, peers=None):
        hq, c, n = self.hq, self.case, self.name
        if n == "nf4_gemv":
            hq.gemv_nf4(self.x[i], self.B[i], self.absmax[i], self.lut, c["N"], c["K"], c["bs"], 0,
                        self.out[i] if out is None else out, weights_resident=pdl)
        elif n == "nf4_dequant":
            hq.dequantize_nf4(self.B[i], self.absmax[i], self.lut, c["N"] * c["K"], c["bs"], 0,
                              self.W)
        elif n.startswith("q3_gemv_f32"):
            hq.vecquant3matmul(self.x[i], self.mat[i], self.out[i], self.sc, self.z, self.height,
                               c["W"])
        elif n.startswith("q3_gemv_f16"):
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
        elif n == "gemv_int8":
            hq.gemv_int8_quantized(self.mat[i], self.x[i], c["scale"], c["zp"], out=self.out[i])
        elif n == "gemv_int4":
            hq.gemv_int4_quantized(self.mat[i], self.x[i], c["scale"], c["zp"], out=self.out[i])
        elif n.startswith("fused_"):
            kw = (dict(absmax=self.absmax[i], lut16=self.lut, blocksize=64) if c["fmt"] == "nf4"
                  else dict(scale=c["scale"], zero_point=c["zp"]))
            if c["fmt"] == "nf4":
                kw["weights_resident"] = pdl
            hq.gemv_fused(c["fmt"], self.x[i], self.mat[i], c["rows_out"], gamma=self.gamma,
                          eps=1e-5, act=hq.ACT_SWIGLU, out=self.out[i], **kw)
        elif n == "mxfp4_qdq_f16":
            hq.mxfp4(self.y, self.xin[i], c["numel"])
        elif n == "mxfp4_quantize_f16":
            hq.mxfp4_quantize(self.xin[i], self.codes, self.scales8)
        elif n == "bcq_quantize":
            hq.quantize_bcq(self.W[i], 3, 128, True)
        elif n == "q3_quantize":
            hq.quantize_q3(self.W[i], self.mat3, self.sc3, self.z3)
        elif n == "nf4_quantize":
            hq.quantize_nf4(self.W[i], self.lut, c["bs"], 0, self.B, self.absmax)
        elif n == "zero_point":
            hq.zero_point(self.lo[i], self.hi[i], -127, 127, c["size"], True, self.sc, self.zp)
        elif n == "vllm_static_f16":
            hq.static_scaled_int8_quant(self.q, self.xin[i], c["hidden"], c["tokens"], 0.1, 0)
        elif n.startswith("vllm_dynamic"):
            hq.dynamic_scaled_int8_quant(self.q, self.xin[i], c["hidden"], c["tokens"],
                                         self.scales, self.azp if "azp" in n else None)
        elif n.startswith("qgemm_q3"):
            hq.qgemm_q3(self.x[i], self.mat[i], self.sc, self.z, self.n_local, c["K"], 128,
                        out=self.out[i] if out is None else out, peers=peers)
        elif n.startswith("qgemm_nf4"):
            hq.qgemm_nf4(self.x[i], self.B[i], self.absmax, self.lut, self.n_local, c["K"], c["bs"],
                         0, out=self.out[i] if out is None else out, peers=peers)

    def launch_unfused(self, i: int, pdl: bool = PDL):
        """The fused workloads as three launches: torch's RMSNorm, the library's plain
        mat-vec over all 2 * rows_out rows, torch's SiLU-and-multiply of the pairs."""
        hq, c, F = self.hq, self.case, self.torch.nn.functional
        xn = F.rms_norm(self.x[i], (c["n"],), self.gamma, 1e-5)
        rows = 2 * c["rows_out"]
        if not hasattr(self, "pairs"):
            self.pairs = self.torch.empty(rows, dtype=self.torch.float16, device=self.dev)
        if c["fmt"] == "nf4":
            hq.gemv_nf4(xn, self.mat[i], self.absmax[i], self.lut, rows, c["n"], 64, 0, self.pairs,
                        weights_resident=pdl)
        elif c["fmt"] == "int8":
            hq.gemv_int8_quantized(self.mat[i], xn, c["scale"], c["zp"], out=self.pairs)
        else:
            hq.gemv_int4_quantized(self.mat[i], xn, c["scale"], c["zp"], out=self.pairs)
        self.torch.mul(F.silu(self.pairs[1::2]), self.pairs[0::2], out=self.out[i])

    # host <-> device traffic of one launch on the end-to-end path
    def host_io(self):
        """(pinned host inputs, pinned host outputs) or None."""
        torch = self.torch
        if not hasattr(self, "x") or not hasattr(self, "out"):
            return None
        hin = [torch.empty_like(self.x[i], device="cpu").pin_memory().copy_(self.x[i])
               for i in range(self.R)]
        hout = [torch.empty_like(self.out[i], device="cpu").pin_memory() for i in range(self.R)]
        return hin, hout

    def oracle_rows(self, i: int, x_half: np.ndarray, rows: int):
        """fp64 oracle of the first `rows` outputs of replica i (NF4 GEMV only)."""
        from oracle import oracle as O
        c = self.case
        B = self.B[i].cpu().numpy()[:rows * c["K"] // 2]
        am = self.absmax[i].cpu().numpy()[:rows * c["K"] // c["bs"]]
        return O.nf4_gemv_f64(x_half, B, am, c["lut"], rows, c["K"], c["bs"], 0)

    def check_one(self):
        """One replica against the CPU oracle (cheap sanity guard before timing)."""
        from oracle import oracle as O
        if self.name != "nf4_gemv":
            return None
        self.launch(0)
        self.torch.cuda.synchronize()
        y = self.out[0].cpu().numpy().astype(np.float64)
        rows = 512
        return O.rel_err(y[:rows], self.oracle_rows(0, self.case["A"], rows))


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
    full_bytes = float(c["bytes"])
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
        cols = min(c["W"], 4096)
        mat = np.ascontiguousarray(c["mat"][:, :cols])
        zero = np.zeros(cols, dtype=np.float32)
        fn = lambda: O.q3_gemv_f32(c["vec"], mat, zero, c["sc"][:cols], c["z"][:cols])
        sample = f"{cols} of {c['W']} output columns, reference fp32 order"
        c = dict(c, bytes=c["bytes"] * cols / c["W"])
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
    elif name.startswith("gemv_int"):
        fn = lambda: O.gemv_uniform_f64(c["mat"], c["vec"], c["bits"], c["scale"], c["zp"])
        sample = "full mat-vec (fp64 oracle)"
    elif name.startswith("vllm"):
        if name == "vllm_static_f16":
            fn = lambda: O.vllm_static_quant(c["x"], "float16", 0.1, 0)
        else:
            fn = lambda: O.vllm_dynamic_quant(c["x"], "float16", "azp" in name)
        sample = "full tensor"
    elif name.startswith("qgemm_q3"):
        cols = 128
        mat = np.ascontiguousarray(c["mat"][:, :cols])
        sc, z = (np.ascontiguousarray(c[k][:, :cols]) for k in ("scales", "zeros"))
        fn = lambda: O.gemm_f16_f64(c["X"], O.q3g_dequant_f16(mat, sc, z, c["K"], cols, 128))
        sample = f"{cols} of {c['N']} output features (dequantise + fp64 product)"
        c = dict(c, bytes=c["bytes"] * cols / c["N"])
    elif name.startswith("qgemm_nf4"):
        cols = 128
        B = c["B"][:cols * c["K"] // 2]
        fn = lambda: O.gemm_f16_nk_f64(
            c["X"], O.nf4_dequant_f16(B, c["absmax"], c["lut"], cols * c["K"], c["bs"],
                                      0).reshape(cols, c["K"]))
        sample = f"{cols} of {c['N']} output features (dequantise + fp64 product)"
        c = dict(c, bytes=c["bytes"] * cols / c["N"])
    elif name.startswith("fused_"):
        rows = 1024  # output pairs of the sample
        kw = (dict(absmax=c["absmax"][:2 * rows * c["n"] // 64], lut16=c["lut"], blocksize=64)
              if c["fmt"] == "nf4" else dict(scale=c["scale"], zero_point=c["zp"]))
        mat = np.ascontiguousarray(c["mat"][:2 * rows])
        fn = lambda: O.gemv_fused_f64(c["fmt"], mat, c["x"], c["gamma"], 1e-5, rows, 1, **kw)
        sample = f"{rows} of {c['rows_out']} outputs (fp64 oracle)"
        c = dict(c, bytes=c["bytes"] * rows / c["rows_out"])
    elif name.startswith("mxfp4"):
        n = 1 << 22
        xs = np.ascontiguousarray(c["x"][:n]).view(np.uint16)
        fn = (lambda: O.mxfp4_quantize(xs)) if c["pack"] else (lambda: O.mxfp4_qdq(xs))
        sample = f"{n} of {c['numel']} values"
        c = dict(c, bytes=c["bytes"] * n / c["numel"])
    elif name == "zero_point":
        n = 1 << 22
        lo, hi = np.ascontiguousarray(c["lo"][:n]), np.ascontiguousarray(c["hi"][:n])
        if O.ref_zero_point(lo[:8], hi[:8], -127, 127, True) is not None:
            kind, threads = "reference", 1
            fn = lambda: O.ref_zero_point(lo, hi, -127, 127, True)
        else:
            threads = 1
            fn = lambda: O.zero_point(lo, hi, -127, 127, True)
        sample = f"{n} of {c['size']} channels, one thread (the host function is serial)"
        c = dict(c, bytes=c["bytes"] * n / c["size"])
    elif name == "nf4_quantize":
        n = c["n"] // 8
        w = c["W"][:n].astype(np.float32)
        threads = 1
        fn = lambda: O.nf4_quantize(w, c["bs"], c["lut"], 0)
        sample = f"{n} of {c['n']} weights, one thread"
        c = dict(c, bytes=c["bytes"] / 8)
    elif name in ("q3_quantize", "bcq_quantize"):
        cols = 512
        w = np.ascontiguousarray(c["W"][:, :cols]).astype(np.float32)
        fn = (lambda: O.q3_quantize(w)) if name == "q3_quantize" else \
            (lambda: O.lutgemm_quantize(w, 3, 128, True))
        sample = f"{cols} of {c['N']} output columns"
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
    full_us = per * 1e6 * full_bytes / c["bytes"]  # a sampled time scaled to the whole call
    return {"value": c["bytes"] / per / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
            "sample": f"{sample}; {reps} repetitions in {el:.1f} s", "us_per_call": per * 1e6,
            "us_per_full_call": full_us}


def _subprocess_json(code_or_cmd, env=None, timeout=600):
    out = subprocess.run(code_or_cmd, env=env, capture_output=True, text=True, timeout=timeout,
                         check=True).stdout
    return json.loads(out.strip().splitlines()[-1])


def cpu_baseline_clean(name: str, budget_s: float = 12.0):
    """cpu_baseline in a fresh interpreter (no CUDA context, no helper threads of
    this process competing for the host cores), all host threads."""
    env = dict(os.environ, OMP_NUM_THREADS=str(os.cpu_count() or 1))
    code = ("import json, sys; sys.path.insert(0, %r); import bench; "
            "print(json.dumps(bench.cpu_baseline(%r, %r)))" % (str(ROOT), name, budget_s))
    try:
        return _subprocess_json([sys.executable, "-c", code], env=env, timeout=300)
    except Exception:
        return cpu_baseline(name, budget_s)


def cpu_baselines_clean(names, budget_s: float):
    """Short CPU-oracle timings of several workloads in ONE fresh interpreter."""
    env = dict(os.environ, OMP_NUM_THREADS=str(os.cpu_count() or 1))
    code = ("import json, sys; sys.path.insert(0, %r); import bench; "
            "print(json.dumps({n: bench.cpu_baseline(n, %r) for n in %r}))"
            % (str(ROOT), budget_s, list(names)))
    try:
        return _subprocess_json([sys.executable, "-c", code], env=env, timeout=600)
    except Exception as exc:
        print(f"[bench] CPU baselines of the workloads block failed: {exc}", file=sys.stderr)
        return {}


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
        "vs_baseline": None, "dtype": dtype_of(name), "data": "synthetic",
        "config": {"workload": c["desc"], "host_threads": last["cores"]},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": last["cores"], "kind": last["kind"],
                         "sample": last["sample"]},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def ref_gpu_kernel_times(target_bytes: float):
    """The reference's own CUDA kernels, compiled for sm_100a from their own
    sources, timed by oracle/_ref/ref_gpu_bench in a process of its own (so that
    this process never loads anything built from the reference)."""
    exe = ROOT / "oracle" / "_ref" / "ref_gpu_bench"
    if not exe.exists():
        return {"unavailable": "oracle/_ref/ref_gpu_bench was not built (reference tree absent)"}
    try:
        return _subprocess_json([str(exe), str(target_bytes)], timeout=600)
    except Exception as exc:
        return {"unavailable": f"ref_gpu_bench failed: {exc}"}


def run_refgpu(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    print(json.dumps({"impl": "refgpu", "unit": "us per launch",
                      "protocol": "rotating replicas >> L2, CUDA graph, CUDA events",
                      "ref_kernel_us": ref_gpu_kernel_times(args.replica_bytes)}), flush=True)


def time_replicas(torch, stream, launch, R, replays, warm=3, graph=True):
    """us per launch of `launch(i)`, i = 0..R-1 captured as one CUDA graph."""
    with torch.cuda.stream(stream):
        for i in range(R):
            launch(i)
        stream.synchronize()
        g = None
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(R):
                    launch(i)

        def one():
            if g is not None:
                g.replay()
            else:
                for i in range(R):
                    launch(i)
        for _ in range(warm):
            one()
        a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(replays):
            one()
        b.record(stream)
        stream.synchronize()
        return a.elapsed_time(b) * 1e3 / (replays * R)


def roofline_of(case, us, name):
    peak, peak_src = measured_peak()
    achieved = case["bytes"] / (us * 1e-6) / 1e9
    if "flops" in case:
        # batch 64: 14.7 us of HBM time against 18.2 us of tensor time -> tensor bound
        tpeak, tsrc = measured_tensor_peak()
        tf = case["flops"] / (us * 1e-6) / 1e12
        return {"bound": "tensor", "achieved": tf, "peak": tpeak, "unit": "TFLOP/s",
                "frac": tf / tpeak, "peak_source": f"of {tsrc}", "traffic": ncu_traffic(name),
                "hbm_frac": achieved / peak}
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "frac_of_spec_8tbs": achieved / SPEC_HBM_GBS,
            "peak_source": f"of {peak_src}", "traffic": ncu_traffic(name)}


def workloads_block(torch, dev, stream, target_bytes, skip):
    """Every other workload of the family, each in a short graph loop."""
    out = {}
    plan = [(n, 64) for n in WORKLOADS if n != skip]
    plan += [(n, mb) for n in ("qgemm_q3", "qgemm_nf4") for mb in (16, 32, 128)]
    for name, mb in plan:
        key = name if mb == 64 else f"{name}_m{mb}"
        try:
            wl = DeviceWorkload(name, dev, seed=1, target_bytes=target_bytes, Mb=mb)
            est = time_replicas(torch, stream, wl.launch, wl.R, 2, warm=1)
            replays = int(min(200, max(5, 40e3 / (est * wl.R))))  # about 40 ms
            us = time_replicas(torch, stream, wl.launch, wl.R, replays)
            roof = roofline_of(wl.case, us, name)
            ent = {"us": us, "bound": roof["bound"], "frac": roof["frac"],
                   "achieved": roof["achieved"], "unit": roof["unit"], "replicas": wl.R,
                   "bytes": wl.bytes, "desc": wl.case["desc"]}
            if "gather_bytes" in wl.case:
                ent["gather_gbs"] = wl.case["gather_bytes"] / (us * 1e-6) / 1e9
            out[key] = ent
            del wl
        except Exception as exc:
            out[key] = {"error": str(exc)[:200]}
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "refgpu"])
    ap.add_argument("--workload", default="nf4_gemv", choices=WORKLOADS)
    ap.add_argument("--replica-bytes", type=float, default=640e6,
                    help="bytes of packed weights resident per GPU (>> L2)")
    ap.add_argument("--passes", type=int, default=0,
                    help="graph replays per step (0: as many as make a step last about 10 ms)")
    ap.add_argument("--batch", type=int, default=64, help="tokens of the batched workloads")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-workloads", action="store_true",
                    help="skip the block that times every other workload and the reference kernels")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly (for profilers)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="N > 1: every rank its own shard of an N-times wider layer (weak), or "
                         "the one layer's output features split over the ranks (strong)")
    ap.add_argument("--gather", default=None, choices=["packets", "fused", "publish", "nccl"],
                    help="N > 1: how the output slices of a layer are gathered")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "refgpu":
        return run_refgpu(args)

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
    name = args.workload
    batched = name.startswith("qgemm")
    strong = world > 1 and args.scaling == "strong"
    if strong and not batched:
        raise SystemExit("--scaling strong is wired for the batched workloads (qgemm_*)")
    gather = args.gather or ("packets" if name == "nf4_gemv" else "fused" if batched else "publish")
    if gather == "packets" and name != "nf4_gemv":
        raise SystemExit("--gather packets is the NF4 GEMV's low-latency form")
    if gather == "fused" and not batched:
        raise SystemExit("--gather fused is the batched product's form (tiles stored to all GPUs "
                         "by the epilogue)")
    if world > 1 and not (batched or name == "nf4_gemv"):
        raise SystemExit("N > 1 is wired for nf4_gemv and the batched workloads")

    from hecbench_b200.shard import FeatureShard, PacketGather, PeerGather
    shard = None
    if strong:
        n_total = 8192 if name.endswith("down") else 28672
        shard = FeatureShard(rank, world, n_total, multiple=128)
    # weak scaling: every rank holds a different layer shard (seed = rank); strong:
    # all ranks cut their slice out of the same layer (seed 0)
    wl = DeviceWorkload(name, dev, seed=0 if strong else rank, target_bytes=args.replica_bytes,
                        Mb=args.batch, shard=shard)
    R, c = wl.R, wl.case
    err = wl.check_one()
    if err is not None and err > 1e-2:
        raise SystemExit(f"parity guard failed before timing: rel err {err}")

    # ---- N > 1: gathered outputs ------------------------------------------------
    packets = peer = None
    gathered = None
    stride = 1
    if world > 1:
        if strong:
            gshard = shard
            rows_out = c["Mb"]
        else:
            n_loc = wl.out[0].shape[-1] if hasattr(wl, "out") else 0
            gshard = FeatureShard(rank, world, world * n_loc)
            rows_out = c.get("Mb", 1)
        if gather == "packets":
            packets = PacketGather(gshard, slots=R, device=dev)
            stride = (world * c["N"]) // c["K"]
        elif gather in ("publish", "fused") and hasattr(wl, "out"):
            peer = PeerGather(gshard, slots=R, device=dev, rows=rows_out)
        elif hasattr(wl, "out"):
            gathered = [torch.empty(world * wl.out[i].numel(), dtype=wl.out[i].dtype, device=dev)
                        for i in range(R)]

    def layer(i):
        if packets is not None:
            # every finished row goes as a packet into all GPUs' vector i; layer i > 0
            # takes its input from the packets of layer i - 1 (every stride-th element
            # of the gathered output), as the next layer of a decoder would
            if i == 0:
                packets.gemv_nf4(0, wl.x[0], wl.B[0], wl.absmax[0], wl.lut, c["K"], c["bs"],
                                 weights_resident=PDL)
            else:
                packets.gemv_nf4(i, None, wl.B[i], wl.absmax[i], wl.lut, c["K"], c["bs"],
                                 weights_resident=PDL, a_slot=i - 1, a_stride=stride)
            return
        if peer is not None and gather == "fused":
            # the product's epilogue stores every finished tile into the slice of all
            # GPUs; one small kernel then raises the flags and waits (bounded)
            wl.launch(i, peers=peer.peers(i))
            peer.publish(i, stored=True)
            return
        if peer is not None:
            # ordinary kernel into this rank's slice of its own gathered buffer, then
            # one kernel: peer stores over NVLink, flags, bounded wait
            wl.launch(i, out=peer.local_slice(i))
            peer.publish(i)
            return
        wl.launch(i)
        if gathered is not None:
            dist.all_gather_into_tensor(gathered[i], wl.out[i].view(-1))

    def finish_pass():
        if packets is not None:  # the last layer's gather is waited for explicitly
            packets.unpack(R - 1, out=pk_plain)
    pk_plain = (torch.empty(packets.slot_elems, dtype=torch.float16, device=dev)
                if packets is not None else None)

    stream = torch.cuda.Stream()
    graph = None
    with torch.cuda.stream(stream):
        for i in range(R):
            layer(i)
        finish_pass()
        stream.synchronize()
        if not args.no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for i in range(R):
                        layer(i)
                    finish_pass()
            except Exception as exc:  # NCCL capture not available: launch eagerly
                print(f"[bench] graph capture failed ({exc}); running eagerly", file=sys.stderr)
                graph = None
                torch.cuda.synchronize()

    def one_pass():
        if graph is not None:
            graph.replay()
        else:
            for i in range(R):
                layer(i)
            finish_pass()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # passes per step: a step lasts about 10 ms, so that 20 steps give the clock
    # sampler (20 ms period) ten samples or more
    with torch.cuda.stream(stream):
        one_pass(); stream.synchronize()
        t0 = time.perf_counter()
        for _ in range(3):
            one_pass()
        stream.synchronize()
        est_pass_ms = (time.perf_counter() - t0) / 3 * 1e3
    passes = args.passes or int(min(4096, max(1, round(10.0 / max(est_pass_ms, 1e-3)))))
    if world > 1:
        tp = torch.tensor([passes], device=dev)
        dist.broadcast(tp, 0)
        passes = int(tp.item())

    def step():
        for _ in range(passes):
            one_pass()

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

    launches = R * passes * args.steps
    us_per_launch = ms * 1e3 / launches
    # weak: every rank streams a whole case per launch; strong: the ranks share one
    total_bytes = wl.bytes * launches * (1 if strong else world)
    value = total_bytes / (ms * 1e-3) / 1e9

    # ---- N > 1: the gathered results of this program against the CPU oracle --------
    gather_check = None
    if world > 1 and (packets is not None or peer is not None or gathered is not None):
        gather_check = check_gather(torch, dist, wl, packets, peer, gathered, rank, world, stride,
                                    strong, shard)

    # ---- N > 1: this rank's kernel alone (no gather), max over ranks -----------------
    kernel_only_us = None
    if world > 1 and hasattr(wl, "out"):
        k_us = time_replicas(torch, stream, lambda i: wl.launch(i), R, 20)
        tk = torch.tensor([k_us], device=dev)
        dist.all_reduce(tk, op=dist.ReduceOp.MAX)
        kernel_only_us = float(tk.item())

    # ---- N = 1 extras: isolated launches, pure-read ceiling -----------------------
    read_us = no_pdl_us = unfused_us = None
    if name.startswith("fused_") and world == 1:
        unfused_us = time_replicas(torch, stream, wl.launch_unfused, R, 20)
    if name == "nf4_gemv" and world == 1:
        no_pdl_us = time_replicas(torch, stream, lambda i: wl.launch(i, pdl=False), R, 50)
        probe = ROOT / "hecbench_b200" / "libhq_probe.so"
        if probe.exists():
            plib = ctypes.CDLL(str(probe))
            plib.hq_probe_stream_read.argtypes = [ctypes.c_void_p, ctypes.c_size_t,
                                                  ctypes.c_void_p, ctypes.c_void_p]
            sink = torch.zeros(1, dtype=torch.int32, device=dev)
            nbytes = wl.B[0].numel()
            read_us = time_replicas(
                torch, stream,
                lambda i: plib.hq_probe_stream_read(wl.B[i].data_ptr(), nbytes, sink.data_ptr(),
                                                    torch.cuda.current_stream().cuda_stream),
                R, 50)

    # ---- end to end: host activations in, host results out, every launch ----------
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
                if packets is None or i == 0:
                    wl.x[i].copy_(hin[i], non_blocking=True)
                layer(i)
                if packets is not None:
                    return
                if peer is not None:  # this rank's slice of the gathered buffer
                    hout[i].copy_(peer.local_slice(i), non_blocking=True)
                else:
                    hout[i].copy_(wl.out[i], non_blocking=True)

            def e2e_pass():
                if not chains:
                    for i in range(R):
                        e2e_one(i)
                    if packets is not None:
                        # the chain's result: this rank's slice of the last gathered vector
                        finish_pass()
                        hout[R - 1].copy_(pk_plain[rank * c["N"]:(rank + 1) * c["N"]],
                                          non_blocking=True)
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
                for _ in range(passes):
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
            # latency of ONE request alone: copy in, kernel, copy out, wait
            single_us = None
            if world == 1:
                lat = []
                for k in range(60):
                    i = k % R
                    stream.synchronize()
                    t0 = time.perf_counter()
                    e2e_one(i)
                    stream.synchronize()
                    lat.append((time.perf_counter() - t0) * 1e6)
                single_us = float(np.median(lat[10:]))
        if world > 1:
            tt = torch.tensor([ems], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ems = float(tt.item())
        n_in = R if packets is None else 1
        n_out = R if packets is None else 1
        e2e = {"value": total_bytes / (ems * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": int(passes * sum(h.numel() * h.element_size()
                                                      for h in hin[:n_in])),
               "d2h_bytes_per_step": int(passes * sum(h.numel() * h.element_size()
                                                      for h in hout[:n_out])),
               "us_per_call": ems * 1e3 / launches,
               "single_request_latency_us": single_us,
               "launch": ("cuda graph of R x (H2D copy, kernel, D2H copy)" if e2e_graph is not None
                          else "eager") + (f", {len(chains)} requests in flight" if chains else
                                           (", one chain of R dependent layers: input of layer 0 "
                                            "from the host, last gathered slice back to the host"
                                            if packets is not None else ""))}

    status_bad = any(g is not None and int(g.status.item()) != 0 for g in (packets, peer))
    if status_bad:
        raise SystemExit("a bounded gather wait ran out")
    ok = gather_check is None or gather_check["ranks_ok"] == world
    if rank == 0:
        roof = roofline_of(c, us_per_launch, name)
        if strong:  # per-GPU kernel works on 1/world of the layer
            roof["note"] = "per-GPU share of the layer; achieved is the whole job's rate"
        if read_us is not None:
            roof["same_size_pure_read_us"] = read_us
        par = "single GPU"
        if world > 1:
            how = {"packets": "every finished row stored as an 8-byte {value, epoch} packet into "
                              "every GPU's vector over NVLink by the GEMV itself; the next layer "
                              "reads its input from the packets (bounded waits)",
                   "fused": "every finished 128-feature tile stored into every GPU's gathered "
                            "buffer over NVLink by the product's own epilogue; a one-CTA kernel "
                            "raises the flags and waits (bounded) after every layer",
                   "publish": "slices copied into every GPU's gathered buffer by our own kernel "
                              "(peer stores over NVLink + flags), bounded wait after every layer",
                   "nccl": "NCCL all-gather of the slices after every layer"}[gather]
            if packets is not None and packets.multicast:
                how += ("; each packet is ONE multimem.st through the NVSwitch multicast mapping of "
                        "the vector (HQ_LL_MULTICAST=0: one store per GPU)")
            par = (f"output features sharded over {world} GPUs ({args.scaling} scaling), "
                   f"gather '{gather}': {how}")
        line = {
            "metric": "effective_weight_bandwidth", "value": value, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": dtype_of(name), "data": "synthetic",
            "config": {"workload": c["desc"], "replicas_per_gpu": R,
                       "passes_per_step": passes, "launches_per_step": R * passes,
                       "resident_weight_bytes_per_gpu": int(wl.bytes * R /
                                                            (world if strong else 1)),
                       "l2": "inputs larger than L2 (replicas rotate, R x bytes >> 126 MB)",
                       "algorithmic_bytes_per_launch": wl.bytes,
                       "launch": ("cuda graph of R launches" if graph is not None else "eager") +
                                 ("; weights flagged resident: a launch fetches its weights while "
                                  "the previous launch's tail drains (programmatic dependent launch)"
                                  if PDL and name in ("nf4_gemv", "fused_nf4_swiglu") else ""),
                       "parallelism": par},
            "us_per_gemv": us_per_launch,
            "roofline": roof,
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
        }
        if no_pdl_us is not None:
            line["value_no_pdl"] = wl.bytes / (no_pdl_us * 1e-6) / 1e9
            line["us_per_gemv_no_pdl"] = no_pdl_us
            line["roofline"]["frac_no_pdl"] = line["value_no_pdl"] / roof["peak"]
        if unfused_us is not None:
            line["us_as_three_launches"] = unfused_us  # torch rms_norm, plain mat-vec, torch silu * mul
        if gather_check is not None:
            line["gather_check"] = gather_check
        if kernel_only_us is not None:
            line["kernel_only_us_per_layer"] = kernel_only_us
        if world == 1 and name == "nf4_gemv" and not args.no_workloads:
            del wl
            torch.cuda.empty_cache()
            block = workloads_block(torch, dev, stream, args.replica_bytes, skip=name)
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
            ref = ref_gpu_kernel_times(args.replica_bytes)
            for k, v in ref.items():
                if k in block and isinstance(v, dict):
                    block[k]["ref_kernel_us"] = v.get("us")
                    block[k]["ref_kernel_launch"] = v.get("launch")
            if "unavailable" in ref:
                line["ref_kernel"] = ref
            if not args.no_cpu_baseline:
                cpu = cpu_baselines_clean([n for n in WORKLOADS if n != name and n in block], 1.5)
                for k, v in cpu.items():
                    block[k]["cpu_baseline_us"] = v.get("us_per_full_call")
                    block[k]["cpu_cores"] = v.get("cores")
            line["workloads"] = block
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_clean(name)
        print(json.dumps(line), flush=True)
    if world > 1:
        # Tearing the NCCL communicator down after its collectives were captured in
        # a CUDA graph blocked forever on this stack; the ranks agree that they are
        # done and leave without the teardown.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0 if ok else 1)


def check_gather(torch, dist, wl, packets, peer, gathered, rank, world, stride, strong, shard):
    """Replica 0 and replica R-1 of this rank's gathered results against the CPU
    oracle of the whole (world x wider, or sharded) layer.  For the oracle every
    rank contributes the first rows of its weights of those two replicas."""
    from oracle import oracle as O
    c, R, name = wl.case, wl.R, wl.name
    dev = wl.dev
    worst = 0.0
    rows = 128

    def allgather_np(t):
        out = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(out, t.contiguous())
        return [o.cpu().numpy() for o in out]

    for i in sorted({0, R - 1}):
        if name == "nf4_gemv":
            n_loc = c["N"]
            if packets is not None:
                got = packets.unpack(i, check_epoch=False).cpu().numpy()
                if i == 0:
                    x = None
                else:
                    prev = packets.unpack(i - 1, check_epoch=False).cpu().numpy()
                    x = np.ascontiguousarray(prev[::stride][:c["K"]])
            else:
                got = (peer.slot(i) if peer is not None else gathered[i]).cpu().numpy()
                x = None
            # weak scaling: rank r computed its slice from ITS input vector (and table)
            xs = allgather_np(wl.x[i])
            luts = allgather_np(wl.lut)
            Bs = allgather_np(wl.B[i][:rows * c["K"] // 2])
            As = allgather_np(wl.absmax[i][:rows * c["K"] // c["bs"]])
            for r in range(world):
                xr = xs[r] if (x is None or i == 0) else x
                ref = O.nf4_gemv_f64(xr, Bs[r], As[r], luts[r], rows, c["K"], c["bs"], 0)
                worst = max(worst, O.rel_err(
                    got[r * n_loc:r * n_loc + rows].astype(np.float64), ref))
        elif name.startswith("qgemm"):
            Mb, K = c["Mb"], c["K"]
            n_loc = wl.n_local
            if peer is not None:
                got = peer.slot(i).cpu().numpy()  # [G][Mb][n_loc]
            else:
                got = gathered[i].view(world, Mb, n_loc).cpu().numpy()
            Xs = allgather_np(wl.x[i])
            if name.startswith("qgemm_q3"):
                mats = allgather_np(wl.mat[i][:, :rows])
                scs = allgather_np(wl.sc[:, :rows]); zs = allgather_np(wl.z[:, :rows])
                for r in range(world):
                    W16 = O.q3g_dequant_f16(np.ascontiguousarray(mats[r]),
                                            np.ascontiguousarray(scs[r]),
                                            np.ascontiguousarray(zs[r]), K, rows, 128)
                    ref = O.gemm_f16_f64(Xs[r], W16)
                    worst = max(worst, O.rel_err(got[r][:, :rows].astype(np.float64), ref))
            else:
                Bs = allgather_np(wl.B[i][:rows * K // 2])
                As = allgather_np(wl.absmax[:rows * K // c["bs"]])
                luts = allgather_np(wl.lut)
                for r in range(world):
                    W16 = O.nf4_dequant_f16(Bs[r], As[r], luts[r], rows * K, c["bs"],
                                            0).reshape(rows, K)
                    ref = O.gemm_f16_nk_f64(Xs[r], W16)
                    worst = max(worst, O.rel_err(got[r][:, :rows].astype(np.float64), ref))
        else:
            return None
    ok = torch.tensor([1 if worst < 1e-2 else 0], device=dev)
    dist.all_reduce(ok)
    w = torch.tensor([worst], device=dev)
    dist.all_reduce(w, op=dist.ReduceOp.MAX)
    return {"max_rel_err": float(w.item()), "ranks_ok": int(ok.item()),
            "checked": f"replicas 0 and {R - 1}, first {rows} output features of every rank's "
                       "slice, on every rank's own gathered copy, against the fp64 CPU oracle"}


if __name__ == "__main__":
    main()
