"""Output-feature sharding of one quantized layer over the GPUs of a node.

Every output feature of the mat-vec family is independent, so a layer is split
by output features: rank r of G owns features [r*N/G, (r+1)*N/G).  For the
row-major [N][K] formats (NF4, AQLM codes) that is a contiguous row range of
the packed matrix; for the column-major formats (quant3MatMul `mat`, LUT-GEMM
bit planes, whose last axis is the output feature) it is a column slab of every
packed row.  Inputs are replicated; the only exchange is one all-gather of the
output slices (NCCL over NVLink when the tensors are on GPUs).  K is never
split, so no reduction is needed.

The compute is injected (`local_fn`): on GPUs it is one of the libhq launchers;
the CPU tests of the partition / gather logic pass the oracle instead.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Tuple

import numpy as np
import torch
import torch.distributed as dist


@dataclass(frozen=True)
class FeatureShard:
    rank: int
    world: int
    n_total: int
    multiple: int = 1  # slice boundaries are multiples of this (kernel tile width)

    def __post_init__(self):
        if self.n_total % (self.world * self.multiple) != 0:
            raise ValueError(
                f"{self.n_total} output features do not split into {self.world} slices "
                f"of a multiple of {self.multiple}")

    @property
    def n_local(self) -> int:
        return self.n_total // self.world

    @property
    def begin(self) -> int:
        return self.rank * self.n_local

    @property
    def end(self) -> int:
        return self.begin + self.n_local

    def rows(self, packed_row_major):
        """Slice of a packed [N][...] matrix (NF4 bytes, AQLM codes, per-row scales)."""
        return packed_row_major[self.begin:self.end]

    def cols(self, packed_col_major):
        """Slab of a packed [...][N] matrix (q3 `mat`, LUT-GEMM planes, per-column params)."""
        return packed_col_major[..., self.begin:self.end]

    def nf4_absmax(self, absmax, K: int, blocksize: int):
        """absmax entries of this rank's rows (rows must start on block boundaries)."""
        if (self.n_local * K) % blocksize != 0:
            raise ValueError("a slice must hold a whole number of absmax blocks")
        per = self.n_local * K // blocksize
        return absmax[self.rank * per:(self.rank + 1) * per]


def gather_features(local_out: torch.Tensor, shard: FeatureShard, group=None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather of the last-axis output slices into [..., n_total]."""
    if shard.world == 1:
        return local_out
    lead = local_out.shape[:-1]
    if out is None:
        out = torch.empty(shard.world, *lead, shard.n_local, dtype=local_out.dtype,
                          device=local_out.device)
    dist.all_gather_into_tensor(out.view(-1), local_out.contiguous().view(-1), group=group)
    if len(lead) == 0:
        return out.view(shard.n_total)
    # [G][..., n_local] -> [..., G*n_local]
    return out.movedim(0, -2).reshape(*lead, shard.n_total)


def sharded_apply(local_fn: Callable[[], torch.Tensor], shard: FeatureShard, group=None):
    """Run the rank-local kernel and gather the feature slices."""
    return gather_features(local_fn(), shard, group)
