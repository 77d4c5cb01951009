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


class PeerGather:
    """Buffers for the fused GEMV + all-gather: every rank's gathered vectors and
    flag words live in peer-mapped ("symmetric") device memory, so the kernel of
    one GPU stores its output slice directly into the vectors of all GPUs over
    NVLink and announces it with one flag word per (receiver, sender).

    Layout of each rank's symmetric buffer: [256 bytes of flags][slots] with
    slot = world * n_local fp16 values.  `sync` is a rank-local pair of words
    (CTA counter, launch count) and `status` a rank-local error word.
    """

    def __init__(self, shard: FeatureShard, slots: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.shard, self.slots = shard, slots
        self.slot_elems = shard.world * shard.n_local
        nbytes = 256 + slots * self.slot_elems * 2
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        grp = group if group is not None else dist.group.WORLD
        self.handle = symm_mem.rendezvous(self.buf, grp.group_name)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        # device arrays of pointers: flag arrays and data regions of every rank
        self.peer_flags = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self.peer_data = torch.tensor([p + 256 for p in ptrs], dtype=torch.int64, device=device)
        self.sync = torch.zeros(2, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=grp)

    def slot(self, i: int) -> torch.Tensor:
        """This rank's copy of gathered vector i (fp16 [world * n_local])."""
        off = 256 + i * self.slot_elems * 2
        return self.buf[off:off + self.slot_elems * 2].view(torch.float16)

    def gemv_nf4(self, i: int, A, B, absmax, lut16, K: int, blocksize: int = 64,
                 nibble_order: int = 0, wait: bool = True, wait_previous: bool = False) -> None:
        """Fused NF4 GEMV of this rank's rows into gathered vector i of every rank.

        wait: enqueue the bounded wait for THIS gather right after the kernel.
        wait_previous: let the kernel wait, before it reads A, for the gather of
        the previous fused call (a layer's input is the previous layer's gathered
        output); the caller then only needs `wait_all()` after the last layer."""
        from ._lib import check, load_library
        lib = load_library()
        sh = self.shard
        stream = torch.cuda.current_stream().cuda_stream
        off = i * self.slot_elems + sh.rank * sh.n_local
        check("hq_nf4_gemv_f16_gather", lib.hq_nf4_gemv_f16_gather(
            A.data_ptr(), B.data_ptr(), absmax.data_ptr(), lut16.data_ptr(), sh.n_local, K,
            blocksize, nibble_order, self.peer_data.data_ptr(), off, self.peer_flags.data_ptr(),
            self.sync.data_ptr(), sh.world, sh.rank,
            self.buf.data_ptr() if wait_previous else 0, self.status.data_ptr(), stream))
        if wait:
            check("hq_gather_wait", lib.hq_gather_wait(
                self.buf.data_ptr(), self.sync.data_ptr(), sh.world, self.status.data_ptr(),
                stream))

    def wait_all(self) -> None:
        """Bounded wait until the slices of the latest fused call have landed here."""
        from ._lib import check, load_library
        check("hq_gather_wait", load_library().hq_gather_wait(
            self.buf.data_ptr(), self.sync.data_ptr(), self.shard.world, self.status.data_ptr(),
            torch.cuda.current_stream().cuda_stream))

    def local_slice(self, i: int) -> torch.Tensor:
        """This rank's own slice inside its copy of gathered vector i: an ordinary
        kernel writes its outputs here, then `publish(i)` sends them to the peers."""
        sh = self.shard
        return self.slot(i)[sh.rank * sh.n_local:(sh.rank + 1) * sh.n_local]

    def publish(self, i: int) -> None:
        """Copy the local slice of vector i to all peers, flag it, and wait (bounded)
        for the peers' slices of the same round."""
        from ._lib import check, load_library
        sh = self.shard
        check("hq_gather_publish", load_library().hq_gather_publish(
            self.peer_data.data_ptr(), i * self.slot_elems + sh.rank * sh.n_local, sh.n_local,
            self.peer_flags.data_ptr(), self.sync.data_ptr(), sh.world, sh.rank,
            self.status.data_ptr(), torch.cuda.current_stream().cuda_stream))
