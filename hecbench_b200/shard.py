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
from typing import Callable

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


def _symmetric(nbytes: int, device, group):
    """Zeroed peer-mapped buffer of nbytes on every rank; returns (tensor, [base pointers])."""
    import torch.distributed._symmetric_memory as symm_mem
    buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
    buf.zero_()
    grp = group if group is not None else dist.group.WORLD
    handle = symm_mem.rendezvous(buf, grp.group_name)
    ptrs = [int(p) for p in handle.buffer_ptrs]
    torch.cuda.synchronize(device)
    dist.barrier(group=grp)
    return buf, handle, ptrs


class PacketGather:
    """Low-latency gather for the batch-1 path (hq_nf4_gemv_f16_ll): every rank's
    gathered vectors live in peer-mapped ("symmetric") device memory as arrays of
    8-byte packets {fp16 value, epoch}.  The GEMV of one GPU stores each finished
    row straight into the packet vectors of all GPUs over NVLink, and the next
    layer's GEMV reads its input from the packets, waiting (bounded) for each
    until it carries the epoch of the round - no fence, no flag round trip, no
    follow-up kernel.

    `slots` packet vectors of world * n_local packets each; a chain of layers
    must alternate between at least two of them, because a vector may be
    rewritten as soon as the following round is complete on this rank.  `sync`
    is the rank-local pair (CTA counter, epoch of the latest completed round),
    `status` a rank-local word that becomes 1 if a bounded wait ran out.
    """

    def __init__(self, shard: FeatureShard, slots: int, device, group=None, max_polls: int = 0,
                 multicast: bool | None = None):
        """multicast: write every packet with one multimem.st through the NVSwitch
        multicast mapping of the buffer instead of one store per GPU (None: when the
        allocation has such a mapping and HQ_LL_MULTICAST is not 0)."""
        import os
        if slots < 2:
            raise ValueError("a chain of gathers needs at least two packet vectors to alternate")
        self.shard, self.slots, self.max_polls = shard, slots, max_polls
        self.slot_elems = shard.world * shard.n_local
        self.buf, self.handle, ptrs = _symmetric(slots * self.slot_elems * 8, device, group)
        self._ptrs = ptrs
        mc_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0) if shard.world > 1 else 0
        if multicast is None:
            multicast = mc_ptr != 0 and os.environ.get("HQ_LL_MULTICAST", "1") != "0"
        if multicast and mc_ptr == 0:
            raise RuntimeError("this symmetric-memory allocation has no multicast mapping")
        self.multicast = bool(multicast)
        # device arrays holding the multicast address of slot i
        self.mc_ll = [torch.tensor([mc_ptr + i * self.slot_elems * 8], dtype=torch.int64,
                                   device=device) for i in range(slots)] if self.multicast else None
        # device arrays of pointers to every rank's copy of slot i
        self.peer_ll = [torch.tensor([p + i * self.slot_elems * 8 for p in ptrs], dtype=torch.int64,
                                     device=device) for i in range(slots)]
        self.sync = torch.zeros(2, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)

    def packets(self, i: int) -> torch.Tensor:
        """This rank's copy of packet vector i as int32 [n_total][2] (value, epoch)."""
        off = i * self.slot_elems * 8
        return self.buf[off:off + self.slot_elems * 8].view(torch.int32).view(-1, 2)

    def gemv_nf4(self, i: int, A, B, absmax, lut16, K: int, blocksize: int = 64,
                 nibble_order: int = 0, weights_resident: bool = False, a_slot=None,
                 a_stride: int = 1, a_first: int = 0) -> None:
        """NF4 GEMV of this rank's rows; results go as packets into vector i of
        every rank.  Input: the plain fp16 tensor A, or (a_slot given) elements
        a_first, a_first + a_stride, ... of this rank's copy of packet vector
        a_slot - the gathered output of an earlier layer."""
        from ._lib import check, load_library
        lib = load_library()
        sh = self.shard
        flags = nibble_order | (2 if weights_resident else 0) | (4 if self.multicast else 0)
        table = self.mc_ll[i] if self.multicast else self.peer_ll[i]
        a_ll = 0
        if a_slot is not None:
            a_ll = self.buf.data_ptr() + (a_slot * self.slot_elems + a_first) * 8
        check("hq_nf4_gemv_f16_ll", lib.hq_nf4_gemv_f16_ll(
            0 if a_slot is not None else A.data_ptr(), a_ll, a_stride, B.data_ptr(),
            absmax.data_ptr(), lut16.data_ptr(), 0, sh.n_local, K, blocksize, flags,
            table.data_ptr(), sh.rank * sh.n_local, self.sync.data_ptr(), sh.world,
            sh.rank, self.max_polls, self.status.data_ptr(),
            torch.cuda.current_stream().cuda_stream))

    def unpack(self, i: int, out: torch.Tensor | None = None, check_epoch: bool = True):
        """Plain fp16 copy of gathered vector i; with check_epoch it waits (bounded)
        until every packet carries the epoch of the latest completed round."""
        from ._lib import check, load_library
        if out is None:
            out = torch.empty(self.slot_elems, dtype=torch.float16, device=self.buf.device)
        check("hq_ll_unpack", load_library().hq_ll_unpack(
            self.buf.data_ptr() + i * self.slot_elems * 8, self.slot_elems, out.data_ptr(),
            self.sync.data_ptr() if check_epoch else 0, self.max_polls, self.status.data_ptr(),
            torch.cuda.current_stream().cuda_stream))
        return out


class PeerGather:
    """Copy + flag gather for larger slices and for any kernel of the family
    (hq_gather_publish): an ordinary launch writes this rank's slice into its own
    copy of the gathered buffer, then one small kernel copies the slice to every
    peer with 16-byte stores over NVLink, fences, raises one flag word per
    (receiver, sender) and waits (bounded) for the peers' slices of the round.

    Layout of each rank's symmetric buffer: [256 bytes of flags][slots] with
    slot = world * rows * n_local fp16 values laid out [world][rows][n_local]
    (rows = 1 for a mat-vec, the batch for the batched product).  A chain of
    rounds must alternate between at least two slots: a rank that has seen round
    L complete may start storing round L + 1 while a slower rank still reads the
    vector of round L - 1.
    """

    def __init__(self, shard: FeatureShard, slots: int, device, group=None, rows: int = 1,
                 max_polls: int = 0):
        if slots < 2:
            raise ValueError("a chain of gathers needs at least two gathered vectors to alternate")
        self.shard, self.slots, self.rows, self.max_polls = shard, slots, rows, max_polls
        self.slice_elems = rows * shard.n_local
        self.slot_elems = shard.world * self.slice_elems
        self.buf, self.handle, ptrs = _symmetric(256 + slots * self.slot_elems * 2, device, group)
        # device arrays of pointers: flag arrays and data regions of every rank
        self.peer_flags = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self.peer_data = torch.tensor([p + 256 for p in ptrs], dtype=torch.int64, device=device)
        self.sync = torch.zeros(2, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)

    def slot(self, i: int) -> torch.Tensor:
        """This rank's copy of gathered buffer i: fp16 [world][rows][n_local]
        (flattened to [world * n_local] when rows == 1)."""
        off = 256 + i * self.slot_elems * 2
        t = self.buf[off:off + self.slot_elems * 2].view(torch.float16)
        if self.rows == 1:
            return t
        return t.view(self.shard.world, self.rows, self.shard.n_local)

    def local_slice(self, i: int) -> torch.Tensor:
        """This rank's own slice inside its copy of gathered buffer i: an ordinary
        kernel writes its outputs here, then `publish(i)` sends them to the peers."""
        sh = self.shard
        if self.rows == 1:
            return self.slot(i)[sh.rank * sh.n_local:(sh.rank + 1) * sh.n_local]
        return self.slot(i)[sh.rank]

    def _slice_offset(self, i: int) -> int:
        """Element offset of this rank's slice of buffer i inside every rank's data
        region (index arithmetic shared with the C hosts: hq_shard_layout)."""
        import ctypes
        from ._lib import check, load_library
        sh = self.shard
        first = ctypes.c_longlong()
        check("hq_shard_layout", load_library().hq_shard_layout(
            sh.world, self.rows, sh.n_local, self.slots, sh.rank, i, None, ctypes.byref(first), None))
        return first.value

    def peers(self, i: int):
        """(pointer table, element offset, world) of this rank's slice of buffer i on
        every GPU: the `peers` argument of qgemm_q3 / qgemm_nf4, whose epilogue then
        stores each finished tile to all GPUs; follow with publish(i, stored=True)."""
        return (self.peer_data.data_ptr(), self._slice_offset(i), self.shard.world)

    def publish(self, i: int, stored: bool = False) -> None:
        """Copy the local slice of buffer i to all peers, flag it, and wait (bounded)
        for the peers' slices of the same round.  stored=True: the producing kernel
        has stored the slice to the peers itself; only flag and wait."""
        from ._lib import check, load_library
        sh = self.shard
        check("hq_gather_publish", load_library().hq_gather_publish(
            self.peer_data.data_ptr(), self._slice_offset(i), 0 if stored else self.slice_elems,
            self.peer_flags.data_ptr(), self.sync.data_ptr(), sh.world, sh.rank,
            self.max_polls, self.status.data_ptr(), torch.cuda.current_stream().cuda_stream))

    def wait_all(self) -> None:
        """Bounded wait until the slices of the latest round have landed here."""
        from ._lib import check, load_library
        check("hq_gather_wait", load_library().hq_gather_wait(
            self.buf.data_ptr(), self.sync.data_ptr(), self.shard.world, self.max_polls,
            self.status.data_ptr(), torch.cuda.current_stream().cuda_stream))
