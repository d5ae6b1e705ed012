"""All-gather of the shards of a sequence-parallel tensor as peer stores.

At the exit of every parallelised transformer forward the reference reassembles the output with
``get_complete_tensor`` = transpose -> contiguous -> NCCL all_gather -> transpose
(src/para_attn/primitives.py:139-148). Here every rank stores its shard straight into its place
inside every rank's result buffer (``pa_cp_push``: 16-byte peer stores over NVLink plus one
release per CTA on an arrival counter there) and then waits, bounded and in stream order, until
all shards have arrived in its own (``pa_flag_wait``). No transposes, no collective library
call; the buffers live in a symmetric-memory workspace that is allocated once per group and
grown on demand, double-buffered by call parity like the attention staging (a rank can be at
most one call ahead of any other, because each call waits for every rank's shard).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib as L
from . import _status
from . import config

_ALIGN = 1024
_CTAS = 8  # pushing CTAs per destination: a transformer output shard is a few MB at most


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def plan_blocks(shape, dim: int, esz: int) -> Optional[Tuple[int, int, int]]:
    """(outer blocks, rows per block, row width in 16-bit units) of a contiguous shard whose copies
    are concatenated along ``dim``, or None when a block is not a whole number of 128- or
    256-byte rows (the copy kernel moves such rows)."""
    dim = dim % len(shape)
    outer = 1
    for s in shape[:dim]:
        outer *= s
    block_bytes = esz
    for s in shape[dim:]:
        block_bytes *= s
    for width in (128, 64):  # in 16-bit units: rows of 256 or 128 bytes
        if block_bytes % (width * 2) == 0 and block_bytes > 0:
            return outer, block_bytes // (width * 2), width
    return None


class PeerGather:
    def __init__(self, group: dist.ProcessGroup, device: torch.device):
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world <= L.PA_MAX_CHUNKS, f"at most {L.PA_MAX_CHUNKS} ranks per group"
        self.capacity = 0
        self.buf: Optional[torch.Tensor] = None
        self.peer = []
        self.calls = 0
        self.expect = [0, 0]
        self.status: Optional[_status.StatusMirror] = None

    def _ensure(self, result_bytes: int) -> None:
        if result_bytes <= self.capacity:
            return
        import torch.distributed._symmetric_memory as symm_mem

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer stores only
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # nobody may still be writing into the old buffer
        cap = _round_up(result_bytes, _ALIGN)
        total = 2 * cap + 256
        buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        buf.zero_()
        hdl = symm_mem.rendezvous(buf, self.group)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.capacity, self.buf, self.hdl = cap, buf, hdl
        self.peer = [int(p) for p in hdl.buffer_ptrs]
        self.calls, self.expect = 0, [0, 0]
        self.status = _status.StatusMirror(buf[2 * cap + 128:2 * cap + 132].view(torch.int32))

    def gather(self, shard: torch.Tensor, dim: int) -> Optional[torch.Tensor]:
        """The shards of all ranks concatenated along ``dim`` (a fresh contiguous tensor), or None
        when this shape cannot take the peer-store path."""
        shard = shard.contiguous()
        esz = shard.element_size()
        blocks = plan_blocks(tuple(shard.shape), dim, esz)
        if blocks is None or shard.data_ptr() % 16:
            return None
        outer, rows, width = blocks
        shard_bytes = shard.numel() * esz
        self._ensure(shard_bytes * self.world)
        self.status.check()
        par = self.calls & 1
        self.calls += 1
        self.expect[par] += self.world * _CTAS
        cap = self.capacity
        stream = torch.cuda.current_stream(self.device).cuda_stream
        block_units = rows * width                  # one block of my shard, in 16-bit units
        pa = L.CpPushArgs()
        for d in range(self.world):
            j = pa.jobs[d]
            j.src = shard.data_ptr()
            # my block b goes behind the blocks of the ranks before me inside result block b
            j.dst = self.peer[d] + par * cap + self.rank * block_units * 2
            j.src_stride[0], j.src_stride[1], j.src_stride[2] = block_units, block_units, width
            j.dst_stride[0], j.dst_stride[1], j.dst_stride[2] = block_units * self.world, block_units, width
            j.head0, j.heads, j.batch, j.rows = 0, 1, outer, rows
            j.dest, j.head_dim = d, width
            pa.flag[d] = self.peer[d] + 2 * cap + 64 * par
        pa.n_jobs, pa.n_dest, pa.ctas_per_dest, pa.first_dest = self.world, self.world, _CTAS, self.rank
        L.check(L.load().pa_cp_push(C.byref(pa), stream))
        flags = (C.c_void_p * 1)(self.peer[self.rank] + 2 * cap + 64 * par)
        L.check(L.load().pa_flag_wait(flags, 1, self.expect[par], self.status.word.data_ptr(),
                                      config.cp.wait_limit_ns, L.PA_DEV_TIMEOUT_OUT, stream))
        shape = list(shard.shape)
        shape[dim % len(shape)] *= self.world
        n = shard_bytes * self.world
        out = self.buf[par * cap:par * cap + n].view(shard.dtype).view(shape).clone()
        self.status.refresh()
        return out

    def reset(self) -> None:
        if self.buf is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.buf[2 * self.capacity:].zero_()
        self.calls, self.expect = 0, [0, 0]
        self.status.reset()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)


_gathers: Dict[Tuple, PeerGather] = {}


def get_gather(group: dist.ProcessGroup, device: torch.device) -> PeerGather:
    key = (group.group_name if hasattr(group, "group_name") else id(group), device.index)
    g = _gathers.get(key)
    if g is None:
        g = PeerGather(group, device)
        _gathers[key] = g
    return g


def all_gathers():
    return list(_gathers.values())
