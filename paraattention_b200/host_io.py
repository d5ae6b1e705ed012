"""Attention on tensors that live in (pinned) host memory.

``attention_from_host(q, k, v, out=None, ...)`` takes [B, H, S, D] host tensors and returns the
result in host memory. Heads are independent, so the call is pipelined over groups of heads on
three streams: while group g is being computed, group g+1 is on its way in over PCIe and the
result of group g-1 is on its way out (PCIe is full duplex). The whole call then costs about
as much as the slowest of the three legs instead of their sum. With more than one rank each
rank handles its own sequence shard the same way and every group is one context-parallel
attention call (``unified_attn_func`` over the given meshes).

There is no counterpart in the reference, which only takes device tensors; this is the
host-buffer entry point the benchmark's end-to-end figure goes through.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import ops as para_attn_ops

__all__ = ["attention_from_host", "HostAttentionPipeline"]



def _default_groups(heads: int, rows: int, batch: int, multiple_of: int, shard: int, sm_count: int = 148) -> int:
    """How many groups of heads a call is split into; heads per group stay a multiple of
    ``multiple_of`` (the Ulysses size). A CTA covers 256 query rows of one head.

    One GPU: launches of neighbouring groups overlap (two compute streams), so up to 12 groups
    as long as a launch still has 1.5 waves of CTAs. Context parallel: the calls of one rank run
    one after the other and each costs whole rounds of the SMs (148 on a B200), so at most 4 groups, and only
    if splitting adds no more than a tenth to the number of rounds (24 heads on 8 ranks: three
    calls of 128 CTAs are exactly the three rounds of one call of 384)."""
    pairs = (rows + 255) // 256

    def ctas(g):
        return batch * (heads // g // multiple_of) * shard * pairs

    single_gpu = multiple_of * shard == 1
    best = 1
    rounds_1 = -(-ctas(1) // sm_count)
    for g in range(2, (12 if single_gpu else 4) + 1):
        if heads % g or (heads // g) % multiple_of:
            continue
        if single_gpu:
            ok = ctas(g) >= (3 * sm_count) // 2
        else:
            ok = g * -(-ctas(g) // sm_count) <= 1.1 * rounds_1
        if ok:
            best = g
    return best


class HostAttentionPipeline:
    """Streams, events and device staging for ``attention_from_host``; reusable across calls of
    the same shape (the benchmark keeps one)."""

    def __init__(self, device: torch.device):
        self.device = device
        self.s_in = torch.cuda.Stream(device)
        self.s_out = torch.cuda.Stream(device)
        self.s_compute2 = torch.cuda.Stream(device)
        self._bufs = {}

    def _staging(self, q_shape, kv_shape, dtype):
        key = (tuple(q_shape), tuple(kv_shape), dtype)
        if key not in self._bufs:
            self._bufs.clear()
            mk = lambda shp: torch.empty(shp, dtype=dtype, device=self.device)  # noqa: E731
            self._bufs[key] = (mk(q_shape), mk(kv_shape), mk(kv_shape), mk(q_shape))
        return self._bufs[key]

    def run(self, attn: Callable, q_h, k_h, v_h, out_h, groups: int, overlap_launches: bool = True):
        B, H, Sq, D = q_h.shape
        hg = H // groups
        main = torch.cuda.current_stream(self.device)
        # Device staging has the hosts' own layout [B, H, S, D], so that a group of heads of one
        # batch element is one contiguous block on both sides and every transfer is a plain copy.
        qd, kd, vd, od = self._staging(q_h.shape, k_h.shape, q_h.dtype)
        # With two compute streams the last, partly filled wave of one group's launch shares the
        # GPU with the first wave of the next group's (single-GPU calls only: context-parallel
        # calls of one rank must follow each other on one stream).
        compute = [main, self.s_compute2] if overlap_launches and groups > 1 else [main]
        self.s_in.wait_stream(main)    # staging may still be read by the previous call
        self.s_out.wait_stream(main)
        for cs in compute[1:]:
            cs.wait_stream(main)
        arrived = []
        with torch.cuda.stream(self.s_in):
            for g in range(groups):
                hs = slice(g * hg, (g + 1) * hg)
                for b in range(B):
                    qd[b, hs].copy_(q_h[b, hs], non_blocking=True)
                    kd[b, hs].copy_(k_h[b, hs], non_blocking=True)
                    vd[b, hs].copy_(v_h[b, hs], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.s_in)
                arrived.append(ev)
        for g in range(groups):
            hs = slice(g * hg, (g + 1) * hg)
            cs = compute[g % len(compute)]
            cs.wait_event(arrived[g])
            with torch.cuda.stream(cs):
                od[:, hs].copy_(attn(qd[:, hs], kd[:, hs], vd[:, hs]))
            done = torch.cuda.Event()
            done.record(cs)
            self.s_out.wait_event(done)
            with torch.cuda.stream(self.s_out):
                for b in range(B):
                    out_h[b, hs].copy_(od[b, hs], non_blocking=True)
        for cs in compute[1:]:
            main.wait_stream(cs)
        main.wait_stream(self.s_out)   # in stream order the call is complete when the last copy is
        return out_h


_pipelines = {}


def attention_from_host(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                        out: Optional[torch.Tensor] = None, *, is_causal: bool = False,
                        scale: Optional[float] = None, head_groups: Optional[int] = None,
                        ulysses_mesh=None, ring_mesh=None, flat_group=None,
                        device: Optional[torch.device] = None) -> torch.Tensor:
    """softmax(scale q k^T) v for host tensors [B, H, S, D] (pinned memory for the copies to
    overlap), result in ``out`` (host, same shape and dtype as ``query``; allocated pinned when
    None). Work is enqueued on the current stream of ``device``; the result is complete once
    that stream has been synchronised. In a multi-rank run pass the rank's sequence shard and
    the meshes, as for ``unified_attn_func``."""
    from . import primitives as DP
    from .para_attn_interface import unified_attn_func

    assert query.device.type == "cpu" and key.device.type == "cpu" and value.device.type == "cpu", \
        "attention_from_host takes host tensors; use torch.ops.para_attn.attention_forward for device tensors"
    assert query.ndim == 4 and key.ndim == 4 and value.ndim == 4, "query, key and value must be [B, H, S, D]"
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, H, Sq, D = query.shape
    U = DP.get_world_size(ulysses_mesh) if ulysses_mesh is not None else 1
    R = DP.get_world_size(ring_mesh) if ring_mesh is not None else 1
    if out is None:
        out = torch.empty(query.shape, dtype=query.dtype).pin_memory()
    if head_groups is None:
        head_groups = _default_groups(H, Sq, B, U, U,
                                      torch.cuda.get_device_properties(device).multi_processor_count)
    assert H % head_groups == 0 and (H // head_groups) % U == 0, "head_groups must split the heads evenly per rank"
    # a causal mask couples nothing across heads either, so the same grouping applies
    if U * R > 1:
        def attn(q, k, v):
            return unified_attn_func(q, k, v, None, 0.0, is_causal, scale=scale, ulysses_mesh=ulysses_mesh,
                                     ring_mesh=ring_mesh, flat_group=flat_group)
    else:
        def attn(q, k, v):
            return para_attn_ops.attention_forward(q, k, v, is_causal=is_causal, scale=scale)
    pipe = _pipelines.get(device)
    if pipe is None:
        pipe = _pipelines[device] = HostAttentionPipeline(device)
    return pipe.run(attn, query, key, value, out, head_groups, overlap_launches=(U * R == 1))
