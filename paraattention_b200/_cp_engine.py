"""Context-parallel attention over NVLink peer memory: the host side.

Replaces, for one attention call on a (ring x ulysses) mesh, the reference's sequence of
NCCL all_to_all -> per-step SDPA + K/V rotation + out/LSE merge -> all_to_all
(src/para_attn/para_attn_interface.py:52-119, 162-239, 445-479) by

  1. ONE launch of ``pa_cp_attn_fwd`` per rank. Its leading CTAs first store the head-slices
     of the local Q/K/V shard that other ranks need directly into those ranks' staging
     buffers (peer stores over NVLink) and bump arrival counters there; every CTA then
     computes attention, consuming the K/V chunks in arrival order (own shard first) while
     later chunks are still in flight, keeping the running softmax state on chip, and
     writing every output tile straight into the buffer of the rank that owns those rows;
  2. a bounded, stream-ordered wait until all tiles owed to this rank have arrived.

``CpPlan`` is the pure-python description of who sends what where; it is what the CPU tests
exercise. ``CpEngine`` owns the symmetric-memory workspace (allocated once per group and
grown on demand - the kernels themselves never allocate) and issues the launches.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import math
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib as L
from . import _status
from . import config

_ALIGN = 1024


_SM_COUNTS: Dict[int, int] = {}


def _sm_count(device: torch.device) -> int:
    n = _SM_COUNTS.get(device.index)
    if n is None:
        n = torch.cuda.get_device_properties(device).multi_processor_count
        _SM_COUNTS[device.index] = n
    return n


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


@dataclasses.dataclass(frozen=True)
class PushJobSpec:
    tensor: str        # "q", "k" or "v"
    dest: int          # flat rank of the destination
    head0: int         # first head of the slice that is sent
    heads: int
    chunk: int         # chunk slot inside the destination's staging buffer


@dataclasses.dataclass(frozen=True)
class CpPlan:
    """Who sends what where for one rank of a ulysses x ring mesh.

    Flat rank = ring_idx * ulysses + ulysses_idx (ulysses is the fastest mesh dim, as in
    src/para_attn/context_parallel/__init__.py:38-39). Rank (u, r) ends up computing heads
    [u*H/U, (u+1)*H/U) for the query rows of the U ranks of its Ulysses group against the
    keys/values of all W ranks: exactly what ulysses_attn_func around ring_attn_func computes.
    """

    ulysses: int
    ring: int
    u: int
    r: int
    heads: int  # total heads H

    def __post_init__(self):
        assert self.heads % self.ulysses == 0, "h must be divisible by world_size, got {} and {}".format(
            self.heads, self.ulysses)

    @property
    def world(self) -> int:
        return self.ulysses * self.ring

    @property
    def rank(self) -> int:
        return self.r * self.ulysses + self.u

    @property
    def local_heads(self) -> int:
        return self.heads // self.ulysses

    def flat(self, u: int, r: int) -> int:
        return r * self.ulysses + u

    def push_jobs(self, skip_self: bool = False) -> List[PushJobSpec]:
        """Copies this rank owes to every rank. With ``skip_self`` the copies into its own
        staging buffer are left out (the kernel then reads the own shard in place)."""
        hl = self.local_heads
        jobs = []
        for r_d in range(self.ring):
            for u_d in range(self.ulysses):
                dest = self.flat(u_d, r_d)
                if skip_self and dest == self.rank:
                    continue
                # Q only to my Ulysses group (first: a consumer needs it before any key); chunk slot =
                # my ulysses index
                if r_d == self.r:
                    jobs.append(PushJobSpec("q", dest, u_d * hl, hl, self.u))
                # K and V of my shard go to every rank; chunk slot = my flat rank
                jobs.append(PushJobSpec("k", dest, u_d * hl, hl, self.rank))
                jobs.append(PushJobSpec("v", dest, u_d * hl, hl, self.rank))
        return jobs

    def q_sources(self) -> List[int]:
        """Flat rank that fills query chunk slot c of this rank (c = ulysses index of the source)."""
        return [self.flat(c, self.r) for c in range(self.ulysses)]

    def kv_sources(self) -> List[int]:
        return list(range(self.world))

    def out_dest(self, q_chunk: int) -> Tuple[int, int]:
        """(flat rank, head offset) where output rows of query chunk q_chunk are written."""
        return self.flat(q_chunk, self.r), self.u * self.local_heads

    def out_writers(self) -> List[int]:
        """Flat ranks that write tiles into this rank's output buffer."""
        return [self.flat(c, self.r) for c in range(self.ulysses)]


@dataclasses.dataclass
class _Layout:
    """Byte offsets inside one rank's symmetric workspace (identical on every rank)."""

    stage_bytes: int
    off_k: Tuple[int, int]
    off_v: Tuple[int, int]
    off_q: Tuple[int, int]
    off_o: Tuple[int, int]
    off_arrive: Tuple[int, int]
    off_done: Tuple[int, int]
    off_status: int
    total: int


def _make_layout(world: int, ulysses: int, kv_chunk_bytes: int, q_chunk_bytes: int, out_bytes: int) -> _Layout:
    off = 0
    offs = {}
    for name, size in (("k", world * kv_chunk_bytes), ("v", world * kv_chunk_bytes), ("q", ulysses * q_chunk_bytes),
                       ("o", out_bytes)):
        pair = []
        for _ in range(2):
            pair.append(off)
            off += _round_up(size, _ALIGN)
        offs[name] = tuple(pair)
    stage = off
    arrive = (off, off + 64)
    off += 128
    done = (off, off + 64)
    off += 128
    status = off
    off += 64
    return _Layout(stage, offs["k"], offs["v"], offs["q"], offs["o"], arrive, done, status, _round_up(off, _ALIGN))


@dataclasses.dataclass
class Workspace:
    """One rank's view of the exchange buffers: its own buffer and the device addresses of
    every rank's buffer, indexed by plan rank (ring_idx * ulysses + ulysses_idx)."""

    layout: _Layout
    buf: torch.Tensor          # this rank's buffer (uint8)
    peer: List[int]            # base address of each plan rank's buffer as seen from this device
    me: int                    # this rank's plan rank

    @property
    def base(self) -> int:
        return self.peer[self.me]

    def status_tensor(self) -> torch.Tensor:
        off = self.layout.off_status
        return self.buf[off:off + 4].view(torch.int32)


@dataclasses.dataclass
class CallState:
    """Counters that advance identically on every rank with each attention call."""

    calls: int = 0
    arrive_expect: List[int] = dataclasses.field(default_factory=lambda: [0, 0])
    done_expect: List[int] = dataclasses.field(default_factory=lambda: [0, 0])


def _fix(x: torch.Tensor) -> torch.Tensor:
    esz = x.element_size()
    ok = x.stride(-1) == 1 and x.data_ptr() % 16 == 0 and all((x.stride(i) * esz) % 16 == 0 for i in range(3))
    return x if ok else x.contiguous()


def build_push_args(plan: CpPlan, ws: Workspace, par: int, q, k, v, ctas: int,
                    skip_self: bool = True) -> "L.CpPushArgs":
    """Describe the pushes of this rank: which head-slice of q/k/v goes to which rank's buffer.
    By default nothing is copied into the own buffer: the kernel reads the own shard in place."""
    lay = ws.layout
    B, H, sq, D = q.shape
    skv = k.shape[2]
    hl = plan.local_heads
    esz = q.element_size()
    src = {"q": q, "k": k, "v": v}
    rows = {"q": sq, "k": skv, "v": skv}
    chunk_bytes = {"q": B * hl * sq * D * esz, "k": B * hl * skv * D * esz, "v": B * hl * skv * D * esz}
    stage_off = {"q": lay.off_q[par], "k": lay.off_k[par], "v": lay.off_v[par]}
    pa = L.CpPushArgs()
    jobs = plan.push_jobs(skip_self=skip_self)
    assert len(jobs) <= L.PA_MAX_PUSH_JOBS
    for i, js in enumerate(jobs):
        t = src[js.tensor]
        j = pa.jobs[i]
        n_rows = rows[js.tensor]
        j.src = t.data_ptr()
        j.dst = ws.peer[js.dest] + stage_off[js.tensor] + js.chunk * chunk_bytes[js.tensor]
        for d in range(3):
            j.src_stride[d] = t.stride(d)
        j.dst_stride[0], j.dst_stride[1], j.dst_stride[2] = js.heads * n_rows * D, n_rows * D, D
        j.head0, j.heads, j.batch, j.rows = js.head0, js.heads, B, n_rows
        j.dest = js.dest
        j.head_dim = D
    pa.n_jobs = len(jobs)
    pa.n_dest = plan.world
    for d in range(plan.world):
        if skip_self and d == plan.rank:
            continue  # nothing goes to my own buffer, nobody waits for that counter
        # counter slot on the destination = my plan rank (= chunk slot of my K/V there)
        pa.flag[d] = ws.peer[d] + lay.off_arrive[par] + 4 * plan.rank
    pa.ctas_per_dest = ctas
    pa.first_dest = plan.rank  # own buffer first, then the ranks below: rank-1 needs my chunk first
    return pa


def fused_push_ctas(plan: CpPlan, B: int, sq: int, ctas: int, sm_count: int = 148) -> int:
    """How many leading CTAs of the attention grid push (the library applies the same cap)."""
    grid = ((sq + 255) // 256) * plan.local_heads * B * plan.ulysses
    return max(1, min(ctas, grid, sm_count))


def launch_attention(plan: CpPlan, ws: Workspace, par: int, shape, dtype: torch.dtype, skv: int, scale: float,
                     arrive_expect: int, wait_ns: int, stream: int, out_local: Optional[torch.Tensor],
                     push: Optional["L.CpPushArgs"] = None, local_qkv=None, is_causal: bool = False,
                     key_bits: Optional[torch.Tensor] = None, split_ws: Optional[torch.Tensor] = None) -> None:
    """Build the arguments (``build_attention_args``) and launch pa_cp_attn_fwd."""
    a = build_attention_args(plan, ws, par, shape, dtype, skv, scale, arrive_expect, wait_ns, out_local, push,
                             local_qkv, is_causal, key_bits, split_ws)
    L.check(L.load().pa_cp_attn_fwd(C.byref(a), stream))


def build_attention_args(plan: CpPlan, ws: Workspace, par: int, shape, dtype: torch.dtype, skv: int, scale: float,
                         arrive_expect: int, wait_ns: int, out_local: Optional[torch.Tensor],
                         push: Optional["L.CpPushArgs"] = None, local_qkv=None,
                         is_causal: bool = False, key_bits: Optional[torch.Tensor] = None,
                         split_ws: Optional[torch.Tensor] = None) -> "L.CpAttnArgs":
    """Arguments of pa_cp_attn_fwd for this rank. ``out_local`` (ring-only meshes) receives the result in
    place; otherwise tiles go to the owners' output staging buffers. With ``push`` the launch
    also performs this rank's part of the exchange (fused form). ``local_qkv`` = this rank's own
    (q, k, v): its chunk is then read in place instead of from the staging buffer."""
    lay = ws.layout
    B, H, sq, D = shape
    hl = plan.local_heads
    base = ws.base
    a = L.CpAttnArgs()
    a.q_stage, a.k_stage, a.v_stage = base + lay.off_q[par], base + lay.off_k[par], base + lay.off_v[par]
    a.batch, a.heads, a.head_dim, a.dtype = B, hl, D, {torch.bfloat16: L.PA_BF16, torch.float16: L.PA_F16}[dtype]
    a.n_q_chunks, a.q_rows, a.q_first = plan.ulysses, sq, plan.u
    a.n_kv_chunks, a.kv_rows, a.kv_first = plan.world, skv, plan.rank
    a.scale = scale
    if out_local is not None:
        assert plan.ulysses == 1
        a.out[0] = out_local.data_ptr()
        a.o_stride[0], a.o_stride[1], a.o_stride[2] = out_local.stride(0), out_local.stride(1), out_local.stride(2)
        a.out_head_offset = 0
    else:
        for c in range(plan.ulysses):
            dest, _ = plan.out_dest(c)
            a.out[c] = ws.peer[dest] + lay.off_o[par]
            a.done_flag[c] = ws.peer[dest] + lay.off_done[par]
        # destination memory is [B, s, H, D]
        a.o_stride[0], a.o_stride[1], a.o_stride[2] = sq * H * D, D, H * D
        a.out_head_offset = plan.u * hl
    for c, s_plan in enumerate(plan.q_sources()):
        a.q_flag[c] = base + lay.off_arrive[par] + 4 * s_plan
    for c, s_plan in enumerate(plan.kv_sources()):
        a.kv_flag[c] = base + lay.off_arrive[par] + 4 * s_plan
    a.flag_expect = arrive_expect
    a.status = base + lay.off_status
    a.wait_limit_ns = wait_ns
    a.fused_push = C.addressof(push) if push is not None else None
    if local_qkv is not None:
        ql, kl, vl = local_qkv
        a.q_local, a.k_local, a.v_local = ql.data_ptr(), kl.data_ptr(), vl.data_ptr()
        for d in range(3):
            a.q_local_stride[d], a.k_local_stride[d], a.v_local_stride[d] = ql.stride(d), kl.stride(d), vl.stride(d)
        a.local_head_offset = plan.u * hl
        a.local_total_heads = H
    if is_causal:
        # The sequence is sharded in flat-rank order: the Ulysses exchange concatenates the
        # shards of a group in ulysses-index order (src/para_attn/para_attn_interface.py:60-72)
        # and causal ring attention orders blocks by ring index (torch:...:394-437).
        a.is_causal = 1
        for c in range(plan.ulysses):
            a.q_pos[c] = plan.flat(c, plan.r) * sq
        for c in range(plan.world):
            a.kv_pos[c] = c * skv
    if key_bits is not None:
        assert key_bits.shape == (B, plan.world, (skv + 63) // 64) and key_bits.is_contiguous()
        a.key_bits = key_bits.data_ptr()
    # scratch for a split last wave: used by launches without pushers only (the engine's own
    # launches push, and with real peers the split was measured slower: it passes none)
    if split_ws is not None:
        a.workspace, a.workspace_bytes = split_ws.data_ptr(), split_ws.numel()
    return a


def launch_out_wait(ws: Workspace, par: int, done_expect: int, wait_ns: int, stream: int) -> None:
    lay = ws.layout
    flags = (C.c_void_p * 1)(ws.base + lay.off_done[par])
    L.check(L.load().pa_flag_wait(flags, 1, done_expect, ws.base + lay.off_status, wait_ns, 4, stream))


def out_tiles_per_call(plan: CpPlan, B: int, sq: int) -> int:
    """How many CTAs add 1 to this rank's output-arrival counter in one call."""
    return plan.ulysses * ((sq + 255) // 256) * plan.local_heads * B


def stage_sizes(plan: CpPlan, B: int, sq: int, skv: int, D: int, esz: int) -> Tuple[int, int, int]:
    hl = plan.local_heads
    return B * hl * skv * D * esz, B * hl * sq * D * esz, B * sq * plan.heads * D * esz


class CpEngine:
    """Per (flat group, ulysses, ring) state: workspace, peer pointers, counters."""

    def __init__(self, flat_group: dist.ProcessGroup, ulysses: int, ring: int, u: int, r: int, device: torch.device):
        self.group = flat_group
        self.ulysses, self.ring, self.u, self.r = ulysses, ring, u, r
        self.world = ulysses * ring
        assert self.world == dist.get_world_size(flat_group)
        assert self.world <= L.PA_MAX_CHUNKS, f"at most {L.PA_MAX_CHUNKS} ranks per attention group"
        self.device = device
        self.capacity = (0, 0, 0)  # kv_chunk_bytes, q_chunk_bytes, out_bytes
        self.ws: Optional[Workspace] = None
        self.status: Optional[_status.StatusMirror] = None
        self.hdl = None
        self.state = CallState()
        self._launch_cache: Dict[Tuple, Tuple] = {}
        # group rank of mesh coordinate (u, r): the mesh may order ranks differently from r*U+u
        me = torch.tensor([u, r], dtype=torch.int64, device=device)
        coords = [torch.empty_like(me) for _ in range(self.world)]
        dist.all_gather(coords, me, group=flat_group)
        self.group_rank_of_plan = [-1] * self.world
        for i, c in enumerate(coords):
            self.group_rank_of_plan[int(c[1]) * ulysses + int(c[0])] = i
        assert all(g >= 0 for g in self.group_rank_of_plan), "mesh coordinates are not unique"
        assert self.group_rank_of_plan[r * ulysses + u] == dist.get_rank(flat_group)

    def _ensure(self, need: Tuple[int, int, int]) -> None:
        if all(n <= c for n, c in zip(need, self.capacity)):
            return
        import torch.distributed._symmetric_memory as symm_mem

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer stores only
        cap = tuple(max(n, c) for n, c in zip(need, self.capacity))
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # nobody may still be writing into the old workspace
        layout = _make_layout(self.world, self.ulysses, *cap)
        buf = symm_mem.empty(layout.total, dtype=torch.uint8, device=self.device)
        buf.zero_()
        hdl = symm_mem.rendezvous(buf, self.group)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        peer = [ptrs[g] for g in self.group_rank_of_plan]
        self.capacity, self.hdl = cap, hdl
        self.ws = Workspace(layout, buf, peer, self.r * self.ulysses + self.u)
        self.state = CallState()
        self.status = _status.StatusMirror(self.ws.status_tensor())
        self._launch_cache.clear()

    def check_status(self) -> None:
        """Host-synchronising check of the device status word."""
        if self.status is not None:
            self.status.check_now()

    def reset(self) -> None:
        """Recover after a timed-out wait: collective over the group. Clears the status word and
        the exchange counters on every rank and restarts the call count, so that the expected
        counter values agree again whatever each rank managed to do in the failed call."""
        if self.ws is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # nobody is still adding to anybody's counters
        lay = self.ws.layout
        self.ws.buf[lay.stage_bytes:lay.total].zero_()  # arrival and output counters, status word
        self.state = CallState()
        self._launch_cache.clear()
        self.status.reset()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float],
                  is_causal: bool = False, key_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """q: [B, H, s_q, D], k/v: [B, H, s_kv, D] local shards -> [B, H, s_q, D] local output.
        ``is_causal`` masks over the whole sequence, shards taken in flat-rank order. ``key_mask``
        ([B, world * s_kv] bool, the same on every rank) drops keys, chunks in flat-rank order."""
        B, H, sq, D = q.shape
        skv = k.shape[2]
        plan = CpPlan(self.ulysses, self.ring, self.u, self.r, H)
        self._ensure(stage_sizes(plan, B, sq, skv, D, q.element_size()))
        # a wait that ran out in an earlier call is raised here, from host memory (no device sync)
        self.status.check()
        ws, st = self.ws, self.state
        par = st.calls & 1
        st.calls += 1
        sms = _sm_count(self.device)
        ctas = config.cp.push_ctas_per_dest
        if ctas <= 0:
            # automatic: about one pushing CTA per 5 MB this rank has to send, between 16 and 64
            # (a CTA sustains a few tens of GB/s of peer stores; 64 of them saturate NVLink)
            hl = plan.local_heads
            esz = q.element_size()
            sent = (self.world - 1) * 2 * B * hl * skv * D * esz + (self.ulysses - 1) * B * hl * sq * D * esz
            ctas = (sent + (5 << 20) - 1) // (5 << 20)
            # SMs that the last, partly filled wave of the grid leaves idle can push for free
            grid = ((sq + 255) // 256) * hl * B * self.ulysses
            spare = (-grid) % sms
            ctas = max(16, min(64, max(ctas, min(spare, 48))))
        wait_ns = config.cp.wait_limit_ns
        scale = (1.0 / math.sqrt(D)) if scale is None else float(scale)
        main = torch.cuda.current_stream(self.device)
        q, k, v = _fix(q), _fix(k), _fix(v)

        # 1 + 2. one launch: the leading CTAs push this rank's shard to its consumers, all CTAs
        # compute attention over the chunks as they arrive. The argument structures depend only
        # on shapes, strides and the staging parity: they are built once and then only the
        # pointers and the expected counter value are patched (the host side of a 30 us kernel
        # must not cost more than the kernel).
        n_push = fused_push_ctas(plan, B, sq, ctas, sms)
        st.arrive_expect[par] += n_push
        out_local = None
        if self.ulysses == 1:
            out_local = torch.empty((B, sq, H, D), dtype=q.dtype, device=q.device).transpose(1, 2)
        key_bits = None
        if key_mask is not None:
            from . import ops as _ops

            key_bits = _ops.pack_key_mask(key_mask, self.world, skv)
        key = (B, H, sq, skv, D, q.dtype, par, n_push, scale, wait_ns, q.stride(), k.stride(), v.stride(),
               is_causal, key_bits is not None)
        ent = self._launch_cache.get(key)
        if ent is None:
            push = build_push_args(plan, ws, par, q, k, v, n_push)
            a = build_attention_args(plan, ws, par, (B, H, sq, D), q.dtype, skv, scale, st.arrive_expect[par],
                                     wait_ns, out_local, push, (q, k, v), is_causal, key_bits)
            which = [js.tensor for js in plan.push_jobs(skip_self=True)]
            ent = (a, push, which)
            if len(self._launch_cache) > 64:
                self._launch_cache.clear()
            self._launch_cache[key] = ent
        else:
            a, push, which = ent
            ptr = {"q": q.data_ptr(), "k": k.data_ptr(), "v": v.data_ptr()}
            for i, name in enumerate(which):
                push.jobs[i].src = ptr[name]
            a.q_local, a.k_local, a.v_local = ptr["q"], ptr["k"], ptr["v"]
            a.flag_expect = st.arrive_expect[par]
            if key_bits is not None:
                a.key_bits = key_bits.data_ptr()
            if out_local is not None:
                a.out[0] = out_local.data_ptr()
        L.check(L.load().pa_cp_attn_fwd(C.byref(a), main.cuda_stream))
        if is_causal:
            # A causal kernel does not wait for the chunks it cannot see, so an early rank could
            # run two calls ahead and overwrite staging memory a later rank still reads. Waiting
            # for every rank's arrival counter keeps the ranks within one call of each other,
            # which is what the two staging parities allow.
            lay = ws.layout
            others = [s for s in range(self.world) if s != plan.rank]  # nobody counts into its own slot
            flags = (C.c_void_p * len(others))(*[ws.base + lay.off_arrive[par] + 4 * s for s in others])
            L.check(L.load().pa_flag_wait(flags, len(others), st.arrive_expect[par], ws.base + lay.off_status,
                                          wait_ns, 3, main.cuda_stream))
        if out_local is not None:
            self.status.refresh()
            return out_local

        # 3. wait for the tiles owed to me, then hand out a private copy
        st.done_expect[par] += out_tiles_per_call(plan, B, sq)
        launch_out_wait(ws, par, st.done_expect[par], wait_ns, main.cuda_stream)
        lay = ws.layout
        out_bytes = B * sq * H * D * q.element_size()
        o_stage = ws.buf[lay.off_o[par]:lay.off_o[par] + out_bytes].view(q.dtype).view(B, sq, H, D)
        self.status.refresh()
        if config.cp.zero_copy_output:
            # the staging view itself: valid until the second-next call of this engine reuses the parity
            return o_stage.transpose(1, 2)
        return o_stage.clone().transpose(1, 2)


_engines: Dict[Tuple, CpEngine] = {}


def get_engine(flat_group: dist.ProcessGroup, ulysses: int, ring: int, u: int, r: int, device: torch.device) -> CpEngine:
    key = (flat_group.group_name if hasattr(flat_group, "group_name") else id(flat_group), ulysses, ring, u, r,
           device.index)
    eng = _engines.get(key)
    if eng is None:
        eng = CpEngine(flat_group, ulysses, ring, u, r, device)
        _engines[key] = eng
    return eng


_engine_list: List[CpEngine] = []


def engine_id(flat_group: dist.ProcessGroup, ulysses: int, ring: int, u: int, r: int, device_index: int) -> int:
    """A small integer standing for the engine of this (group, mesh position, device): what the
    ``para_attn::cp_attention_forward`` custom op carries instead of Python objects, so that
    a tracing compiler sees a constant. Creating an engine is collective over the group."""
    eng = get_engine(flat_group, ulysses, ring, u, r, torch.device("cuda", device_index))
    for i, e in enumerate(_engine_list):
        if e is eng:
            return i
    _engine_list.append(eng)
    return len(_engine_list) - 1


def engine_by_id(i: int) -> CpEngine:
    return _engine_list[i]


def check_device_status() -> None:
    """Raise if any attention kernel of this process reported a timed-out wait (synchronises)."""
    from . import _peer_gather

    for eng in _engines.values():
        eng.check_status()
    for g in _peer_gather.all_gathers():
        if g.status is not None:
            g.status.check_now()
    for mirror in _status.all_mirrors():
        mirror.check_now()


def reset_device_status() -> None:
    """Clear every status word and resynchronise the exchange counters (collective over each
    engine's group): the way back to a usable state after a ``PaError(PA_ETIMEDOUT)``."""
    from . import _peer_gather

    for eng in _engines.values():
        eng.reset()
    for g in _peer_gather.all_gathers():
        g.reset()
    for mirror in _status.all_mirrors():
        mirror.reset()
