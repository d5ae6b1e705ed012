"""Shared test helpers: tolerance checks, bf16 fixtures, a one-GPU stand-in for a CP cluster."""
from __future__ import annotations

import math
from typing import List

import numpy as np
import torch

from oracle import cp_attention_oracle as O

# north-star tolerances for bf16 attention against an fp32 reference
OUT_MAX_ABS = 2e-2
OUT_REL_L2 = 5e-3
LSE_MAX_ABS = 1e-3


def bf16_from_bits(bits: np.ndarray, device="cuda") -> torch.Tensor:
    t = torch.from_numpy(bits.astype(np.int16))
    return t.view(torch.bfloat16).to(device)


def assert_attention_close(out: torch.Tensor, ref: np.ndarray, what: str = ""):
    got = out.float().cpu().numpy()
    ref = np.asarray(ref, dtype=np.float32)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    max_abs = float(np.abs(got - ref).max())
    rel_l2 = float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))
    assert max_abs <= OUT_MAX_ABS, f"{what}: max-abs {max_abs:.3e} > {OUT_MAX_ABS}"
    assert rel_l2 <= OUT_REL_L2, f"{what}: rel-L2 {rel_l2:.3e} > {OUT_REL_L2}"


def assert_lse_close(lse: torch.Tensor, ref: np.ndarray, what: str = ""):
    err = float(np.abs(lse.float().cpu().numpy() - np.asarray(ref, dtype=np.float32)).max())
    assert err <= LSE_MAX_ABS, f"{what}: lse max-abs {err:.3e} > {LSE_MAX_ABS}"


def seeded_qkv(B, H, Sq, Skv, D=128, dtype=torch.bfloat16, seed=0, device="cuda", bshd=False, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    shp_q = (B, Sq, H, D) if bshd else (B, H, Sq, D)
    shp_k = (B, Skv, H, D) if bshd else (B, H, Skv, D)
    q = (torch.randn(shp_q, generator=g) * scale).to(dtype).to(device)
    k = (torch.randn(shp_k, generator=g) * scale).to(dtype).to(device)
    v = (torch.randn(shp_k, generator=g) * scale).to(dtype).to(device)
    if bshd:
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    return q, k, v


def oracle_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale=None):
    return O.sdpa_with_lse(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), scale=scale)


class LocalCluster:
    """All ranks of a ulysses x ring mesh emulated on ONE GPU with the product's own launch
    helpers: every rank gets its own exchange buffer, "peer" addresses are those buffers, and
    the phases run one after the other on one stream (all pushes, then all attention
    launches, then the output waits), so no kernel ever waits for a later launch."""

    def __init__(self, ulysses: int, ring: int, device="cuda"):
        from paraattention_b200 import _cp_engine as E

        self.E = E
        self.U, self.R, self.W = ulysses, ring, ulysses * ring
        self.device = torch.device(device)
        self.capacity = None
        self.ws: List = []
        self.state = E.CallState()
        # scratch for launches that split their last wave (None: no launch does); the emulated
        # ranks' launches follow each other on one stream and may share it
        self.split_ws = None

    def _ensure(self, plan0, B, sq, skv, D, esz):
        E = self.E
        need = E.stage_sizes(plan0, B, sq, skv, D, esz)
        if self.capacity is not None and all(n <= c for n, c in zip(need, self.capacity)):
            return
        layout = E._make_layout(self.W, self.U, *need)
        bufs = [torch.zeros(layout.total, dtype=torch.uint8, device=self.device) for _ in range(self.W)]
        peer = [b.data_ptr() for b in bufs]
        self.ws = [E.Workspace(layout, bufs[g], peer, g) for g in range(self.W)]
        self.capacity = need
        self.state = E.CallState()

    def attention_fused_single_rank(self, q, k, v, scale=None, ctas=4, wait_ns=200_000_000, in_place=False):
        """World size 1 only: the exchange rides inside the attention launch (the form multi-GPU
        runs use). The pushing CTAs belong to the same launch as the CTAs that wait for them."""
        assert self.W == 1
        E = self.E
        B, H, sq, D = q.shape
        skv = k.shape[2]
        plan = E.CpPlan(1, 1, 0, 0, H)
        self._ensure(plan, B, sq, skv, D, q.element_size())
        st = self.state
        par = st.calls & 1
        st.calls += 1
        n_push = E.fused_push_ctas(plan, B, sq, ctas)
        st.arrive_expect[par] += n_push
        q, k, v = E._fix(q), E._fix(k), E._fix(v)
        # in_place=False keeps the self-push so that the fused pusher path is exercised on one GPU
        push = E.build_push_args(plan, self.ws[0], par, q, k, v, n_push, skip_self=in_place)
        out = torch.empty((B, sq, H, D), dtype=q.dtype, device=self.device).transpose(1, 2)
        scale = (1.0 / math.sqrt(D)) if scale is None else scale
        E.launch_attention(plan, self.ws[0], par, (B, H, sq, D), q.dtype, skv, scale, st.arrive_expect[par], wait_ns,
                           torch.cuda.current_stream(self.device).cuda_stream, out, push, (q, k, v) if in_place else None)
        torch.cuda.synchronize(self.device)
        code = int(self.ws[0].status_tensor().item())
        assert code == 0, f"device status {code}"
        return out

    def attention(self, qs, ks, vs, scale=None, ctas=4, wait_ns=200_000_000, in_place=True, is_causal=False,
                  key_mask=None):
        E = self.E
        B, H, sq, D = qs[0].shape
        skv = ks[0].shape[2]
        plans = [E.CpPlan(self.U, self.R, g % self.U, g // self.U, H) for g in range(self.W)]
        self._ensure(plans[0], B, sq, skv, D, qs[0].element_size())
        st = self.state
        par = st.calls & 1
        st.calls += 1
        st.arrive_expect[par] += ctas
        stream = torch.cuda.current_stream(self.device).cuda_stream
        scale = (1.0 / math.sqrt(D)) if scale is None else scale
        keep = []
        for g in range(self.W):
            q, k, v = E._fix(qs[g]), E._fix(ks[g]), E._fix(vs[g])
            keep.append((q, k, v))
            pa = E.build_push_args(plans[g], self.ws[g], par, q, k, v, ctas, skip_self=in_place)
            from paraattention_b200 import _lib as L
            import ctypes as C

            L.check(L.load().pa_cp_push(C.byref(pa), stream))
        key_bits = None
        if key_mask is not None:  # [B, W * skv] bool, the same on every rank
            from paraattention_b200 import ops

            key_bits = ops.pack_key_mask(key_mask, self.W, skv)
        outs = [None] * self.W
        for g in range(self.W):
            if self.U == 1:
                outs[g] = torch.empty((B, sq, H, D), dtype=qs[g].dtype, device=self.device).transpose(1, 2)
            E.launch_attention(plans[g], self.ws[g], par, (B, H, sq, D), qs[g].dtype, skv, scale, st.arrive_expect[par],
                               wait_ns, stream, outs[g], None, keep[g] if in_place else None, is_causal, key_bits,
                               self.split_ws)
        if self.U > 1:
            st.done_expect[par] += E.out_tiles_per_call(plans[0], B, sq)
            for g in range(self.W):
                E.launch_out_wait(self.ws[g], par, st.done_expect[par], wait_ns, stream)
                lay = self.ws[g].layout
                nbytes = B * sq * H * D * qs[g].element_size()
                stage = self.ws[g].buf[lay.off_o[par]:lay.off_o[par] + nbytes].view(qs[g].dtype).view(B, sq, H, D)
                outs[g] = stage.clone().transpose(1, 2)
        torch.cuda.synchronize(self.device)
        for g in range(self.W):
            code = int(self.ws[g].status_tensor().item())
            assert code == 0, f"rank {g}: device status {code}"
        return outs
