"""Generates the golden fixtures in this folder by running the ParaAttention reference itself.

Run where a checkout of the reference is available (it is imported from ``--ref``, the
``src`` folder of that checkout): CPU only, gloo, fp32 compute on bf16-representable inputs.

    python tests/golden/make_golden.py [--ref <checkout>/src]      (from the repository root)

Writes
  cp_attention_w2.npz   world 2: ulysses_attn_func, ring_attn_func (non-causal and causal)
  cp_attention_w4.npz   world 4: UnifiedAttnMode on a 2x2 (ring x ulysses) mesh, RingAttnMode on 4
  fbcache_steps.npz     CachedTransformerBlocks decisions over a scripted bf16 sequence
  sparse_kv.npz         _attention_forward_sparse_kv (key-padding masks, batch 3) on one process
  taylorseer.npz        TaylorSeer.step over a scripted bf16 sequence, three configurations

The only change made to the reference is the rebinding of
``para_attn.ops._attention_forward_with_lse`` (which asserts CUDA tensors at
src/para_attn/ops/__init__.py:123) to an fp32 math function returning (out, lse); torch's own
ring loop and merger then run unmodified.
"""
from __future__ import annotations

import argparse
import math
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent

B, H, S, D = 1, 2, 192, 128
S_KV_SHORT = 96


def bf16_inputs(seed: int, s_q: int, s_kv: int):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, s_q, D, generator=g).bfloat16()
    k = torch.randn(B, H, s_kv, D, generator=g).bfloat16()
    v = torch.randn(B, H, s_kv, D, generator=g).bfloat16()
    return q, k, v


def bits(x: torch.Tensor) -> np.ndarray:
    return x.contiguous().view(torch.int16).numpy().view(np.uint16)


def math_attention_with_lse(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, *, scale=None):
    assert attn_mask is None and dropout_p == 0.0
    scale = 1.0 / math.sqrt(query.shape[-1]) if scale is None else scale
    s = torch.matmul(query.float(), key.float().transpose(-1, -2)) * scale
    if is_causal:
        sq, sk = s.shape[-2:]
        s = s.masked_fill(~torch.ones(sq, sk, dtype=torch.bool).tril(), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    out = torch.matmul(torch.softmax(s, dim=-1), value.float())
    return out.to(query.dtype), lse


def _worker(rank: int, world: int, port: int, ref: str, ret):
    sys.path.insert(0, ref)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import para_attn  # noqa: F401
    import para_attn.ops as ref_ops
    from para_attn.para_attn_interface import RingAttnMode, UnifiedAttnMode, ring_attn_func, ulysses_attn_func

    ref_ops._attention_forward_with_lse = math_attention_with_lse
    torch.set_num_threads(2)
    out = {}

    def shard(x):
        return x.float().chunk(world, dim=-2)[rank]

    q, k, v = bf16_inputs(1234, S, S)
    qs, ks, vs = shard(q), shard(k), shard(v)
    if world == 2:
        out["ulysses"] = ulysses_attn_func(qs, ks, vs)
        out["ring"] = ring_attn_func(qs, ks, vs)
        out["ring_causal"] = ring_attn_func(qs, ks, vs, is_causal=True)
        out["ulysses_causal"] = ulysses_attn_func(qs, ks, vs, is_causal=True)
        q2, k2, v2 = bf16_inputs(4321, S, S_KV_SHORT)
        out["ring_short_kv"] = ring_attn_func(shard(q2), shard(k2), shard(v2))
        out["ulysses_short_kv"] = ulysses_attn_func(shard(q2), shard(k2), shard(v2))
    else:
        mesh = dist.init_device_mesh("cpu", (2, 2), mesh_dim_names=("ring", "ulysses"))
        with UnifiedAttnMode(mesh):
            out["unified_2x2"] = F.scaled_dot_product_attention(qs, ks, vs)
        with RingAttnMode():
            out["ring4"] = F.scaled_dot_product_attention(qs, ks, vs)
    gathered = {}
    for name, t in out.items():
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        gathered[name] = torch.stack(parts).numpy()
    if rank == 0:
        ret.put(gathered)
    dist.barrier()
    dist.destroy_process_group()


def run_world(world: int, port: int, ref: str):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ref, ret)) for r in range(world)]
    for p in procs:
        p.start()
    res = ret.get(timeout=600)
    for p in procs:
        p.join()
    return res


def make_attention(ref: str):
    q, k, v = bf16_inputs(1234, S, S)
    q2, k2, v2 = bf16_inputs(4321, S, S_KV_SHORT)
    single = F.scaled_dot_product_attention(q.float(), k.float(), v.float()).numpy()
    w2 = run_world(2, 29611, ref)
    np.savez(HERE / "cp_attention_w2.npz", q=bits(q), k=bits(k), v=bits(v), q2=bits(q2), k2=bits(k2), v2=bits(v2),
             single=single, **w2)
    w4 = run_world(4, 29613, ref)
    np.savez(HERE / "cp_attention_w4.npz", **w4)  # same q, k, v as cp_attention_w2.npz
    for name, arr in {**w2, **w4}.items():
        print(name, arr.shape)


def make_fbcache(ref: str):
    sys.path.insert(0, ref)
    from para_attn.first_block_cache import utils as fbc

    T, N, C = 16, 32, 128
    rng = np.random.default_rng(7)
    base = rng.standard_normal((1, N, C)).astype(np.float32)
    drift = rng.standard_normal((1, N, C)).astype(np.float32)
    first_block_outputs, inputs = [], []
    # residual evolves slowly, with two abrupt changes so that both outcomes occur
    for t in range(T):
        jump = 0.6 if t in (5, 11) else 0.0
        h0 = torch.from_numpy(base * (1.0 + 0.01 * t)).bfloat16()
        resid = torch.from_numpy(0.5 * base + (0.02 * t + jump) * drift + 0.01 * rng.standard_normal((1, N, C)).astype(np.float32))
        h1 = (h0.float() + resid).bfloat16()
        inputs.append(h0)
        first_block_outputs.append(h1)

    class Block0(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.t = 0

        def forward(self, hidden_states, encoder_hidden_states):
            out = first_block_outputs[self.t]
            self.t += 1
            return out, (encoder_hidden_states.float() + 0.25).bfloat16()

    class Block1(torch.nn.Module):
        def forward(self, hidden_states, encoder_hidden_states):
            return (hidden_states.float() * 1.5).bfloat16(), (encoder_hidden_states.float() * 0.5).bfloat16()

    cases = {
        "thr008": dict(residual_diff_threshold=0.08),
        "thr003_warm2": dict(residual_diff_threshold=0.03, warmup_steps=2),
        "thr02_ds2": dict(residual_diff_threshold=0.2, downsample_factor=2),
        "thr0": dict(residual_diff_threshold=0.0),
        "thr008_taylor": dict(residual_diff_threshold=0.08, enable_taylorseer=True,
                              taylorseer_kwargs=dict(n_derivatives=2)),
    }
    enc = torch.from_numpy(rng.standard_normal((1, 8, C)).astype(np.float32)).bfloat16()
    store = {"h0": np.stack([bits(x) for x in inputs]), "h1": np.stack([bits(x) for x in first_block_outputs]),
             "enc": bits(enc)}
    for name, kw in cases.items():
        blocks = fbc.CachedTransformerBlocks(torch.nn.ModuleList([Block0(), Block1()]))
        decisions, outs, enc_outs = [], [], []
        with fbc.cache_context(fbc.create_cache_context(**kw)):
            for t in range(T):
                calls = {"n": 0}
                orig = fbc.apply_prev_hidden_states_residual

                def spy(*a, **k):
                    calls["n"] += 1
                    return orig(*a, **k)

                fbc.apply_prev_hidden_states_residual = spy
                try:
                    o, eo = blocks(inputs[t], enc)
                finally:
                    fbc.apply_prev_hidden_states_residual = orig
                decisions.append(calls["n"] > 0)
                outs.append(bits(o))
                enc_outs.append(bits(eo))
        store[f"{name}_hit"] = np.array(decisions)
        if name in ("thr008", "thr02_ds2", "thr008_taylor"):
            store[f"{name}_out"] = np.stack(outs)
        if name == "thr008":
            store[f"{name}_enc_out"] = np.stack(enc_outs)
        print(name, "".join("H" if d else "." for d in decisions))
    np.savez_compressed(HERE / "fbcache_steps.npz", **store)


def make_sparse_kv(ref: str):
    """The reference's key-dropping attention (src/para_attn/ops/__init__.py:248-299) run as is on
    CPU in fp32: batch 3 with a prefix mask, a scattered mask and an all-valid row of flags."""
    sys.path.insert(0, ref)
    import para_attn.ops as ref_ops

    Bm, Hm, Sq, Skv = 3, 1, 48, 160
    g = torch.Generator().manual_seed(99)
    q = torch.randn(Bm, Hm, Sq, D, generator=g).bfloat16()
    k = torch.randn(Bm, Hm, Skv, D, generator=g).bfloat16()
    v = torch.randn(Bm, Hm, Skv, D, generator=g).bfloat16()
    mask = torch.ones(Bm, 1, 1, Skv, dtype=torch.bool)
    mask[0, ..., 97:] = False                                     # padded tail
    mask[1] = torch.rand(1, 1, Skv, generator=g) < 0.6             # scattered
    out = ref_ops._attention_forward_sparse_kv(q.float(), k.float(), v.float(), attn_mask=mask)
    np.savez_compressed(HERE / "sparse_kv.npz", q=bits(q), k=bits(k), v=bits(v), mask=mask.numpy(), out=out.numpy())
    print("sparse_kv", tuple(out.shape), "kept keys per batch element:", mask.sum(dim=-1).flatten().tolist())


def make_taylorseer(ref: str):
    """The reference's TaylorSeer class driven step by step with bf16 tensors on CPU."""
    sys.path.insert(0, ref)
    from para_attn.first_block_cache.taylorseer import TaylorSeer

    T, N = 14, 512
    rng = np.random.default_rng(11)
    a, b, c = (rng.standard_normal(N).astype(np.float32) for _ in range(3))
    ys = [torch.from_numpy(a + 0.07 * t * b + 0.004 * t * t * c).bfloat16() for t in range(T)]
    store = {"y": np.stack([bits(y) for y in ys])}
    cases = {
        "d2_w1_s3": dict(n_derivatives=2, warmup_steps=1, skip_interval_steps=3),
        "d3_w2_s4": dict(n_derivatives=3, warmup_steps=2, skip_interval_steps=4),
        "d1_map": dict(n_derivatives=1, compute_step_map=[True, True, False, True, False, False, False, True, False,
                                                          False, True, False, False, False]),
    }
    for name, kw in cases.items():
        seer = TaylorSeer(**kw)
        outs = [seer.step(y) for y in ys]
        store[name] = np.stack([bits(o) for o in outs])
        print(name, "computed steps:", [t for t in range(T) if seer.should_compute_full(t)])
    np.savez_compressed(HERE / "taylorseer.npz", **store)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("PARA_ATTN_REF", "../reference/src"),
                    help="src folder of a ParaAttention checkout")
    ap.add_argument("--only", choices=["attention", "fbcache", "sparse_kv", "taylorseer"], default=None)
    args = ap.parse_args()
    args.ref = os.path.abspath(args.ref)
    if args.only in (None, "attention"):
        make_attention(args.ref)
    if args.only in (None, "fbcache"):
        make_fbcache(args.ref)
    if args.only in (None, "sparse_kv"):
        make_sparse_kv(args.ref)
    if args.only in (None, "taylorseer"):
        make_taylorseer(args.ref)
