"""CPU oracle for the context-parallel attention path, key-padding masks, the First-Block-Cache
decision and its TaylorSeer extrapolation.

TEST INFRASTRUCTURE ONLY. This module is a numpy restatement of the arithmetic the
ParaAttention reference performs for its ring / Ulysses / unified attention and for the
cache decision. It exists to check the CUDA library and must never be imported by the
product package: only the tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` use it.

Pinning: ``tests/golden/make_golden.py`` runs the reference itself (CPU, gloo, fp32 attention;
bf16 cache and TaylorSeer tensors) and stores its inputs and outputs; ``tests/test_oracle.py``
checks every function below against those fixtures (attention to 2e-6, cache decisions
identical, TaylorSeer outputs bit for bit).

Citations are ``file:line`` in the ParaAttention source tree; ``torch:`` marks
torch/distributed/tensor/experimental/_context_parallel/_attention.py of PyTorch 2.11,
the un-vendored dependency that holds the ring loop and the out/LSE merger.

All "rank" loops below run inside one process: a list index stands for a rank.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np

Array = np.ndarray


# --------------------------------------------------------------------------------------
# per-device attention (src/para_attn/ops/__init__.py:112-179)
# --------------------------------------------------------------------------------------
def sdpa_with_lse(q: Array, k: Array, v: Array, *, scale: Optional[float] = None, is_causal: bool = False,
                  dtype=np.float32, key_mask: Optional[Array] = None) -> Tuple[Array, Array]:
    """out = softmax(scale * q k^T [+ causal mask]) v and lse = logsumexp of the scaled logits.

    Mirrors what ``attention_forward_with_lse`` returns (src/para_attn/ops/__init__.py:160-179):
    ``out`` shaped like ``q``, ``lse`` of shape [B, H, S_q] holding the natural-log LSE. The
    causal mask is top-left aligned like torch SDPA. Shapes are [B, H, S, D].

    ``key_mask`` ([B, S_kv] bool) drops keys the way ``_attention_forward_sparse_kv`` does
    (src/para_attn/ops/__init__.py:271-292: per batch element, keep ``k[..., indices[m], :]``);
    a batch element without any kept key yields zeros, as SDPA over zero keys does.
    """
    q = np.asarray(q, dtype=dtype)
    k = np.asarray(k, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    s = np.matmul(q, np.swapaxes(k, -1, -2)) * dtype(scale)
    if is_causal:
        sq, sk = s.shape[-2], s.shape[-1]
        mask = np.tril(np.ones((sq, sk), dtype=bool))
        s = np.where(mask, s, dtype(-np.inf))
    if key_mask is not None:
        km = np.asarray(key_mask, dtype=bool)
        s = np.where(km[:, None, None, :], s, dtype(-np.inf))
    m = s.max(axis=-1, keepdims=True)
    dead = ~np.isfinite(m)            # rows without any visible key
    m = np.where(dead, dtype(0), m)
    p = np.exp(s - m)
    l = p.sum(axis=-1, keepdims=True)
    with np.errstate(divide="ignore", invalid="ignore"):
        out = np.matmul(np.where(dead, dtype(0), p / np.where(dead, dtype(1), l)), v)
        lse = np.where(dead, dtype(-np.inf), m + np.log(np.where(dead, dtype(1), l)))[..., 0]
    return out, lse


def split_key_shares(n_tiles: int, k: int) -> List[Tuple[int, int]]:
    """Tile ranges [begin, end) of the k CTAs that share one work unit of a split last wave:
    share i takes tiles [n*i/k, n*(i+1)/k) of the unit's tile list (integer division). No
    counterpart in the reference, whose library kernels schedule themselves."""
    return [(n_tiles * i // k, n_tiles * (i + 1) // k) for i in range(k)]


def combine_key_shares(q: Array, k: Array, v: Array, shares: Sequence[Tuple[int, int]], *, tile: int = 128,
                       scale: Optional[float] = None, key_mask: Optional[Array] = None,
                       stale: Optional[Sequence[float]] = None) -> Tuple[Array, Array]:
    """Attention computed share by share over ranges of key tiles and combined the way the
    split epilogue does: every share yields an unnormalised output O_i, a reference m_i and a
    row sum l_i (both relative to m_i); the result is
    sum_i e^(m_i - m) O_i / sum_i e^(m_i - m) l_i with m = max_i m_i, shares added in index order,
    a share without any visible key (m_i = -inf) weighing nothing. ``stale[i]`` subtracts a
    constant from share i's true row maximum to stand for the kernel's lazily updated reference:
    the result must not depend on it."""
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    parts = []
    for i, (t0, t1) in enumerate(shares):
        sl = slice(t0 * tile, min(t1 * tile, k.shape[-2]))
        s = np.matmul(q, np.swapaxes(k[..., sl, :], -1, -2)) * np.float32(scale)
        if key_mask is not None:
            s = np.where(np.asarray(key_mask, dtype=bool)[:, None, None, sl], s, np.float32(-np.inf))
        m = s.max(axis=-1, keepdims=True) if s.shape[-1] else np.full(s.shape[:-1] + (1,), -np.inf, np.float32)
        if stale is not None:
            m = m - np.float32(stale[i])
        with np.errstate(invalid="ignore"):
            p = np.where(np.isneginf(m), np.float32(0), np.exp(s - np.where(np.isneginf(m), np.float32(0), m)))
        parts.append((m, p.sum(axis=-1, keepdims=True), np.matmul(p, v[..., sl, :])))
    m_tot = parts[0][0]
    for m, _, _ in parts[1:]:
        m_tot = np.maximum(m_tot, m)
    acc_o = np.zeros_like(parts[0][2])
    acc_l = np.zeros_like(parts[0][1])
    for m, l, o in parts:
        with np.errstate(invalid="ignore"):
            w = np.where(np.isneginf(m), np.float32(0), np.exp(m - np.where(np.isneginf(m_tot), np.float32(0), m_tot)))
        acc_o += o * w
        acc_l += l * w
    dead = ~(acc_l > 0)
    with np.errstate(divide="ignore", invalid="ignore"):
        out = np.where(dead, np.float32(0), acc_o / np.where(dead, np.float32(1), acc_l))
        lse = np.where(dead, np.float32(-np.inf), m_tot + np.log(np.where(dead, np.float32(1), acc_l)))[..., 0]
    return out, lse


def _sigmoid(x: Array) -> Array:
    return 1.0 / (1.0 + np.exp(-x))


def _logsigmoid(x: Array) -> Array:
    # log(sigmoid(x)) = -softplus(-x), evaluated without overflow
    return -(np.maximum(-x, 0) + np.log1p(np.exp(-np.abs(x))))


def merge_out_lse(out: Array, lse: Array, block_out: Array, block_lse: Array) -> Tuple[Array, Array]:
    """One step of torch's ``_SDPAMerger._merge_one`` (torch:182-183), in the arrays' dtype.

    ``out -= sigmoid(block_lse - lse) * (out - block_out)``;
    ``lse -= logsigmoid(lse - block_lse)``. ``lse`` arrays are [B, H, S]; they broadcast
    against ``out`` [B, H, S, D] through a trailing axis exactly like the unsqueeze at torch:153-158.
    """
    lse_e = lse[..., None]
    blse_e = block_lse[..., None]
    new_out = out - _sigmoid(blse_e - lse_e) * (out - block_out)
    new_lse = lse - _logsigmoid(lse - block_lse)
    return new_out, new_lse


# --------------------------------------------------------------------------------------
# ring attention (src/para_attn/para_attn_interface.py:162-239 + torch:309-478)
# --------------------------------------------------------------------------------------
def ring_attention(qs: Sequence[Array], ks: Sequence[Array], vs: Sequence[Array], *, scale: Optional[float] = None,
                   is_causal: bool = False, dtype=np.float32) -> List[Array]:
    """Per-rank outputs of ``ring_attn_func`` for ranks holding (qs[r], ks[r], vs[r]).

    Step i on rank r consumes the K/V of rank (r - i) mod R, because every step passes the
    buffer to rank+1 (torch:247-263, 421-432). Without load balancing (disabled at
    src/para_attn/para_attn_interface.py:138-140) a causal run masks step 0, uses earlier
    ranks' blocks in full and skips later ranks' (torch:83-100). Blocks are merged in fp32
    (``convert_to_f32``, para_attn_interface.py:133-137) and LSE is dropped at the end (:196-197).
    """
    R = len(qs)
    outs = []
    for r in range(R):
        out = lse = None
        for i in range(R):
            src = (r - i) % R
            if is_causal and i > 0 and src > r:
                continue
            b_out, b_lse = sdpa_with_lse(qs[r], ks[src], vs[src], scale=scale, is_causal=is_causal and i == 0,
                                         dtype=dtype)
            if out is None:
                out, lse = b_out, b_lse
            else:
                out, lse = merge_out_lse(out, lse, b_out, b_lse)
        outs.append(out)
    return outs


# --------------------------------------------------------------------------------------
# Ulysses (src/para_attn/para_attn_interface.py:52-119)
# --------------------------------------------------------------------------------------
def ulysses_input_all_to_all(xs: Sequence[Array]) -> List[Array]:
    """[b, h, s, d] per rank -> [b, h/U, U*s, d] per rank (para_attn_interface.py:60-72).

    Rank u receives head block u of every rank; along the sequence the pieces appear in
    source-rank order (the reshape/permute at :71 after the equal-split all-to-all at :70).
    """
    U = len(xs)
    b, h, s, d = xs[0].shape
    assert h % U == 0, "h must be divisible by world_size"
    hl = h // U
    return [np.concatenate([xs[src][:, u * hl:(u + 1) * hl] for src in range(U)], axis=2) for u in range(U)]


def ulysses_output_all_to_all(xs: Sequence[Array]) -> List[Array]:
    """[b, h/U, S, d] per rank -> [b, h, S/U, d] per rank (para_attn_interface.py:75-87)."""
    U = len(xs)
    b, hl, S, d = xs[0].shape
    assert S % U == 0, "s must be divisible by world_size"
    sl = S // U
    return [np.concatenate([xs[src][:, :, u * sl:(u + 1) * sl] for src in range(U)], axis=1) for u in range(U)]


def ulysses_attention(qs, ks, vs, *, scale=None, is_causal=False, dtype=np.float32) -> List[Array]:
    """Per-rank outputs of ``ulysses_attn_func`` (para_attn_interface.py:90-119)."""
    q2, k2, v2 = ulysses_input_all_to_all(qs), ulysses_input_all_to_all(ks), ulysses_input_all_to_all(vs)
    o2 = [sdpa_with_lse(q, k, v, scale=scale, is_causal=is_causal, dtype=dtype)[0] for q, k, v in zip(q2, k2, v2)]
    return ulysses_output_all_to_all(o2)


# --------------------------------------------------------------------------------------
# unified: Ulysses outside, ring inside (src/para_attn/para_attn_interface.py:445-479)
# --------------------------------------------------------------------------------------
def unified_attention(qs, ks, vs, *, ulysses: int, ring: int, scale=None, is_causal=False,
                      dtype=np.float32) -> List[Array]:
    """Per-rank outputs under ``UnifiedAttnMode`` on a (ring, ulysses) mesh.

    Global rank = ring_idx * ulysses + ulysses_idx: the mesh built at
    src/para_attn/context_parallel/__init__.py:38-39 puts "ulysses" last, i.e. fastest.
    Each Ulysses group (fixed ring_idx) re-partitions heads, then every ring group (fixed
    ulysses_idx) runs ring attention over the re-partitioned tensors.
    """
    U, R = ulysses, ring
    assert len(qs) == U * R
    q2, k2, v2 = [None] * (U * R), [None] * (U * R), [None] * (U * R)
    for r in range(R):
        ranks = [r * U + u for u in range(U)]
        for name, src, dst in (("q", qs, q2), ("k", ks, k2), ("v", vs, v2)):
            conv = ulysses_input_all_to_all([np.asarray(src[g], dtype=dtype) for g in ranks]) if U > 1 else [
                np.asarray(src[g], dtype=dtype) for g in ranks]
            for u, g in enumerate(ranks):
                dst[g] = conv[u]
    o2 = [None] * (U * R)
    for u in range(U):
        ranks = [r * U + u for r in range(R)]
        outs = ring_attention([q2[g] for g in ranks], [k2[g] for g in ranks], [v2[g] for g in ranks], scale=scale,
                              is_causal=is_causal, dtype=dtype)
        for r, g in enumerate(ranks):
            o2[g] = outs[r]
    res = [None] * (U * R)
    for r in range(R):
        ranks = [r * U + u for u in range(U)]
        conv = ulysses_output_all_to_all([o2[g] for g in ranks]) if U > 1 else [o2[g] for g in ranks]
        for u, g in enumerate(ranks):
            res[g] = conv[u]
    return res


# --------------------------------------------------------------------------------------
# bf16 emulation
# --------------------------------------------------------------------------------------
def bf16_round(x) -> Array:
    """Round fp32 values to the nearest bfloat16 (ties to even), returned as fp32."""
    a = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
    u = a.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    out = rounded.view(np.float32).reshape(a.shape)
    return np.where(np.isnan(a), a, out)


def bf16_bits_to_f32(bits: Array) -> Array:
    """uint16 bfloat16 bit patterns -> fp32 values."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: Array) -> Array:
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


# --------------------------------------------------------------------------------------
# First Block Cache (src/para_attn/first_block_cache/utils.py)
# --------------------------------------------------------------------------------------
def fbc_partial_sums(prev: Array, cur: Array) -> Tuple[float, float]:
    """fp32 sums behind the two bf16 means of ``are_two_tensors_similar`` (utils.py:228-229).

    ``prev`` and ``cur`` hold bf16-representable values. ``(t1 - t2)`` is a bf16 tensor, so
    each difference is rounded to bf16 before ``abs().mean()``; the mean accumulates in fp32.
    Returns (sum |bf16(prev - cur)|, sum |prev|).
    """
    prev = np.asarray(prev, dtype=np.float32)
    cur = np.asarray(cur, dtype=np.float32)
    diff = np.abs(bf16_round(prev - cur))
    return float(diff.sum(dtype=np.float64)), float(np.abs(prev).sum(dtype=np.float64))


def fbc_decision(sum_diff: Sequence[float], sum_prev: Sequence[float], numel: int, threshold: float) -> bool:
    """``are_two_tensors_similar`` (utils.py:220-234) from per-rank partial sums.

    Per rank the two means are bf16 scalars (mean of a bf16 tensor); with several ranks each
    is averaged over the world group (utils.py:230-232, primitives.py:90-94) and stays bf16;
    the ratio is a bf16 division; the comparison is against a python float.
    """
    if threshold <= 0.0:
        return False
    md = [bf16_round(np.float32(s / numel)) for s in sum_diff]
    mp = [bf16_round(np.float32(s / numel)) for s in sum_prev]
    if len(md) > 1:
        mean_diff = bf16_round(np.float32(np.sum(md, dtype=np.float32) / np.float32(len(md))))
        mean_prev = bf16_round(np.float32(np.sum(mp, dtype=np.float32) / np.float32(len(mp))))
    else:
        mean_diff, mean_prev = md[0], mp[0]
    with np.errstate(divide="ignore", invalid="ignore"):
        ratio = bf16_round(np.float32(mean_diff) / np.float32(mean_prev))
    return bool(float(np.asarray(ratio).reshape(-1)[0]) < threshold)


class FbcStateOracle:
    """Step bookkeeping of ``CacheContext`` + ``get_can_use_cache`` (utils.py:12-120, 269-295).

    Feed it the first-block residual of every transformer forward (bf16-representable fp32
    array, one rank) and it answers whether the reference would reuse the cache, keeping
    the previous residual only when the reference does (it is overwritten on a miss,
    utils.py:367-381, and left alone on a hit).
    """

    def __init__(self, residual_diff_threshold: float = 0.0, warmup_steps: int = 0, downsample_factor: int = 1,
                 enable_alter_cache: bool = False, alter_residual_diff_threshold: Optional[float] = None):
        self.threshold = residual_diff_threshold
        self.alter_threshold = alter_residual_diff_threshold
        self.warmup_steps = warmup_steps
        self.downsample_factor = downsample_factor
        self.enable_alter_cache = enable_alter_cache
        self.executed_steps = 0
        self.is_alter_cache = True
        self.prev = {}

    def _key(self) -> str:
        return "alter" if (self.enable_alter_cache and self.is_alter_cache) else "main"

    def step(self, first_residual: Array) -> bool:
        # mark_step_begin, utils.py:83-92
        if not self.enable_alter_cache:
            self.executed_steps += 1
        else:
            self.is_alter_cache = not self.is_alter_cache
            if not self.is_alter_cache:
                self.executed_steps += 1
        cur = np.asarray(first_residual, dtype=np.float32)
        if self.downsample_factor > 1:
            cur = cur[..., ::self.downsample_factor]
        thr = self.threshold
        if self.enable_alter_cache and self.is_alter_cache and self.alter_threshold is not None:
            thr = self.alter_threshold
        hit = False
        in_warmup = (self.executed_steps - 1) < self.warmup_steps
        prev = self.prev.get(self._key())
        if not in_warmup and thr > 0.0 and prev is not None and prev.shape == cur.shape:
            sd, sp = fbc_partial_sums(prev, cur)
            hit = fbc_decision([sd], [sp], cur.size, thr)
        if not hit:
            self.prev[self._key()] = cur.copy()
        return hit


# --------------------------------------------------------------------------------------
# TaylorSeer (src/para_attn/first_block_cache/taylorseer.py:4-64)
# --------------------------------------------------------------------------------------
class TaylorSeerOracle:
    """The reference's extrapolator on bf16 tensors, as arrays of bf16-representable fp32 values.

    Every tensor operation of the reference produces a bf16 tensor, so every intermediate is
    rounded: ``(d_i - prev_i)`` then ``/ window`` (taylorseer.py:35); ``(1 / i!) * d_i`` then
    ``* elapsed**i`` then ``output += term`` (taylorseer.py:44-45). The scalars enter the
    arithmetic as fp32, which is what a Python float against a bf16 tensor becomes.
    """

    def __init__(self, n_derivatives=2, warmup_steps=1, skip_interval_steps=1, compute_step_map=None):
        self.n_derivatives = n_derivatives
        self.order = n_derivatives + 1
        self.warmup_steps = warmup_steps
        self.skip_interval_steps = skip_interval_steps
        self.compute_step_map = compute_step_map
        self.prev = [None] * self.order
        self.cur = [None] * self.order
        self.current_step = -1
        self.last_full = -1

    def should_compute_full(self) -> bool:
        s = self.current_step
        if self.compute_step_map is not None:
            return bool(self.compute_step_map[s])
        return s < self.warmup_steps or (s - self.warmup_steps + 1) % self.skip_interval_steps == 0

    def update(self, y: Array) -> None:
        new = [None] * self.order
        new[0] = np.asarray(y, dtype=np.float32)
        window = np.float32(self.current_step - self.last_full)
        for i in range(self.n_derivatives):
            if self.cur[i] is not None and self.current_step > 1:
                new[i + 1] = bf16_round(bf16_round(new[i] - self.cur[i]) / window)
            else:
                break
        self.prev, self.cur = self.cur, new
        self.last_full = self.current_step

    def approximate_value(self) -> Array:
        elapsed = self.current_step - self.last_full
        out = None
        for i, d in enumerate(self.cur):
            if d is None:
                break
            if i == 0:
                out = d.copy()  # 0 + (1.0 * d_0) * 1 is d_0 itself
                continue
            coef = np.float32(1.0 / math.factorial(i))
            term = bf16_round(bf16_round(coef * d) * np.float32(elapsed ** i))
            out = bf16_round(out + term)
        return out

    def step(self, y: Array) -> Array:
        self.current_step += 1
        if self.should_compute_full():
            self.update(y)
            return np.asarray(y, dtype=np.float32)
        return self.approximate_value()
