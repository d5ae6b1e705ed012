"""The numpy oracle against fixtures produced by the reference itself (tests/golden/make_golden.py)."""
import numpy as np
import pytest

from oracle import cp_attention_oracle as O


def _f32(bits):
    return O.bf16_bits_to_f32(bits)


@pytest.fixture(scope="module")
def w2(golden_dir):
    return np.load(golden_dir / "cp_attention_w2.npz")


@pytest.fixture(scope="module")
def w4(golden_dir):
    return np.load(golden_dir / "cp_attention_w4.npz")


def _shards(x, world):
    return np.split(x, world, axis=-2)


def test_single_device_sdpa(w2):
    q, k, v = _f32(w2["q"]), _f32(w2["k"]), _f32(w2["v"])
    out, lse = O.sdpa_with_lse(q, k, v)
    np.testing.assert_allclose(out, w2["single"], atol=2e-6, rtol=1e-5)
    s = np.matmul(q.astype(np.float64), np.swapaxes(k.astype(np.float64), -1, -2)) / np.sqrt(128.0)
    ref_lse = np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1)
    np.testing.assert_allclose(lse, ref_lse, atol=1e-5)


@pytest.mark.parametrize("name,causal", [("ulysses", False), ("ulysses_causal", True)])
def test_ulysses_world2(w2, name, causal):
    q, k, v = (_shards(_f32(w2[n]), 2) for n in ("q", "k", "v"))
    outs = O.ulysses_attention(q, k, v, is_causal=causal)
    np.testing.assert_allclose(np.stack(outs), w2[name], atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("name,causal", [("ring", False), ("ring_causal", True)])
def test_ring_world2(w2, name, causal):
    q, k, v = (_shards(_f32(w2[n]), 2) for n in ("q", "k", "v"))
    outs = O.ring_attention(q, k, v, is_causal=causal)
    np.testing.assert_allclose(np.stack(outs), w2[name], atol=2e-6, rtol=1e-5)


def test_short_kv_world2(w2):
    q, k, v = (_shards(_f32(w2[n]), 2) for n in ("q2", "k2", "v2"))
    np.testing.assert_allclose(np.stack(O.ring_attention(q, k, v)), w2["ring_short_kv"], atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(np.stack(O.ulysses_attention(q, k, v)), w2["ulysses_short_kv"], atol=2e-6, rtol=1e-5)


def test_unified_and_ring_world4(w2, w4):
    q, k, v = (_shards(_f32(w2[n]), 4) for n in ("q", "k", "v"))
    uni = O.unified_attention(q, k, v, ulysses=2, ring=2)
    np.testing.assert_allclose(np.stack(uni), w4["unified_2x2"], atol=2e-6, rtol=1e-5)
    ring = O.ring_attention(q, k, v)
    np.testing.assert_allclose(np.stack(ring), w4["ring4"], atol=2e-6, rtol=1e-5)


def test_sharded_equals_single_device(w2):
    # the reference's own pinned contract (tests/test_interface.py:70): shard r == chunk r of single-device SDPA
    q, k, v = (_shards(_f32(w2[n]), 4) for n in ("q", "k", "v"))
    full = np.concatenate(O.unified_attention(q, k, v, ulysses=2, ring=2), axis=-2)
    np.testing.assert_allclose(full, w2["single"], atol=1e-5)


def test_merge_is_order_free():
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, 2, 16, 8)).astype(np.float32)
    k = rng.standard_normal((1, 2, 48, 8)).astype(np.float32)
    v = rng.standard_normal((1, 2, 48, 8)).astype(np.float32)
    full, full_lse = O.sdpa_with_lse(q, k, v)
    parts = [O.sdpa_with_lse(q, k[:, :, i:i + 16], v[:, :, i:i + 16]) for i in (32, 0, 16)]
    out, lse = parts[0]
    for bo, bl in parts[1:]:
        out, lse = O.merge_out_lse(out, lse, bo, bl)
    np.testing.assert_allclose(out, full, atol=1e-5)
    np.testing.assert_allclose(lse, full_lse, atol=1e-5)


def test_bf16_round_matches_torch():
    import torch

    x = np.random.default_rng(1).standard_normal(4096).astype(np.float32) * 100
    x[:4] = [0.0, -0.0, 1.00390625, 3.3895314e38]
    want = torch.from_numpy(x).bfloat16().float().numpy()
    np.testing.assert_array_equal(O.bf16_round(x), want)
    np.testing.assert_array_equal(O.bf16_bits_to_f32(O.f32_to_bf16_bits(x)), want)


@pytest.mark.parametrize("case,kw", [
    ("thr008", dict(residual_diff_threshold=0.08)),
    ("thr003_warm2", dict(residual_diff_threshold=0.03, warmup_steps=2)),
    ("thr02_ds2", dict(residual_diff_threshold=0.2, downsample_factor=2)),
    ("thr0", dict(residual_diff_threshold=0.0)),
])
def test_fbcache_decisions(golden_dir, case, kw):
    g = np.load(golden_dir / "fbcache_steps.npz")
    h0, h1 = _f32(g["h0"]), _f32(g["h1"])
    state = O.FbcStateOracle(**kw)
    hits = []
    for t in range(h0.shape[0]):
        first_residual = O.bf16_round(h1[t] - h0[t])  # bf16 tensor subtraction, utils.py:359
        hits.append(state.step(first_residual))
    assert hits == list(g[f"{case}_hit"])


def test_key_mask_against_reference_sparse_kv(golden_dir):
    """sdpa_with_lse(key_mask=...) against the reference's own _attention_forward_sparse_kv."""
    g = np.load(golden_dir / "sparse_kv.npz")
    q, k, v = (_f32(g[n]) for n in ("q", "k", "v"))
    mask = g["mask"][:, 0, 0, :]
    out, lse = O.sdpa_with_lse(q, k, v, key_mask=mask)
    np.testing.assert_allclose(out, g["out"], rtol=1e-5, atol=2e-6)
    assert np.isfinite(lse).all()
    # dropping keys == gathering the kept keys, batch element by batch element
    for b in range(q.shape[0]):
        keep = np.nonzero(mask[b])[0]
        o_b, l_b = O.sdpa_with_lse(q[b:b + 1], k[b:b + 1, :, keep], v[b:b + 1, :, keep])
        np.testing.assert_allclose(out[b:b + 1], o_b, rtol=1e-5, atol=2e-6)
        np.testing.assert_allclose(lse[b:b + 1], l_b, rtol=1e-5, atol=2e-6)
    # a batch element without any kept key: zeros and an LSE of -inf
    none = np.zeros_like(mask)
    out0, lse0 = O.sdpa_with_lse(q, k, v, key_mask=none)
    assert (out0 == 0).all() and np.isneginf(lse0).all()


@pytest.mark.parametrize("case,kw", [
    ("d2_w1_s3", dict(n_derivatives=2, warmup_steps=1, skip_interval_steps=3)),
    ("d3_w2_s4", dict(n_derivatives=3, warmup_steps=2, skip_interval_steps=4)),
    ("d1_map", dict(n_derivatives=1, compute_step_map=[True, True, False, True, False, False, False, True, False,
                                                       False, True, False, False, False])),
])
def test_taylorseer_bit_exact_against_reference(golden_dir, case, kw):
    """TaylorSeerOracle.step against the reference's TaylorSeer.step on bf16 tensors, bit for bit."""
    g = np.load(golden_dir / "taylorseer.npz")
    ys = _f32(g["y"])
    seer = O.TaylorSeerOracle(**kw)
    for t in range(ys.shape[0]):
        got = seer.step(ys[t])
        assert np.array_equal(got, _f32(g[case][t])), f"{case}: step {t} differs"


@pytest.mark.parametrize("U,R", [(2, 1), (1, 2), (2, 2), (4, 2), (1, 8)])
def test_causal_composition_equals_whole_sequence_causal(U, R):
    """The oracle's Ulysses-around-causal-ring composition (step 0 causal, earlier ranks in full,
    later ranks skipped) is plain causal attention over the sequence sharded in flat-rank order."""
    W = U * R
    rng = np.random.default_rng(U * 10 + R)
    H, s, D = 2 * U, 24, 16
    q, k, v = (rng.standard_normal((1, H, W * s, D)).astype(np.float32) for _ in range(3))
    qs, ks, vs = (_shards(x, W) for x in (q, k, v))
    outs = O.unified_attention(qs, ks, vs, ulysses=U, ring=R, is_causal=True)
    whole, _ = O.sdpa_with_lse(q, k, v, is_causal=True)
    np.testing.assert_allclose(np.concatenate(outs, axis=-2), whole, rtol=2e-5, atol=2e-6)


def test_key_mask_composes_with_chunks():
    """Masked attention over the whole sequence equals merging per-chunk masked attention: what
    the chunked kernel relies on when a mask meets ring chunks."""
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((2, 2, 40, 16)).astype(np.float32) for _ in range(3))
    mask = rng.random((2, 40)) < 0.6
    mask[1, 20:] = False  # second chunk of batch element 1 is all padding
    whole, whole_lse = O.sdpa_with_lse(q, k, v, key_mask=mask)
    out = lse = None
    for c in range(2):
        sl = slice(c * 20, (c + 1) * 20)
        o_c, l_c = O.sdpa_with_lse(q, k[:, :, sl], v[:, :, sl], key_mask=mask[:, sl])
        if out is None:
            out, lse = o_c, l_c
            continue
        # a chunk without any visible key carries LSE = -inf and must not disturb the merge
        dead = np.isneginf(l_c)
        with np.errstate(over="ignore"):  # the stand-in for -inf overflows exp(); those rows are discarded
            m_out, m_lse = O.merge_out_lse(out, lse, o_c, np.where(dead, -1e30, l_c))
        out, lse = np.where(dead[..., None], out, m_out), np.where(dead, lse, m_lse)
    np.testing.assert_allclose(out, whole, rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(lse, whole_lse, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("k", [2, 3, 5])
def test_shares_of_a_split_unit_combine_to_whole_attention(k):
    """What the split of an under-filled last wave relies on: attention over disjoint ranges of
    key tiles, each with its own (possibly stale) reference, combines exactly to attention over
    all keys - also when one share sees no key at all, and with a ragged last tile."""
    rng = np.random.default_rng(k)
    n_keys, tile = 8 * 16 + 5, 8           # 17 tiles, the last one ragged
    q = rng.standard_normal((2, 2, 24, 16)).astype(np.float32)
    kk, v = (rng.standard_normal((2, 2, n_keys, 16)).astype(np.float32) for _ in range(2))
    shares = O.split_key_shares((n_keys + tile - 1) // tile, k)
    assert shares[0][0] == 0 and shares[-1][1] == 17 and all(a[1] == b[0] for a, b in zip(shares, shares[1:]))
    whole, whole_lse = O.sdpa_with_lse(q, kk, v)
    out, lse = O.combine_key_shares(q, kk, v, shares, tile=tile)
    np.testing.assert_allclose(out, whole, rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(lse, whole_lse, rtol=2e-5, atol=2e-6)
    # references that lag behind the true maximum by up to 2^8 (as the kernel's may) change nothing
    out_s, lse_s = O.combine_key_shares(q, kk, v, shares, tile=tile, stale=[0.7 * i for i in range(k)])
    np.testing.assert_allclose(out_s, whole, rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(lse_s, whole_lse, rtol=2e-5, atol=2e-6)
    # every key of the second share masked, and batch element 1 without any key at all
    mask = rng.random((2, n_keys)) < 0.7
    mask[0, shares[1][0] * tile:shares[1][1] * tile] = False
    mask[1] = False
    whole, whole_lse = O.sdpa_with_lse(q, kk, v, key_mask=mask)
    out, lse = O.combine_key_shares(q, kk, v, shares, tile=tile, key_mask=mask)
    np.testing.assert_allclose(out, whole, rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(lse[0], whole_lse[0], rtol=2e-5, atol=2e-6)
    assert np.isneginf(lse[1]).all() and not out[1].any()
