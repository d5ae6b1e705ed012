"""Context-parallel path on the GPU: exchange (pa_cp_push) + chunked attention
(pa_cp_attn_fwd) + output scatter, checked against the reference's own outputs (golden
fixtures) and the oracle.

One-GPU tests emulate all ranks of a mesh with ``helpers.LocalCluster`` (every rank's buffers
live on the same device; the launches are the product's own). Tests that need real peers
spawn one process per GPU and are skipped when fewer than two GPUs are visible.
"""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import cp_attention_oracle as O
from helpers import LocalCluster, assert_attention_close, bf16_from_bits, seeded_qkv

pytestmark = pytest.mark.gpu


def _golden_shards(golden_dir, names, world):
    g = np.load(golden_dir / "cp_attention_w2.npz")
    return [[t.contiguous() for t in bf16_from_bits(g[n]).chunk(world, dim=-2)] for n in names]


@pytest.mark.parametrize("name,U,R", [("ulysses", 2, 1), ("ring", 1, 2)])
def test_world2_against_reference_outputs(golden_dir, name, U, R):
    g = np.load(golden_dir / "cp_attention_w2.npz")
    qs, ks, vs = _golden_shards(golden_dir, ("q", "k", "v"), 2)
    outs = LocalCluster(U, R).attention(qs, ks, vs)
    for rank in range(2):
        assert_attention_close(outs[rank], g[name][rank], f"{name} rank {rank}")


@pytest.mark.parametrize("name,U,R", [("ulysses_causal", 2, 1), ("ring_causal", 1, 2)])
def test_world2_causal_against_reference_outputs(golden_dir, name, U, R):
    g = np.load(golden_dir / "cp_attention_w2.npz")
    qs, ks, vs = _golden_shards(golden_dir, ("q", "k", "v"), 2)
    outs = LocalCluster(U, R).attention(qs, ks, vs, is_causal=True)
    for rank in range(2):
        assert_attention_close(outs[rank], g[name][rank], f"{name} rank {rank}")


@pytest.mark.parametrize("U,R,H,S", [(8, 1, 8, 8 * 300), (4, 2, 8, 8 * 131), (2, 4, 4, 8 * 257), (1, 8, 2, 8 * 129)])
def test_world8_meshes_causal_against_oracle(U, R, H, S):
    """Causal masking over the sharded sequence: equal to the oracle's composition of Ulysses
    and causal ring attention, and to plain causal attention over the whole sequence."""
    W = U * R
    q, k, v = seeded_qkv(1, H, S, S, seed=U * 10 + R + 100)
    qs, ks, vs = ([t.contiguous() for t in x.chunk(W, dim=-2)] for x in (q, k, v))
    cluster = LocalCluster(U, R)
    outs = cluster.attention(qs, ks, vs, is_causal=True)
    ref = O.unified_attention([t.float().cpu().numpy() for t in qs], [t.float().cpu().numpy() for t in ks],
                              [t.float().cpu().numpy() for t in vs], ulysses=U, ring=R, is_causal=True)
    whole, _ = O.sdpa_with_lse(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(),
                               is_causal=True)
    for rank in range(W):
        assert_attention_close(outs[rank], ref[rank], f"causal {U}x{R} rank {rank}")
    assert_attention_close(torch.cat(outs, dim=-2), whole, f"causal {U}x{R} whole sequence")
    # non-causal calls in between keep working on the same buffers and counters
    plain = cluster.attention(qs, ks, vs)
    again = cluster.attention(qs, ks, vs, is_causal=True)
    for rank in range(W):
        assert torch.equal(again[rank], outs[rank]) and not torch.equal(plain[rank], outs[rank])


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("U,R,H,S", [(2, 1, 4, 2 * 515), (1, 2, 2, 2 * 300), (2, 2, 4, 4 * 257), (4, 2, 8, 8 * 131)])
def test_head_dim_64_meshes_against_oracle(U, R, H, S, causal):
    W = U * R
    q, k, v = seeded_qkv(1, H, S, S, D=64, seed=U * 10 + R + 200)
    qs, ks, vs = ([t.contiguous() for t in x.chunk(W, dim=-2)] for x in (q, k, v))
    outs = LocalCluster(U, R).attention(qs, ks, vs, is_causal=causal)
    ref = O.unified_attention([t.float().cpu().numpy() for t in qs], [t.float().cpu().numpy() for t in ks],
                              [t.float().cpu().numpy() for t in vs], ulysses=U, ring=R, is_causal=causal)
    for rank in range(W):
        assert_attention_close(outs[rank], ref[rank], f"D64 causal={causal} {U}x{R} rank {rank}")


@pytest.mark.parametrize("U,R,H,S,D", [(2, 1, 4, 2 * 515, 128), (1, 2, 2, 2 * 300, 128), (2, 2, 4, 4 * 257, 128),
                                       (4, 2, 8, 8 * 131, 64), (1, 8, 2, 8 * 129, 128)])
def test_key_mask_meshes_against_oracle(U, R, H, S, D):
    """A key-padding mask over the keys of all ranks (chunks in flat-rank order), on Ulysses, ring
    and mixed meshes: equal to masked attention over the whole sequence."""
    W = U * R
    B = 2
    q, k, v = seeded_qkv(B, H, S, S, D=D, seed=U * 10 + R + 300)
    g = torch.Generator().manual_seed(S)
    mask = torch.rand(B, S, generator=g) < 0.6
    mask[1, S - S // W - 7:] = False  # the last rank's keys are all padding for batch element 1
    qs, ks, vs = ([t.contiguous() for t in x.chunk(W, dim=-2)] for x in (q, k, v))
    outs = LocalCluster(U, R).attention(qs, ks, vs, key_mask=mask.cuda())
    whole, _ = O.sdpa_with_lse(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(),
                               key_mask=mask.numpy())
    assert_attention_close(torch.cat(outs, dim=-2), whole, f"key mask {U}x{R}")


@pytest.mark.parametrize("name,U,R", [("ulysses_short_kv", 2, 1), ("ring_short_kv", 1, 2)])
def test_world2_short_kv_against_reference_outputs(golden_dir, name, U, R):
    g = np.load(golden_dir / "cp_attention_w2.npz")
    qs, ks, vs = _golden_shards(golden_dir, ("q2", "k2", "v2"), 2)
    outs = LocalCluster(U, R).attention(qs, ks, vs)
    for rank in range(2):
        assert_attention_close(outs[rank], g[name][rank], f"{name} rank {rank}")


@pytest.mark.parametrize("name,U,R", [("unified_2x2", 2, 2), ("ring4", 1, 4)])
def test_world4_against_reference_outputs(golden_dir, name, U, R):
    g = np.load(golden_dir / "cp_attention_w4.npz")
    qs, ks, vs = _golden_shards(golden_dir, ("q", "k", "v"), 4)
    outs = LocalCluster(U, R).attention(qs, ks, vs)
    for rank in range(4):
        assert_attention_close(outs[rank], g[name][rank], f"{name} rank {rank}")


@pytest.mark.parametrize("U,R,H,S", [(8, 1, 8, 8 * 300), (4, 2, 8, 8 * 131), (2, 4, 4, 8 * 257), (1, 8, 2, 8 * 129)])
def test_world8_meshes_against_oracle(U, R, H, S):
    W = U * R
    q, k, v = seeded_qkv(1, H, S, S, seed=U * 10 + R)
    qs, ks, vs = ([t.contiguous() for t in x.chunk(W, dim=-2)] for x in (q, k, v))
    cluster = LocalCluster(U, R)
    outs = cluster.attention(qs, ks, vs)
    ref = O.unified_attention([t.float().cpu().numpy() for t in qs], [t.float().cpu().numpy() for t in ks],
                              [t.float().cpu().numpy() for t in vs], ulysses=U, ring=R)
    for rank in range(W):
        assert_attention_close(outs[rank], ref[rank], f"{U}x{R} rank {rank}")
    # a second and third call reuse the double-buffered staging and the monotonic counters
    for rep in range(2):
        outs2 = cluster.attention(qs, ks, vs)
        for rank in range(W):
            assert torch.equal(outs2[rank], outs[rank]), f"call {rep + 2} differs on rank {rank}"


def _split_ws():
    from paraattention_b200 import _lib as L

    return torch.empty(int(L.load().pa_attn_workspace_bytes()), dtype=torch.uint8, device="cuda")


@pytest.mark.parametrize("U,R,H,S,D,masked", [(2, 1, 4, 2 * 2048, 128, False), (1, 4, 2, 4 * 1100, 128, False),
                                              (2, 2, 4, 4 * 1030, 64, False), (2, 2, 4, 4 * 1030, 128, True)])
def test_split_last_wave_on_meshes_against_oracle(U, R, H, S, D, masked):
    """Chunked launches whose units are shared by several CTAs (a workspace is given): the shares'
    tile ranges cross the chunks of different source ranks, ragged chunk ends included."""
    W = U * R
    q, k, v = seeded_qkv(1, H, S, S, D=D, seed=U * 10 + R + 77)
    mask = None
    if masked:
        g = torch.Generator().manual_seed(S)
        mask = torch.rand(1, S, generator=g) < 0.7
        mask[0, S // W: 2 * (S // W)] = False  # rank 1's keys are all padding
    qs, ks, vs = ([t.contiguous() for t in x.chunk(W, dim=-2)] for x in (q, k, v))
    cluster = LocalCluster(U, R)
    plain = cluster.attention(qs, ks, vs, key_mask=None if mask is None else mask.cuda())
    cluster.split_ws = _split_ws()
    outs = cluster.attention(qs, ks, vs, key_mask=None if mask is None else mask.cuda())
    again = cluster.attention(qs, ks, vs, key_mask=None if mask is None else mask.cuda())
    whole, _ = O.sdpa_with_lse(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(),
                               key_mask=None if mask is None else mask.numpy())
    assert_attention_close(torch.cat(outs, dim=-2), whole, f"split {U}x{R}")
    for rank in range(W):
        assert torch.equal(again[rank], outs[rank]), "the order in which shares are combined is fixed"
        assert torch.allclose(outs[rank].float(), plain[rank].float(), rtol=2e-2, atol=2e-3)
    # the split did happen: a one-CTA result differs in the last bit somewhere
    assert any(not torch.equal(outs[rank], plain[rank]) for rank in range(W))


def test_sharded_equals_single_device_full_size_shard():
    """The reference's pinned contract (tests/test_interface.py:70): the sharded result is
    chunk r of single-device attention. Shard length 4095 = 32760 / 8 is not a tile multiple."""
    U, R, H, s = 2, 2, 4, 4095
    q, k, v = seeded_qkv(1, H, 4 * s, 4 * s, seed=2, scale=0.5)
    qs, ks, vs = ([t.contiguous() for t in x.chunk(4, dim=-2)] for x in (q, k, v))
    outs = LocalCluster(U, R).attention(qs, ks, vs)
    from paraattention_b200 import ops

    single = ops.attention_forward(q, k, v)
    full = torch.cat(outs, dim=-2)
    assert (full.float() - single.float()).abs().max().item() <= 1e-3 * 4  # atol 1e-3 * world_size
    idx = torch.arange(0, 4 * s, 997, device="cuda")
    ref, _ = O.sdpa_with_lse(q[:, :, idx].float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy())
    assert_attention_close(full[:, :, idx], ref, "sampled rows")


@pytest.mark.parametrize("B,H,S,ctas", [(1, 2, 300, 4), (2, 3, 4095, 16), (1, 1, 100, 64)])
def test_fused_push_inside_attention_launch(B, H, S, ctas):
    """The form multi-GPU runs use: the leading CTAs of the attention grid do the exchange.
    With one rank everything a CTA waits for is produced by CTAs of the same launch."""
    q, k, v = seeded_qkv(B, H, S, S, seed=S, bshd=True)
    cluster = LocalCluster(1, 1)
    ref, _ = O.sdpa_with_lse(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy())
    first = None
    for rep in range(3):  # both staging parities and the monotonic counters
        out = cluster.attention_fused_single_rank(q, k, v, ctas=ctas)
        assert_attention_close(out, ref, f"fused push call {rep}")
        first = out if first is None else first
        assert torch.equal(out, first)


def test_wait_runs_out_and_reports_status():
    """A chunk whose arrival counter nothing sets: the bounded wait gives up, the status word
    says which wait it was, and the context stays usable."""
    from paraattention_b200 import _cp_engine as E
    from paraattention_b200 import _lib as L

    plan = E.CpPlan(1, 2, 0, 0, 2)
    B, H, s, D = 1, 2, 128, 128
    layout = E._make_layout(2, 1, *E.stage_sizes(plan, B, s, s, D, 2))
    buf = torch.zeros(layout.total, dtype=torch.uint8, device="cuda")
    ws = E.Workspace(layout, buf, [buf.data_ptr(), buf.data_ptr()], 0)
    out = torch.empty((B, s, H, D), dtype=torch.bfloat16, device="cuda").transpose(1, 2)
    stream = torch.cuda.current_stream().cuda_stream
    # expect one arrival per chunk, but nobody pushes: 2 ms budget
    E.launch_attention(plan, ws, 0, (B, H, s, D), torch.bfloat16, s, 0.1, 1, 2_000_000, stream, out)
    torch.cuda.synchronize()
    code = int(ws.status_tensor().item())
    assert code in (L.PA_DEV_TIMEOUT_Q, L.PA_DEV_TIMEOUT_KV), f"unexpected status {code}"
    # the device is still healthy: a normal launch afterwards works
    q, k, v = seeded_qkv(1, 1, 128, 128)
    from paraattention_b200 import ops

    assert torch.isfinite(ops.attention_forward(q, k, v).float()).all()


def _mp_worker(rank, world, port, mode, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import paraattention_b200 as pa

    H, S = 4, world * 515
    q, k, v = seeded_qkv(1, H, S, S, D=64 if "d64" in mode else 128, seed=21, device="cpu")
    qs, ks, vs = (x.chunk(world, dim=-2)[rank].cuda() for x in (q, k, v))
    results = {}
    for rep in range(3):
        if mode == "ulysses":
            out = pa.ulysses_attn_func(qs, ks, vs)
        elif mode == "ring":
            out = pa.ring_attn_func(qs, ks, vs)
        elif mode == "ring_causal":
            out = pa.ring_attn_func(qs, ks, vs, is_causal=True)
        elif mode == "ulysses_causal":
            out = pa.ulysses_attn_func(qs, ks, vs, is_causal=True)
        elif mode in ("ulysses_mask", "ring_mask"):
            mask = (torch.rand(1, 1, 1, S, generator=torch.Generator().manual_seed(5)) < 0.6).cuda()
            fn = pa.ulysses_attn_func if mode == "ulysses_mask" else pa.ring_attn_func
            out = fn(qs, ks, vs, attn_mask=mask)
        elif mode == "compiled_ulysses_causal":
            if rep == 0:
                attn_mode = pa.UlyssesAttnMode()

                def fn(a, b, c):
                    with attn_mode:
                        return torch.nn.functional.scaled_dot_product_attention(a, b, c, is_causal=True)

                compiled = torch.compile(fn, fullgraph=True, backend="aot_eager")
            out = compiled(qs, ks, vs)
        elif mode == "ring_d64_causal":
            with pa.RingAttnMode():
                out = torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True)
        elif mode == "ulysses_d64":
            with pa.UlyssesAttnMode():
                out = torch.nn.functional.scaled_dot_product_attention(qs, ks, vs)
        else:
            mesh = dist.init_device_mesh("cuda", (world // 2, 2), mesh_dim_names=("ring", "ulysses")) if rep == 0 else mesh
            with pa.UnifiedAttnMode(mesh):
                out = torch.nn.functional.scaled_dot_product_attention(qs, ks, vs)
        results[rep] = out.float().cpu()
    torch.cuda.synchronize()
    pa.check_device_status()
    gathered = [None] * world
    dist.all_gather_object(gathered, results[2].numpy())
    same = all(torch.equal(results[0], results[i]) for i in (1, 2))
    if rank == 0:
        ret.put((np.concatenate(gathered, axis=-2), same))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["ulysses", "ring", "unified", "ring_causal", "ulysses_causal", "ring_d64_causal",
                                  "ulysses_d64", "ulysses_mask", "ring_mask", "compiled_ulysses_causal"])
def test_multi_gpu_processes(mode):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 4 if (mode == "unified" and n >= 4) else 2
    if mode == "unified" and n < 4:
        pytest.skip("unified 2x2 needs 4 GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = 29700 + {"ulysses": 1, "ring": 2, "unified": 3, "ring_causal": 4, "ulysses_causal": 5, "ring_d64_causal": 6,
                    "ulysses_d64": 7, "ulysses_mask": 8, "ring_mask": 9,
                    "compiled_ulysses_causal": 10}[mode]
    procs = [ctx.Process(target=_mp_worker, args=(r, world, port, mode, ret)) for r in range(world)]
    for p in procs:
        p.start()
    full, same = ret.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
    assert same, "repeated calls gave different results"
    H, S = 4, world * 515
    q, k, v = seeded_qkv(1, H, S, S, D=64 if "d64" in mode else 128, seed=21, device="cpu")
    key_mask = None
    if mode.endswith("mask"):
        key_mask = (torch.rand(1, 1, 1, S, generator=torch.Generator().manual_seed(5)) < 0.6)[:, 0, 0, :].numpy()
    ref, _ = O.sdpa_with_lse(q.float().numpy(), k.float().numpy(), v.float().numpy(),
                             is_causal=mode.endswith("causal"), key_mask=key_mask)
    assert_attention_close(torch.from_numpy(full), ref, f"{mode} world {world}")


def _gather_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import paraattention_b200 as pa
    from paraattention_b200 import config
    from paraattention_b200 import primitives as DP

    ok = True
    cases = [((2, 576, 64), -2, torch.bfloat16), ((1, 300, 128), 1, torch.float32), ((4, 64, 8, 16), 0, torch.float16),
             ((1, 4095, 64), -2, torch.bfloat16), ((2, 7, 3), 1, torch.bfloat16)]  # the last one has no whole rows: NCCL path
    for rep in range(3):  # both parities of the result buffers and the growing counters
        for shape, dim, dtype in cases:
            g = torch.Generator().manual_seed(rank * 100 + rep)
            shard = torch.randn(shape, generator=g).to(dtype).cuda()
            got = DP.get_complete_tensor(shard, dim=dim)
            with config.patch({"cp.peer_gather": False}):
                want = DP.get_complete_tensor(shard, dim=dim)
            ok = ok and got.shape == want.shape and torch.equal(got, want)
            # and against the shards themselves
            parts = [torch.randn(shape, generator=torch.Generator().manual_seed(r * 100 + rep)).to(dtype) for r in range(world)]
            ok = ok and torch.equal(got.cpu(), torch.cat(parts, dim=dim))
    torch.cuda.synchronize()
    pa.check_device_status()
    if rank == 0:
        ret.put(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_get_complete_tensor_as_peer_stores_on_real_peers():
    """The gather at the exit of a parallelised forward (src/para_attn/primitives.py:139-148) through
    peer stores: identical to the NCCL all_gather form and to the concatenated shards."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    world = 2
    procs = [ctx.Process(target=_gather_worker, args=(r, world, 29731, ret)) for r in range(world)]
    for p in procs:
        p.start()
    ok = ret.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
    assert ok
