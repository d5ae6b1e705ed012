"""Host-side logic without a GPU: the exchange plan against the reference's all-to-all layout,
the mesh helper and the shard helpers over gloo (world size 2 and 4), and the cache's step
bookkeeping."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import cp_attention_oracle as O


def _simulate_plan(U, R, H, s, d=8):
    """Move numpy data exactly as CpPlan.push_jobs prescribes and return, per rank, the staged
    (q, k, v) as [b, hl, chunks*s, d] in chunk-slot order."""
    from paraattention_b200._cp_engine import CpPlan

    W = U * R
    rng = np.random.default_rng(U * 100 + R)
    local = {n: [rng.standard_normal((1, H, s, d)).astype(np.float32) for _ in range(W)] for n in "qkv"}
    hl = H // U
    stage = {n: [[None] * (U if n == "q" else W) for _ in range(W)] for n in "qkv"}
    for g in range(W):
        plan = CpPlan(U, R, g % U, g // U, H)
        assert plan.rank == g
        for job in plan.push_jobs():
            stage[job.tensor][job.dest][job.chunk] = local[job.tensor][g][:, job.head0:job.head0 + job.heads]
    for n in "qkv":
        for g in range(W):
            assert all(x is not None for x in stage[n][g]), "a staging slot was never filled"
    return local, stage, hl


@pytest.mark.parametrize("U,R", [(2, 1), (1, 2), (2, 2), (4, 2), (2, 4), (8, 1), (1, 8)])
def test_plan_reproduces_reference_layout(U, R):
    H, s = 8, 5
    W = U * R
    local, stage, hl = _simulate_plan(U, R, H, s)
    from paraattention_b200._cp_engine import CpPlan

    for r in range(R):
        group = [r * U + u for u in range(U)]
        # query side: staged Q of rank (u, r) == reference's Ulysses input all-to-all
        want_q = O.ulysses_input_all_to_all([local["q"][g] for g in group])
        for u, g in enumerate(group):
            got = np.concatenate(stage["q"][g], axis=2)
            np.testing.assert_array_equal(got, want_q[u])
    # key side: rank (u, r) must see head slice u of every rank's K/V exactly once
    for g in range(W):
        u = g % U
        for n in "kv":
            got = np.concatenate(stage[n][g], axis=2)
            want = np.concatenate([local[n][src][:, u * hl:(u + 1) * hl] for src in range(W)], axis=2)
            np.testing.assert_array_equal(got, want)
    # output side: every (rank, head) slot of every rank is written by exactly one q-chunk owner
    writes = {}
    for g in range(W):
        plan = CpPlan(U, R, g % U, g // U, H)
        for c in range(U):
            dest, head_off = plan.out_dest(c)
            for h in range(hl):
                key = (dest, head_off + h)
                assert key not in writes
                writes[key] = g
        assert sorted(plan.out_writers()) == sorted(r_ * U + u_ for r_ in [g // U] for u_ in range(U))
    assert len(writes) == W * H


def test_plan_attention_equals_oracle_unified():
    """Attention over the staged tensors (keys in chunk-slot order) equals the oracle's
    Ulysses-around-ring result: the fused exchange computes the same function."""
    U, R, H, s = 2, 2, 4, 6
    local, stage, hl = _simulate_plan(U, R, H, s)
    W = U * R
    want = O.unified_attention(local["q"], local["k"], local["v"], ulysses=U, ring=R)
    got = [np.zeros_like(local["q"][0]) for _ in range(W)]
    from paraattention_b200._cp_engine import CpPlan

    for g in range(W):
        plan = CpPlan(U, R, g % U, g // U, H)
        k = np.concatenate(stage["k"][g], axis=2)
        v = np.concatenate(stage["v"][g], axis=2)
        for c in range(U):
            out, _ = O.sdpa_with_lse(stage["q"][g][c], k, v)
            dest, head_off = plan.out_dest(c)
            got[dest][:, head_off:head_off + hl] = out
    for g in range(W):
        np.testing.assert_allclose(got[g], want[g], atol=1e-5)


def _gloo_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from paraattention_b200 import primitives as DP
    from paraattention_b200.context_parallel import init_context_parallel_mesh
    import paraattention_b200 as pa

    out = {}
    mesh = init_context_parallel_mesh("cpu", max_ring_dim_size=2)
    out["mesh_shape"] = tuple(mesh.mesh.shape)
    out["names"] = mesh.mesh_dim_names
    out["u"], out["r"] = DP.get_rank(mesh["ulysses"]), DP.get_rank(mesh["ring"])
    x = torch.arange(world * 6, dtype=torch.float32).reshape(1, world * 3, 2)
    mine = DP.get_assigned_chunk(x, dim=-2)
    out["chunk_ok"] = torch.equal(mine, x.chunk(world, dim=-2)[rank])
    out["gather_ok"] = torch.equal(DP.get_complete_tensor(mine, dim=-2), x)
    try:
        DP.get_assigned_chunk(torch.zeros(1, world * 3 + 1, 2), dim=-2)
        out["div_assert"] = False
    except AssertionError:
        out["div_assert"] = True
    # a multi-rank attention call on CPU tensors must fail loudly, never fall back
    q = torch.zeros(1, world, 4, 128, dtype=torch.bfloat16)
    try:
        pa.ulysses_attn_func(q, q, q)
        out["cpu_refused"] = False
    except (AssertionError, NotImplementedError, RuntimeError):
        out["cpu_refused"] = True
    try:
        pa.ring_attn_func(q, q, q, attn_mask=torch.ones(4, 4, dtype=torch.bool))
        out["mask_assert"] = False
    except AssertionError:
        out["mask_assert"] = True
    mode = pa.UnifiedAttnMode(mesh)
    out["mode_groups"] = (mode._ulysses_mesh is not None, mode._ring_mesh is not None)
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        ret.put(gathered)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_mesh_and_shard_helpers_over_gloo(world):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, 29800 + world, ret)) for r in range(world)]
    for p in procs:
        p.start()
    res = ret.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
    ring = 2
    uly = world // ring
    for rank, o in enumerate(res):
        assert o["mesh_shape"] == (1, ring, uly) and o["names"] == ("batch", "ring", "ulysses")
        assert (o["u"], o["r"]) == (rank % uly, rank // uly)  # ulysses is the fastest mesh dim
        assert o["chunk_ok"] and o["gather_ok"] and o["div_assert"] and o["cpu_refused"] and o["mask_assert"]
        assert o["mode_groups"] == (True, True)


def test_cache_context_step_bookkeeping():
    from paraattention_b200.first_block_cache import utils as fbc

    ctx = fbc.create_cache_context(residual_diff_threshold=0.1, warmup_steps=2)
    with fbc.cache_context(ctx):
        assert fbc.get_current_cache_context() is ctx
        for step in range(4):
            fbc.mark_step_begin()
            assert ctx.get_current_step() == step
            assert fbc.is_in_warmup() == (step < 2)
    assert fbc.get_current_cache_context() is None
    # alternate cache: the flag flips every call starting from True, steps count on the non-alter call
    ctx = fbc.create_cache_context(enable_alter_cache=True, alter_residual_diff_threshold=0.3,
                                   residual_diff_threshold=0.1, num_inference_steps=10, slg_layers=[1], slg_end=0.5)
    seen = []
    for _ in range(4):
        ctx.mark_step_begin()
        ctx.set_buffer("x", len(seen))
        seen.append((ctx.is_alter_cache, ctx.executed_steps, ctx.get_residual_diff_threshold(),
                     ctx.slg_should_skip_block(1)))
    assert seen == [(False, 1, 0.1, False), (True, 1, 0.3, True), (False, 2, 0.1, False), (True, 2, 0.3, True)]
    assert set(ctx.buffers) == {"x", "x_alter"}
    # TaylorSeer: one extrapolator per cache (main / alter), stepped with the cache it belongs to
    ctx = fbc.create_cache_context(enable_taylorseer=True, enable_alter_cache=True,
                                   taylorseer_kwargs=dict(n_derivatives=3, warmup_steps=2, skip_interval_steps=3))
    for _ in range(3):
        ctx.mark_step_begin()
    assert (ctx.taylorseer.current_step, ctx.alter_taylorseer.current_step) == (1, 0)
    assert ctx.get_taylorseer() is ctx.taylorseer and ctx.taylorseer.ORDER == 4
    assert [ctx.taylorseer.should_compute_full(s) for s in range(8)] == [True, True, False, False, True, False, False, True]
    with pytest.raises(NotImplementedError):
        fbc.create_cache_context(enable_taylorseer=True, taylorseer_kwargs=dict(n_derivatives=9))
    with pytest.raises(RuntimeError):
        ctx.taylorseer.update(torch.zeros(8, dtype=torch.bfloat16))  # CPU tensor: no CPU path
    with pytest.raises(AssertionError):
        fbc.mark_step_begin()


def _trace_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    import torch.nn.functional as F

    dist.init_process_group("gloo", rank=rank, world_size=world)
    import paraattention_b200 as pa
    from paraattention_b200 import _cp_engine as E
    from paraattention_b200 import para_attn_interface as I

    # Tracing only: stand-ins let CPU tensors reach the context-parallel custom op, which is
    # CUDA-only, so running the traced graph must fail in the op and nowhere before it.
    I._kernel_can_run = lambda *a, **k: True
    E.get_engine = lambda group, U, R, u, r, device: ("engine", U, R, u, r)
    q = torch.randn(1, 2, 16, 128)
    mesh = dist.init_device_mesh("cpu", (1, 2), mesh_dim_names=("ring", "ulysses"))
    report = {}
    for name, mode in (("ulysses", pa.UlyssesAttnMode()), ("ring", pa.RingAttnMode()), ("unified", pa.UnifiedAttnMode(mesh))):
        graphs = []

        def backend(gm, inputs):
            graphs.append([str(n.target) for n in gm.graph.nodes if n.op == "call_function"])
            return gm.forward

        def fn(q, k, v):
            with mode:
                return F.scaled_dot_product_attention(q, k, v, is_causal=True)

        torch._dynamo.reset()
        try:
            torch.compile(fn, fullgraph=True, backend=backend)(q, q, q)
            err = "ran on CPU"
        except NotImplementedError as e:
            err = "op refused CPU" if "cp_attention_forward" in str(e) else f"NotImplementedError: {e}"
        except Exception as e:  # a tracing failure would land here
            err = f"{type(e).__name__}: {str(e)[:200]}"
        report[name] = (graphs, err)
    if rank == 0:
        ret.put(report)
    dist.barrier()
    dist.destroy_process_group()


def test_modes_trace_into_one_custom_op_with_fullgraph():
    """torch.compile(fullgraph=True) around `with <Mode>: F.scaled_dot_product_attention(...)` (the
    reference's tests/test_interface.py:97-98) must trace, on every rank, into a single graph whose
    only call is the context-parallel custom op."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_trace_worker, args=(r, 2, 29655, ret)) for r in range(2)]
    for p in procs:
        p.start()
    report = ret.get(timeout=600)
    for p in procs:
        p.join(timeout=60)
    for name, (graphs, err) in report.items():
        assert graphs == [["para_attn.cp_attention_forward.default"]], f"{name}: traced graphs {graphs} ({err})"
        assert err == "op refused CPU", f"{name}: {err}"


def test_key_mask_of_accepts_only_key_padding_masks():
    from paraattention_b200.ops import key_mask_of

    m = torch.rand(2, 1, 1, 10) < 0.5
    assert torch.equal(key_mask_of(m, 2, 10), m[:, 0, 0, :])
    assert torch.equal(key_mask_of(m[:1], 2, 10), m[:1, 0, 0, :].expand(2, 10))   # batch broadcast
    assert torch.equal(key_mask_of(m[0, 0, 0], 2, 10), m[0, 0, 0].expand(2, 10))  # 1-D mask
    assert key_mask_of(None, 2, 10) is None
    assert key_mask_of(m.float(), 2, 10) is None                     # additive masks are not key masks
    assert key_mask_of(m.expand(2, 4, 1, 10), 2, 10) is None         # per-head
    assert key_mask_of(m.expand(2, 1, 7, 10), 2, 10) is None         # per-query
    assert key_mask_of(m, 2, 11) is None and key_mask_of(m, 3, 10) is None


def test_causal_positions_and_mask_words_in_the_launch_arguments():
    """Chunk c of the sequence sits at c * rows, c = ring index * U + ulysses index: the order
    of the Ulysses all-to-all and of causal ring attention alike."""
    from paraattention_b200 import _cp_engine as E

    U, R, H, sq, D = 2, 3, 4, 100, 64
    plan = E.CpPlan(U, R, 1, 2, H)  # u = 1, r = 2 -> flat rank 5
    layout = E._make_layout(U * R, U, *E.stage_sizes(plan, 1, sq, sq, D, 2))
    buf = torch.zeros(layout.total, dtype=torch.uint8)
    ws = E.Workspace(layout, buf, [buf.data_ptr()] * (U * R), plan.rank)
    a = E.build_attention_args(plan, ws, 0, (1, H, sq, D), torch.bfloat16, sq, 0.125, 7, 1000, None, is_causal=True)
    assert a.is_causal == 1 and a.head_dim == D and a.heads == H // U
    assert (a.n_q_chunks, a.q_first, a.n_kv_chunks, a.kv_first) == (U, 1, U * R, 5)
    assert list(a.q_pos)[:U] == [4 * sq, 5 * sq]
    assert list(a.kv_pos)[:U * R] == [c * sq for c in range(U * R)]
    assert a.key_bits is None
    plain = E.build_attention_args(plan, ws, 0, (1, H, sq, D), torch.bfloat16, sq, 0.125, 7, 1000, None)
    assert plain.is_causal == 0 and list(plain.q_pos) == [0] * 8
    bits = torch.zeros(1, U * R, 2, dtype=torch.int64)
    masked = E.build_attention_args(plan, ws, 0, (1, H, sq, D), torch.bfloat16, sq, 0.125, 7, 1000, None, key_bits=bits)
    assert masked.key_bits == bits.data_ptr()
    jobs = E.build_push_args(plan, ws, 0, *(torch.zeros(1, H, sq, D, dtype=torch.bfloat16),) * 3, 4)
    assert {jobs.jobs[i].head_dim for i in range(jobs.n_jobs)} == {D} and jobs.first_dest == plan.rank


def test_host_pipeline_group_choice():
    from paraattention_b200.host_io import _default_groups

    assert _default_groups(24, 32760, 1, 1, 1) == 12     # one GPU: launches overlap, 1.5 waves are enough
    assert _default_groups(24, 16380, 1, 2, 2) == 4      # two ranks: 4 x 3 rounds against 11 unsplit
    assert _default_groups(24, 8190, 1, 4, 4) == 3       # four ranks: 3 x 2 rounds = the 6 unsplit
    assert _default_groups(24, 4095, 1, 8, 8) == 3       # eight ranks: 3 x 128 CTAs = the three rounds of 384
    assert _default_groups(24, 576, 1, 8, 8) == 1        # small problem on eight ranks: one call
    assert _default_groups(24, 4608, 1, 1, 1) == 1       # small problem: one launch
    for heads, U in ((24, 2), (40, 8), (6, 3)):
        g = _default_groups(heads, 20000, 1, U, U)
        assert heads % g == 0 and (heads // g) % U == 0


def _adapter_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    from paraattention_b200 import config
    from paraattention_b200.context_parallel.diffusers_adapters import parallelize_transformer

    config.attention.allow_sdpa_fallback = True  # fp32 on CPU is outside the kernel's coverage
    from paraattention_b200.shape_models import FluxShapedPipeline, FluxShapedTransformer2DModel
    from paraattention_b200.shape_models_hunyuan import HunyuanVideoShapedTransformer3DModel
    from paraattention_b200.shape_models_video import WanShapedTransformer3DModel

    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, 16, 2, 8, 8, generator=g)
    enc, pooled, t = torch.randn(1, 8, 64, generator=g), torch.randn(1, 32, generator=g), torch.tensor([500.0])
    errs = {}
    torch.manual_seed(0)
    wan = WanShapedTransformer3DModel(dim=256, num_layers=2, ffn_dim=512, text_dim=64)
    want = wan(x, t, enc).sample
    errs["wan"] = (parallelize_transformer(wan)(x, t, enc).sample - want).abs().max().item()
    torch.manual_seed(0)
    hun = HunyuanVideoShapedTransformer3DModel(dim=256, num_layers=2, num_single_layers=2, text_dim=64,
                                               pooled_projection_dim=32)
    mask, guidance = torch.ones(1, 8), torch.tensor([6.0])
    want = hun(x, t, enc, mask, pooled, guidance=guidance).sample
    errs["hunyuan"] = (parallelize_transformer(hun)(x, t, enc, mask, pooled, guidance=guidance).sample - want).abs().max().item()
    torch.manual_seed(0)
    flux = FluxShapedTransformer2DModel(dim=256, num_layers=2, num_single_layers=2, joint_attention_dim=64)
    pipe = FluxShapedPipeline(flux, text_tokens=8, latent_hw=(4, 4))
    want = pipe(num_inference_steps=2, generator=torch.Generator().manual_seed(3))
    parallelize_transformer(flux)
    errs["flux"] = (pipe(num_inference_steps=2, generator=torch.Generator().manual_seed(3)) - want).abs().max().item()
    ret.put(errs)
    dist.destroy_process_group()


def test_adapters_restate_the_forward_exactly_on_one_rank():
    """With a single rank every shard is the whole tensor, so the adapters' re-stated forwards
    (patch grid, embeddings, output projection, un-patchify) must reproduce the models' own
    outputs; runs on CPU in fp32 with the SDPA fallback switched on for the test."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    p = ctx.Process(target=_adapter_worker, args=(0, 1, 29656, ret))
    p.start()
    errs = ret.get(timeout=300)
    p.join(timeout=60)
    for name, e in errs.items():
        assert e < 1e-5, f"{name}: adapter output differs from the model's by {e:.3e}"


def test_attention_outside_the_kernel_is_refused_unless_opted_in():
    """Inside a mode an attention call the sm_100a kernel does not cover (here: CPU fp32) raises;
    only config.attention.allow_sdpa_fallback hands it to PyTorch's SDPA."""
    import torch.nn.functional as F

    import paraattention_b200 as pa
    from paraattention_b200 import config
    from paraattention_b200.para_attn_interface import _local_attention, in_batch_attn_func

    q = torch.randn(2, 2, 8, 64)
    with pytest.raises(NotImplementedError, match="allow_sdpa_fallback"):
        _local_attention(q, q, q)
    with pytest.raises(NotImplementedError, match="allow_sdpa_fallback"):
        with pa.InBatchAttnMode():
            F.scaled_dot_product_attention(q, q, q)
    with config.patch({"attention.allow_sdpa_fallback": True}):
        torch.testing.assert_close(_local_attention(q, q, q), F.scaled_dot_product_attention(q, q, q))
        # every batch element attends to the keys of all batch elements
        folded = q.transpose(0, 1).reshape(1, 2, 16, 64)
        want = F.scaled_dot_product_attention(folded, folded, folded).reshape(2, 2, 8, 64).transpose(0, 1)
        torch.testing.assert_close(in_batch_attn_func(q, q, q), want)


def test_unified_mode_refuses_a_custom_attn_func_on_a_parallel_mesh(monkeypatch):
    """The reference forwards attn_func to ulysses_attn_func; with the exchange fused into the
    kernel a foreign attention function cannot be wrapped, and dropping it silently would be
    worse than saying so."""
    import paraattention_b200 as pa
    from paraattention_b200 import primitives as DP

    mode = pa.UnifiedAttnMode.__new__(pa.UnifiedAttnMode)
    mode._ulysses_mesh, mode._ring_mesh, mode._flat_group = object(), None, None
    mode._skip_small_kv, mode._attn_func = False, (lambda *a, **k: None)
    monkeypatch.setattr(DP, "get_world_size", lambda group=None: 2)
    q = torch.randn(1, 2, 4, 64)
    with pytest.raises(NotImplementedError, match="custom attn_func"):
        mode._call_attn_func(q, q, q)


def test_status_mirror_surfaces_a_sticky_timeout_and_resets():
    """A device status word that an earlier launch set shows up as PaError(PA_ETIMEDOUT) on the
    next check without any device synchronisation on the call path; reset() clears it."""
    from paraattention_b200 import _lib as L
    from paraattention_b200._status import StatusMirror

    word = torch.zeros(1, dtype=torch.int32)
    m = StatusMirror(word)
    m.check()  # nothing reported
    word[0] = L.PA_DEV_TIMEOUT_KV  # what a kernel's bounded wait writes when it gives up
    m.check()  # the mirror has not been refreshed yet: still quiet
    m.refresh()
    with pytest.raises(L.PaError, match="key/value chunk") as e:
        m.check()
    assert e.value.code == L.PA_ETIMEDOUT
    with pytest.raises(L.PaError):
        m.check()  # sticky until reset
    m.reset()
    m.check()
    assert int(word[0]) == 0


def test_taylorseer_schedule_matches_the_reference_rule():
    """Warm-up steps are computed, then every skip_interval-th step; an explicit map wins."""
    from paraattention_b200.first_block_cache.taylorseer import TaylorSeer

    seer = TaylorSeer(n_derivatives=3, warmup_steps=2, skip_interval_steps=3)
    assert seer.ORDER == 4 and set(seer.state) == {"dY_prev", "dY_current"}
    assert [seer.should_compute_full(s) for s in range(9)] == [True, True, False, False, True, False, False, True, False]
    mapped = TaylorSeer(compute_step_map=[True, False, True])
    assert [mapped.should_compute_full(s) for s in range(3)] == [True, False, True]
    with pytest.raises(NotImplementedError):
        TaylorSeer(n_derivatives=5)


def _parallel_decision_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from paraattention_b200.first_block_cache.utils import _decide

    rng = np.random.default_rng(7)
    numel = 4096
    cases = []
    for thr in (0.05, 0.08, 0.12):
        for _ in range(6):
            # per-rank fp32 sums as the cache kernel leaves them, chosen so that ratios land on both sides of thr
            sd = rng.uniform(0.02, 0.2, size=world) * numel
            sp = rng.uniform(0.8, 1.2, size=world) * numel
            cases.append((thr, sd, sp))
    out = []
    for thr, sd, sp in cases:
        md = O.bf16_round(np.float32(sd[rank] / numel))
        mp_ = O.bf16_round(np.float32(sp[rank] / numel))
        result = torch.tensor([sd[rank], sp[rank], float(md), float(mp_), 0.0], dtype=torch.float32)
        got = _decide(result, torch.bfloat16, thr, parallelized=True)
        want = O.fbc_decision(list(sd), list(sp), numel, thr)
        out.append((got, want))
    if rank == 0:
        ret.put(out)
    dist.barrier()
    dist.destroy_process_group()


def test_parallel_cache_decision_matches_the_oracle_over_gloo():
    """_decide(parallelized=True): each rank's two rounded means are averaged over the group before
    the bf16 division (src/para_attn/first_block_cache/utils.py:230-232); two ranks over gloo
    against the oracle's restatement, on thresholds that split the cases."""
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_parallel_decision_worker, args=(r, 2, 29671, ret)) for r in range(2)]
    for p in procs:
        p.start()
    out = ret.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
    assert all(g == w for g, w in out), out
    assert {w for _, w in out} == {True, False}, "the cases must cover both outcomes"


def test_peer_gather_block_plan():
    """A shard is copied as whole rows of 256 or 128 bytes, one block per index of the dims in
    front of the gather dim; shapes without whole rows are left to the collective library."""
    from paraattention_b200._peer_gather import plan_blocks

    assert plan_blocks((1, 576, 64), -2, 2) == (1, 288, 128)      # FLUX-shaped output shard on 8 ranks
    assert plan_blocks((2, 576, 64), 1, 2) == (2, 288, 128)       # one block per batch element
    assert plan_blocks((1, 4095, 64), 1, 2) == (1, 4095, 64)      # 128-byte rows when 256 do not divide
    assert plan_blocks((1, 14850, 64), 1, 4) == (1, 14850, 128)   # fp32: twice the 16-bit units
    assert plan_blocks((4, 64, 8, 16), 0, 2) == (1, 256, 128)     # gather along dim 0: one block
    assert plan_blocks((2, 7, 3), 1, 2) is None
