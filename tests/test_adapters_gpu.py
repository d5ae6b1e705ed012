"""The model adapters (parallelize_* and apply_cache_on_*) driven by shape-only transformers.

Single GPU: the cache adapters. Two GPUs (one process each, skipped otherwise): the
context-parallel adapters against the same model run unsharded."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DT = torch.bfloat16


def _tiny_flux(seed=0):
    from paraattention_b200.shape_models import FluxShapedTransformer2DModel

    torch.manual_seed(seed)
    return FluxShapedTransformer2DModel(dim=256, num_layers=2, num_single_layers=2, joint_attention_dim=64).to("cuda", DT)


def _tiny_wan(seed=0):
    from paraattention_b200.shape_models_video import WanShapedTransformer3DModel

    torch.manual_seed(seed)
    return WanShapedTransformer3DModel(dim=256, num_layers=2, ffn_dim=512, text_dim=64).to("cuda", DT)


def _tiny_hunyuan(seed=0):
    from paraattention_b200.shape_models_hunyuan import HunyuanVideoShapedTransformer3DModel

    torch.manual_seed(seed)
    return HunyuanVideoShapedTransformer3DModel(dim=256, num_layers=2, num_single_layers=2, text_dim=64,
                                                pooled_projection_dim=32).to("cuda", DT)


def _video_inputs(seed=1):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(1, 16, 2, 8, 8, generator=g).to("cuda", DT)      # -> 2*4*4 = 32 tokens
    enc = torch.randn(1, 8, 64, generator=g).to("cuda", DT)
    pooled = torch.randn(1, 32, generator=g).to("cuda", DT)
    return x, enc, pooled


def _count_calls(blocks):
    counter = {"n": 0}
    for b in blocks:
        b.register_forward_hook(lambda *a, c=counter: c.__setitem__("n", c["n"] + 1))
    return counter


def test_flux_cache_on_pipe_threshold_zero_is_identity_and_large_threshold_skips():
    from paraattention_b200.first_block_cache.diffusers_adapters import apply_cache_on_pipe
    from paraattention_b200.shape_models import FluxShapedPipeline

    class FluxShapedPipelineA(FluxShapedPipeline):  # separate classes: the adapter patches __call__ per class
        pass

    class FluxShapedPipelineB(FluxShapedPipeline):
        pass

    plain = FluxShapedPipeline(_tiny_flux(), text_tokens=8, latent_hw=(4, 4))(num_inference_steps=4)
    pipe0 = apply_cache_on_pipe(FluxShapedPipelineA(_tiny_flux(), text_tokens=8, latent_hw=(4, 4)),
                                residual_diff_threshold=0.0)
    assert torch.equal(pipe0(num_inference_steps=4), plain)
    model = _tiny_flux()
    later_blocks = _count_calls(list(model.transformer_blocks[1:]) + list(model.single_transformer_blocks))
    pipe1 = apply_cache_on_pipe(FluxShapedPipelineB(model, text_tokens=8, latent_hw=(4, 4)), residual_diff_threshold=1e3)
    out = pipe1(num_inference_steps=4)
    assert later_blocks["n"] == 3, "only the first step should run the blocks behind the first one"
    assert torch.isfinite(out.float()).all() and not torch.equal(out, plain)
    # applying twice changes nothing
    assert apply_cache_on_pipe(pipe1, residual_diff_threshold=1e3) is pipe1


def test_wan_and_hunyuan_cache_on_transformer():
    from paraattention_b200.first_block_cache import utils as fbc
    from paraattention_b200.first_block_cache.diffusers_adapters import apply_cache_on_transformer

    x, enc, pooled = _video_inputs()
    t = torch.tensor([500.0], device="cuda")
    wan = _tiny_wan()
    want = wan(x, t, enc).sample
    apply_cache_on_transformer(wan)
    with fbc.cache_context(fbc.create_cache_context(residual_diff_threshold=0.0)):
        assert torch.equal(wan(x, t, enc).sample, want)
    with fbc.cache_context(fbc.create_cache_context(residual_diff_threshold=1e3)):
        first = wan(x, t, enc).sample
        second = wan(x, t, enc).sample  # same input: residual unchanged -> hit, output reproduced from the cache
    assert torch.equal(first, want)
    assert (second.float() - want.float()).abs().max().item() < 0.1

    hun = _tiny_hunyuan()
    mask = torch.ones(1, 8, device="cuda")
    g = torch.tensor([6.0], device="cuda")
    want = hun(x, t, enc, mask, pooled, guidance=g).sample
    apply_cache_on_transformer(hun)
    with fbc.cache_context(fbc.create_cache_context(residual_diff_threshold=0.0)):
        assert torch.equal(hun(x, t, enc, mask, pooled, guidance=g).sample, want)


def test_dispatch_by_class_name():
    from paraattention_b200.context_parallel.diffusers_adapters import parallelize_transformer
    from paraattention_b200.first_block_cache.diffusers_adapters import apply_cache_on_transformer

    class MochiThing(torch.nn.Module):
        pass

    class Other(torch.nn.Module):
        pass

    for fn in (parallelize_transformer, apply_cache_on_transformer):
        with pytest.raises(NotImplementedError):
            fn(MochiThing())
        with pytest.raises(ValueError):
            fn(Other())


def _cp_worker(rank, world, port, ring, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import paraattention_b200 as pa
    from paraattention_b200.context_parallel import init_context_parallel_mesh
    from paraattention_b200.context_parallel.diffusers_adapters import parallelize_pipe, parallelize_transformer
    from paraattention_b200.shape_models import FluxShapedPipeline

    mesh = init_context_parallel_mesh("cuda", max_ring_dim_size=2 if ring else None)
    errs = {}
    flux_ref = FluxShapedPipeline(_tiny_flux(), text_tokens=8, latent_hw=(4, 4))(num_inference_steps=2)
    pipe = parallelize_pipe(FluxShapedPipeline(_tiny_flux(), text_tokens=8, latent_hw=(4, 4)), mesh=mesh)
    flux_cp = pipe(num_inference_steps=2, generator=torch.Generator("cuda").manual_seed(0))
    errs["flux"] = ((flux_cp.float() - flux_ref.float()).norm() / flux_ref.float().norm()).item()

    x, enc, pooled = _video_inputs()
    t = torch.tensor([500.0], device="cuda")
    wan = _tiny_wan()
    want = wan(x, t, enc).sample
    got = parallelize_transformer(wan, mesh=mesh)(x, t, enc).sample
    errs["wan"] = ((got.float() - want.float()).norm() / want.float().norm()).item()

    hun = _tiny_hunyuan()
    mask, g = torch.ones(1, 8, device="cuda"), torch.tensor([6.0], device="cuda")
    want = hun(x, t, enc, mask, pooled, guidance=g).sample
    got = parallelize_transformer(hun, mesh=mesh)(x, t, enc, mask, pooled, guidance=g).sample
    errs["hunyuan"] = ((got.float() - want.float()).norm() / want.float().norm()).item()
    # a padded prompt: the key mask travels into the chunked kernel (also with a ring dimension)
    padded = torch.tensor([[1, 1, 1, 1, 1, 0, 0, 0]], device="cuda")
    want = _tiny_hunyuan()(x, t, enc, padded, pooled, guidance=g).sample
    got = hun(x, t, enc, padded, pooled, guidance=g).sample
    errs["hunyuan_padded_prompt"] = ((got.float() - want.float()).norm() / want.float().norm()).item()
    errs["padding_matters"] = ((want.float() - hun(x, t, enc, mask, pooled, guidance=g).sample.float()).norm()
                               / want.float().norm()).item() > 1e-3
    torch.cuda.synchronize()
    pa.check_device_status()
    if rank == 0:
        ret.put(errs)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("ring", [False, True])
def test_context_parallel_adapters_two_gpus(ring):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_cp_worker, args=(r, 2, 29720 + int(ring), ring, ret)) for r in range(2)]
    for p in procs:
        p.start()
    errs = ret.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
    assert errs.pop("padding_matters"), "the padded prompt gave the same result as the full one"
    for name, e in errs.items():
        assert e < 3e-2, f"{name}: relative L2 error {e:.3e} against the unsharded model"
