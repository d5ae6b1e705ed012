"""First-Block-Cache kernels on the GPU against the oracle and the reference's recorded decisions."""
import ctypes as C

import math

import numpy as np
import pytest
import torch

from oracle import cp_attention_oracle as O
from helpers import bf16_from_bits

pytestmark = pytest.mark.gpu


def _abi_residual_diff(h1, h0, prev, downsample=1, store=True):
    from paraattention_b200 import _lib as L

    lib = L.load()
    cols = h1.shape[-1]
    rows = h1.numel() // cols
    cols_ds = (cols + downsample - 1) // downsample
    cur = torch.empty(tuple(h1.shape[:-1]) + (cols_ds,), dtype=h1.dtype, device="cuda") if store else None
    result = torch.full((5,), float("nan"), device="cuda")
    scratch = torch.zeros(int(lib.pa_fbc_scratch_bytes()), dtype=torch.uint8, device="cuda")
    rc = lib.pa_fbc_residual_diff(h1.data_ptr(), h0.data_ptr(), prev.data_ptr() if prev is not None else None,
                                  cur.data_ptr() if cur is not None else None, rows, cols, downsample,
                                  L.PA_BF16 if h1.dtype == torch.bfloat16 else L.PA_F16, result.data_ptr(),
                                  scratch.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.pa_last_error()
    torch.cuda.synchronize()
    # the ticket word must be back to zero so that the scratch can be reused
    assert int(scratch[-4:].view(torch.int32).item()) == 0
    return cur, result.cpu().numpy()


@pytest.mark.parametrize("shape,ds", [((1, 32, 128), 1), ((2, 333, 3072), 1), ((1, 4096, 3072), 1), ((1, 77, 3072), 2),
                                      ((1, 50, 130), 1), ((1, 64, 3072), 4)])
def test_residual_diff_bit_exact_against_oracle(shape, ds):
    g = torch.Generator().manual_seed(shape[1])
    h0 = torch.randn(shape, generator=g).bfloat16()
    h1 = (h0.float() + 0.3 * torch.randn(shape, generator=g)).bfloat16()
    cols_ds = (shape[-1] + ds - 1) // ds
    prev = (0.3 * torch.randn(shape[:-1] + (cols_ds,), generator=g)).bfloat16()
    cur, res = _abi_residual_diff(h1.cuda(), h0.cuda(), prev.cuda(), downsample=ds)
    want_cur = O.bf16_round(h1.float().numpy() - h0.float().numpy())[..., ::ds]
    # residual: bit-exact
    np.testing.assert_array_equal(cur.float().cpu().numpy(), want_cur)
    sd, sp = O.fbc_partial_sums(prev.float().numpy(), want_cur)
    n = want_cur.size
    # fp32 sums: accumulation order differs, values agree to fp32 accuracy
    np.testing.assert_allclose(res[0], sd, rtol=2e-6)
    np.testing.assert_allclose(res[1], sp, rtol=2e-6)
    # the rounded means / ratio the decision is taken from: exact
    assert res[2] == O.bf16_round(np.float32(res[0]) / np.float32(n))
    assert res[3] == O.bf16_round(np.float32(res[1]) / np.float32(n))
    assert O.fbc_decision([res[0]], [res[1]], n, 0.5) == bool(res[4] < 0.5)
    assert res[4] == O.bf16_round(np.float32(res[2]) / np.float32(res[3]))


def test_residual_diff_without_prev_or_store():
    h0 = torch.randn(1, 16, 256).bfloat16().cuda()
    h1 = torch.randn(1, 16, 256).bfloat16().cuda()
    cur, res = _abi_residual_diff(h1, h0, None)
    assert res[0] == 0.0 and res[1] == 0.0
    np.testing.assert_array_equal(cur.float().cpu().numpy(), O.bf16_round(h1.float().cpu().numpy() - h0.float().cpu().numpy()))
    none, res = _abi_residual_diff(h1, h0, cur, store=False)
    assert none is None and res[0] == 0.0 and res[1] > 0.0


def test_axpy_bit_exact():
    from paraattention_b200 import _lib as L

    lib = L.load()
    a = torch.randn(3, 1000, 128).bfloat16().cuda()
    b = torch.randn(3, 1000, 128).bfloat16().cuda()
    out = torch.empty_like(a)
    for sub in (0, 1):
        rc = lib.pa_fbc_axpy(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), sub, L.PA_BF16,
                             torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        want = (a - b) if sub else (a + b)
        assert torch.equal(out, want)


@pytest.mark.parametrize("case,kw", [
    ("thr008", dict(residual_diff_threshold=0.08)),
    ("thr003_warm2", dict(residual_diff_threshold=0.03, warmup_steps=2)),
    ("thr02_ds2", dict(residual_diff_threshold=0.2, downsample_factor=2)),
    ("thr0", dict(residual_diff_threshold=0.0)),
    ("thr008_taylor", dict(residual_diff_threshold=0.08, enable_taylorseer=True, taylorseer_kwargs=dict(n_derivatives=2))),
])
def test_cached_blocks_follow_reference_step_by_step(golden_dir, case, kw):
    """Same scripted sequence as tests/golden/make_golden.py: the skip/compute decision and the
    block outputs must equal what the reference's CachedTransformerBlocks produced."""
    from paraattention_b200.first_block_cache import utils as fbc

    g = np.load(golden_dir / "fbcache_steps.npz")
    h0s, h1s, enc = bf16_from_bits(g["h0"]), bf16_from_bits(g["h1"]), bf16_from_bits(g["enc"])

    class Block0(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.t = 0

        def forward(self, hidden_states, encoder_hidden_states):
            out = h1s[self.t]
            self.t += 1
            return out, (encoder_hidden_states.float() + 0.25).bfloat16()

    class Block1(torch.nn.Module):
        def forward(self, hidden_states, encoder_hidden_states):
            return (hidden_states.float() * 1.5).bfloat16(), (encoder_hidden_states.float() * 0.5).bfloat16()

    blocks = fbc.CachedTransformerBlocks(torch.nn.ModuleList([Block0(), Block1()]))
    hits = []
    with fbc.cache_context(fbc.create_cache_context(**kw)):
        for t in range(h0s.shape[0]):
            before = fbc.get_current_cache_context().get_buffer("first_hidden_states_residual")
            out, enc_out = blocks(h0s[t], enc)
            after = fbc.get_current_cache_context().get_buffer("first_hidden_states_residual")
            hits.append(after is before and before is not None)
            if f"{case}_out" in g:
                assert torch.equal(out, bf16_from_bits(g[f"{case}_out"][t])), f"step {t}: hidden states differ"
            if f"{case}_enc_out" in g:
                assert torch.equal(enc_out, bf16_from_bits(g[f"{case}_enc_out"][t])), f"step {t}: encoder states differ"
    assert hits == list(g[f"{case}_hit"])


def test_full_size_sums_and_bandwidth_shape():
    """FLUX-sized residual (4096 x 3072 bf16): sums agree with a torch fp64 evaluation."""
    n, c = 4096, 3072
    g = torch.Generator(device="cuda").manual_seed(0)
    h0 = torch.randn(1, n, c, generator=g, device="cuda").bfloat16()
    h1 = (h0.float() + 0.2 * torch.randn(1, n, c, generator=g, device="cuda")).bfloat16()
    prev = (0.2 * torch.randn(1, n, c, generator=g, device="cuda")).bfloat16()
    cur, res = _abi_residual_diff(h1, h0, prev)
    want_cur = h1 - h0
    assert torch.equal(cur, want_cur)
    sd = (prev - want_cur).abs().double().sum().item()
    sp = prev.abs().double().sum().item()
    np.testing.assert_allclose(res[0], sd, rtol=1e-5)
    np.testing.assert_allclose(res[1], sp, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case,kw", [
    ("d2_w1_s3", dict(n_derivatives=2, warmup_steps=1, skip_interval_steps=3)),
    ("d3_w2_s4", dict(n_derivatives=3, warmup_steps=2, skip_interval_steps=4)),
    ("d1_map", dict(n_derivatives=1, compute_step_map=[True, True, False, True, False, False, False, True, False,
                                                       False, True, False, False, False])),
])
def test_taylorseer_kernels_bit_exact(golden_dir, case, kw, dtype):
    """TaylorSeer.step on the GPU: for bf16 against the reference's own outputs (fixture), for
    fp16 against the same chain of tensor operations done by ATen on the GPU."""
    from paraattention_b200.first_block_cache.taylorseer import TaylorSeer

    g = np.load(golden_dir / "taylorseer.npz")
    ys = bf16_from_bits(g["y"]).to(dtype)
    seer = TaylorSeer(**kw)
    prev, cur, last = None, None, -1
    for t in range(ys.shape[0]):
        got = seer.step(ys[t])
        if dtype == torch.bfloat16:
            assert torch.equal(got, bf16_from_bits(g[case][t])), f"{case}: step {t} differs from the reference"
        # the same arithmetic as separate tensor operations (true division, as on the CPU)
        if seer.last_non_approximated_step == t:
            new = [ys[t]]
            if t > 1 and cur is not None:
                for i in range(seer.n_derivatives):
                    if i < len(cur):
                        new.append(torch.true_divide(new[i] - cur[i], torch.tensor(float(t - last), device="cuda")).to(dtype))
            prev, cur, last = cur, new, t
            want = ys[t]
        else:
            want = cur[0]
            for i in range(1, len(cur)):
                want = want + (1 / math.factorial(i)) * cur[i] * ((t - last) ** i)
        assert torch.equal(got, want), f"{case} {dtype}: step {t} differs from the chained tensor operations"


def test_taylorseer_fused_add_and_refusals():
    from paraattention_b200.first_block_cache.taylorseer import TaylorSeer

    g = torch.Generator().manual_seed(0)
    ys = [torch.randn(4, 64, generator=g).bfloat16().cuda() for _ in range(4)]
    h = torch.randn(4, 64, generator=g).bfloat16().cuda()
    seer = TaylorSeer(n_derivatives=2, warmup_steps=3, skip_interval_steps=10)
    for y in ys[:3]:
        seer.step(y)
    seer.mark_step_begin()
    plain = seer.approximate_value()
    assert torch.equal(seer.approximate_value(add=h), plain + h)
    with pytest.raises(NotImplementedError):
        seer.update(torch.zeros(3, 5, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(NotImplementedError):
        seer.update(torch.zeros(4, 64, dtype=torch.float32, device="cuda"))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(3, 5, 7), (1, 4097), (2, 33, 129)])
def test_residual_arithmetic_on_sizes_the_vector_kernel_cannot_take(shape, dtype):
    """pa_fbc_axpy's scalar form: sizes that are not multiples of 8 and storage offsets that are not
    16-byte aligned give the same 16-bit results as the tensor operations they replace."""
    from paraattention_b200.first_block_cache import utils as fbc

    g = torch.Generator().manual_seed(sum(shape))
    a = torch.randn(shape, generator=g).to(dtype).cuda()
    b = torch.randn(shape, generator=g).to(dtype).cuda()
    assert torch.equal(fbc._axpy(a, b, sub=True), a - b)
    assert torch.equal(fbc._axpy(a, b, sub=False), a + b)
    # same size, but storage that starts 2 bytes into an allocation
    n = a.numel()
    base_a, base_b = torch.empty(n + 1, dtype=dtype, device="cuda"), torch.empty(n + 1, dtype=dtype, device="cuda")
    a2, b2 = base_a[1:].view(shape), base_b[1:].view(shape)
    a2.copy_(a), b2.copy_(b)
    assert torch.equal(fbc._axpy(a2, b2, sub=True), a - b)
    with pytest.raises(NotImplementedError):
        fbc._axpy(a.float(), b.float(), sub=True)


def test_similarity_of_two_given_tensors_reads_no_third():
    """are_two_tensors_similar passes no h0 to the kernel (the residual is t2 itself): same
    decision and the same sums as forming t2 - 0 explicitly."""
    from paraattention_b200.first_block_cache import utils as fbc

    g = torch.Generator().manual_seed(3)
    t1 = torch.randn(2, 512, 256, generator=g).to(torch.bfloat16).cuda()
    t2 = (t1.float() * (1 + 0.07 * torch.randn(t1.shape, generator=g).cuda())).to(torch.bfloat16)
    _, r_none = fbc.fused_residual_diff(t2, None, t1, store=False)
    _, r_zero = fbc.fused_residual_diff(t2, torch.zeros_like(t2), t1, store=False)
    assert torch.equal(r_none, r_zero)
    ratio = float(r_none[4])
    assert fbc.are_two_tensors_similar(t1, t2, threshold=ratio * 1.5)
    assert not fbc.are_two_tensors_similar(t1, t2, threshold=ratio * 0.5)
