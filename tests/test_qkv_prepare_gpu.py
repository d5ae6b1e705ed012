"""The fused neighbours of attention (pa_qkv_prep through ops.qkv_prepare): per-head RMSNorm of q
and k, rotary embedding, and placement of the streams of a joint-attention block into one
buffer, against the chain of tensor operations it replaces. The two agree bit for bit except
where the fp32 summation order of the mean shows, which moves a 16-bit result by at most one
unit in the last place: the tests allow that on a small fraction of the elements."""
import pytest
import torch

from paraattention_b200 import config, ops
from paraattention_b200.shape_models import _joint_qkv, _rms, _rope, _split_heads

pytestmark = pytest.mark.gpu


def _ulp_close(got, want, what, frac=0.02):
    g, w = got.float(), want.float()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    diff = (g - w).abs()
    ulp = torch.maximum(w.abs(), torch.full_like(w, 1e-30)) * (2.0 ** -7 if got.dtype == torch.bfloat16 else 2.0 ** -10)
    assert bool((diff <= ulp).all()), f"{what}: more than one unit in the last place ({float((diff / ulp).max()):.2f})"
    off = float((diff > 0).float().mean())
    assert off <= frac, f"{what}: {off:.3%} of the elements differ"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,S,H,D", [(1, 300, 4, 128), (2, 77, 3, 64), (1, 4608, 24, 128)])
def test_qkv_prepare_matches_the_tensor_operations(B, S, H, D, dtype):
    g = torch.Generator(device="cuda").manual_seed(S + D)
    proj = torch.randn(B, S, 3 * H * D, device="cuda", generator=g).to(dtype)  # one packed projection output
    q, k, v = (t.unflatten(-1, (H, D)).transpose(1, 2) for t in proj.chunk(3, dim=-1))
    wq = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(dtype)
    wk = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(dtype)
    ang = torch.rand(S, D // 2, device="cuda", generator=g).repeat_interleave(2, dim=-1) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()

    def rms(x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(x.dtype) * w

    want_q, want_k = _rope(rms(q, wq), cos, sin), _rope(rms(k, wk), cos, sin)
    got_q, got_k, got_v = ops.qkv_prepare(q, k, v, wq, wk, (cos, sin))
    _ulp_close(got_q, want_q, "q")
    _ulp_close(got_k, want_k, "k")
    assert torch.equal(got_v, v)
    assert got_q.transpose(1, 2).is_contiguous()  # [B, S, H, D] memory, as the attention ops like it
    # no norm, no rotation: a pure re-layout
    plain_q, plain_k, _ = ops.qkv_prepare(q, k, None)
    assert torch.equal(plain_q, q) and torch.equal(plain_k, k)
    # rotation only is exact (no reduction involved)
    rot_q, _, _ = ops.qkv_prepare(q, k, None, rotary=(cos, sin))
    assert torch.equal(rot_q, _rope(q, cos, sin))


def test_joint_streams_land_in_one_buffer_like_the_concatenation():
    """Two streams (text then image), rotation on the image rows only: the fused path of
    _joint_qkv against its own chain of tensor operations."""
    g = torch.Generator(device="cuda").manual_seed(0)
    B, H, D, n_txt, n_img = 2, 4, 128, 40, 300

    def stream(rows):
        proj = torch.randn(B, rows, 3 * H * D, device="cuda", generator=g).bfloat16()
        q, k, v = proj.chunk(3, dim=-1)
        return (q, k, v, (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16(),
                (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16())

    txt, img = stream(n_txt), stream(n_img)
    ang = torch.rand(n_img, D // 2, device="cuda", generator=g).repeat_interleave(2, dim=-1) * 6.28
    rotary = (ang.cos().contiguous(), ang.sin().contiguous())
    for rows in ((n_txt, n_img), None):
        tab = rotary if rows is not None else tuple(torch.cat([t.new_zeros(n_txt, D) + (i == 0), t]) for i, t in enumerate(rotary))
        with config.patch({"attention.fuse_qkv_prepare": False}):
            want = _joint_qkv([txt, img], tab, rotary_rows=rows)
        got = _joint_qkv([txt, img], tab, rotary_rows=rows)
        for name, a, b in zip("qkv", got, want):
            _ulp_close(a, b, f"joint {name} rows={rows}")
        assert got[0].shape == (B, H, n_txt + n_img, D)


def test_shape_model_forward_with_and_without_the_fused_preparation():
    """A FLUX-shaped transformer forward: fused preparation against the chain of tensor operations."""
    from paraattention_b200.shape_models import FluxShapedTransformer2DModel

    torch.manual_seed(0)
    model = FluxShapedTransformer2DModel(dim=512, num_layers=2, num_single_layers=2, joint_attention_dim=64).cuda().bfloat16()
    g = torch.Generator(device="cuda").manual_seed(1)
    hw, n_txt = 16, 32
    ys, xs = torch.meshgrid(torch.arange(hw), torch.arange(hw), indexing="ij")
    inputs = dict(hidden_states=torch.randn(1, hw * hw, 64, device="cuda", generator=g).bfloat16(),
                  encoder_hidden_states=torch.randn(1, n_txt, 64, device="cuda", generator=g).bfloat16(),
                  pooled_projections=torch.randn(1, 768, device="cuda", generator=g).bfloat16(),
                  timestep=torch.tensor([500.0], device="cuda"),
                  img_ids=torch.stack([torch.zeros_like(ys), ys, xs], -1).reshape(-1, 3).float().cuda(),
                  txt_ids=torch.zeros(n_txt, 3, device="cuda"), guidance=torch.tensor([3.5], device="cuda"),
                  return_dict=False)
    with torch.no_grad():
        fused = model(**inputs)[0]
        with config.patch({"attention.fuse_qkv_prepare": False}):
            eager = model(**inputs)[0]
    err = (fused.float() - eager.float()).abs().max().item()
    assert err <= 0.05 * eager.float().abs().max().item(), f"fused vs eager forward: {err:.3e}"
