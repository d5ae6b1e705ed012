"""No-GPU checks of the boundary: the library builds, loads and exports every symbol that
include/pa_b200.h declares; ctypes structures have the C layout; argument validation answers
without touching a device."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "pa_b200.h"


@pytest.fixture(scope="module")
def lib():
    from paraattention_b200 import build_ext, _lib

    build_ext.build()
    return _lib.load()


def _declared_functions():
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pa_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared_functions()
    assert "pa_attn_fwd" in names and "pa_cp_push" in names and "pa_fbc_residual_diff" in names
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/pa_b200.h but not exported"


def test_struct_layouts_match_c(tmp_path):
    from paraattention_b200 import _lib as L

    src = tmp_path / "sz.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "pa_b200.h"\n'
        'int main(){printf("%zu %zu %zu %zu %zu %zu %zu\\n", sizeof(pa_attn_args), sizeof(pa_cp_attn_args),'
        ' sizeof(pa_push_job), sizeof(pa_cp_push_args), offsetof(pa_cp_attn_args, status),'
        ' offsetof(pa_cp_push_args, flag), offsetof(pa_attn_args, status));'
        'printf("%zu %zu\\n", offsetof(pa_attn_args, workspace), offsetof(pa_cp_attn_args, workspace_bytes));}\n')
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = [C.sizeof(L.AttnArgs), C.sizeof(L.CpAttnArgs), C.sizeof(L.PushJob), C.sizeof(L.CpPushArgs),
            L.CpAttnArgs.status.offset, L.CpPushArgs.flag.offset, L.AttnArgs.status.offset,
            L.AttnArgs.workspace.offset, L.CpAttnArgs.workspace_bytes.offset]
    assert got == want


def test_validation_needs_no_device(lib):
    from paraattention_b200 import _lib as L

    assert lib.pa_version() >= 1
    a = L.AttnArgs()
    assert lib.pa_attn_fwd(C.byref(a), None) == L.PA_EINVAL
    assert lib.pa_attn_fwd(None, None) == L.PA_EINVAL
    c = L.CpAttnArgs()
    assert lib.pa_cp_attn_fwd(C.byref(c), None) == L.PA_EINVAL
    p = L.CpPushArgs()
    p.n_dest = 0
    assert lib.pa_cp_push(C.byref(p), None) == L.PA_EINVAL
    assert lib.pa_fbc_residual_diff(None, None, None, None, 1, 8, 1, 0, None, None, None) == L.PA_EINVAL
    assert lib.pa_fbc_scratch_bytes() > 0
    with pytest.raises(L.PaError):
        L.check(L.PA_EINVAL)


def test_ops_refuse_cpu_tensors():
    import torch

    from paraattention_b200 import ops
    from paraattention_b200.first_block_cache import utils as fbc

    q = torch.zeros(1, 1, 8, 128, dtype=torch.bfloat16)
    with pytest.raises((NotImplementedError, RuntimeError)):
        ops.attention_forward(q, q, q)
    with pytest.raises(RuntimeError):
        fbc.fused_residual_diff(q, q, None)


def test_new_entry_points_validate_without_a_device(lib):
    """pa_pack_key_mask, pa_taylor_update and pa_taylor_approx refuse bad arguments before any
    launch (no GPU is touched on these paths)."""
    from paraattention_b200 import _lib as L

    assert lib.pa_pack_key_mask(None, 8, 1, 1, 8, None, None) == L.PA_EINVAL
    buf = (C.c_uint8 * 64)()
    out = (C.c_uint64 * 4)()
    addr, oaddr = C.addressof(buf), C.addressof(out)
    assert lib.pa_pack_key_mask(addr, 4, 1, 1, 8, oaddr, None) == L.PA_EINVAL      # stride shorter than the keys
    assert lib.pa_pack_key_mask(addr, 8, 0, 1, 8, oaddr, None) == L.PA_EINVAL      # empty batch
    ptrs = (C.c_void_p * 4)()
    assert lib.pa_taylor_update(addr, ptrs, ptrs, 0, 1, 64, L.PA_BF16, None) == L.PA_OK  # depth 0: nothing to do
    assert lib.pa_taylor_update(addr, ptrs, ptrs, 5, 1, 64, L.PA_BF16, None) == L.PA_EINVAL
    assert lib.pa_taylor_update(addr, ptrs, ptrs, 1, 0, 64, L.PA_BF16, None) == L.PA_EINVAL
    assert lib.pa_taylor_update(addr, ptrs, ptrs, 1, 1, 63, L.PA_BF16, None) == L.PA_EINVAL
    assert lib.pa_taylor_update(addr, ptrs, ptrs, 1, 1, 64, L.PA_BF16, None) == L.PA_EINVAL  # NULL prev[0]
    assert lib.pa_taylor_approx(ptrs, 0, 1, None, addr, 64, L.PA_BF16, None) == L.PA_EINVAL
    assert lib.pa_taylor_approx(ptrs, 6, 1, None, addr, 64, L.PA_BF16, None) == L.PA_EINVAL
    assert lib.pa_taylor_approx(ptrs, 1, -1, None, addr, 64, L.PA_BF16, None) == L.PA_EINVAL
    assert lib.pa_taylor_approx(ptrs, 1, 1, None, addr, 64, 7, None) == L.PA_EINVAL
    a = L.AttnArgs()
    a.q = a.k = a.v = a.out = addr
    a.batch = a.heads = a.seq_q = a.seq_kv = 1
    a.head_dim, a.scale = 96, 1.0
    assert lib.pa_attn_fwd(C.byref(a), None) == L.PA_ENOTSUP and b"64 and 128" in lib.pa_last_error()


def test_split_plan_of_the_last_wave(lib):
    """Which launches give the units of their last wave to several CTAs (no device needed)."""
    def plan(units, tiles, sms=148, d=128, causal=0, ws=None, push=0):
        ws = lib.pa_attn_workspace_bytes() if ws is None else ws
        f, k = C.c_int32(-1), C.c_int32(-1)
        assert lib.pa_attn_split_plan(units, sms, tiles, d, causal, push, ws, C.byref(f), C.byref(k)) == 0
        return f.value, k.value

    assert lib.pa_attn_workspace_bytes() >= 440 * 256 * (8 + 128 * 4)
    # 8 ranks of the headline workload: 384 units, 2.59 waves -> the last 88 units go to 5 CTAs each
    assert plan(384, 256) == (296, 5)
    # 4 ranks: 768 units, 28 in the last wave -> 140 CTAs, one round
    assert plan(768, 256) == (740, 5)
    # one GPU: 3072 units, 20.76 waves - nothing to gain
    assert plan(3072, 256) == (3072, 1)
    # whole waves, causal runs, no workspace, too few tiles per CTA: one launch
    assert plan(296, 256) == (296, 1)
    assert plan(384, 256, causal=1) == (384, 1)
    assert plan(384, 256, ws=0) == (384, 1)
    assert plan(384, 15) == (384, 1)
    # a smaller workspace allows fewer CTAs per unit
    f, k = plan(384, 256, ws=40 << 20)
    assert f == 296 and 2 <= k < 5
    # fewer units than SMs (FLUX-sized call on 8 ranks): 54 units -> 108 CTAs
    assert plan(54, 36) == (0, 2)
    # launches led by pushing CTAs are never split (measured slower with real peers)
    assert plan(216, 36) == (148, 2) and plan(216, 36, push=1) == (216, 1)
    assert plan(384, 256, push=1) == (384, 1) and plan(54, 36, push=1) == (54, 1)
    assert lib.pa_attn_split_plan(0, 148, 1, 128, 0, 0, 0, None, None) != 0
