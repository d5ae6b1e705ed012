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
        ' offsetof(pa_cp_push_args, flag), offsetof(pa_attn_args, status));}\n')
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = [C.sizeof(L.AttnArgs), C.sizeof(L.CpAttnArgs), C.sizeof(L.PushJob), C.sizeof(L.CpPushArgs),
            L.CpAttnArgs.status.offset, L.CpPushArgs.flag.offset, L.AttnArgs.status.offset]
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
