"""ctypes binding of libpa_b200.so (declarations mirror include/pa_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PA_MAX_CHUNKS = 8
PA_OK, PA_EINVAL, PA_ENOTSUP, PA_ECUDA, PA_ETIMEDOUT = 0, -1, -2, -3, -4
PA_BF16, PA_F16 = 0, 1
PA_DEV_TIMEOUT_PIPE, PA_DEV_TIMEOUT_Q, PA_DEV_TIMEOUT_KV, PA_DEV_TIMEOUT_OUT = 1, 2, 3, 4
DEV_STATUS_NAMES = {
    0: "ok",
    1: "timeout on an in-kernel pipeline barrier",
    2: "timeout waiting for a query chunk",
    3: "timeout waiting for a key/value chunk",
    4: "timeout waiting for the output-arrival counter",
}

LIB_PATH = Path(__file__).resolve().parent / "libpa_b200.so"


class PaError(RuntimeError):
    """A libpa_b200 entry point returned a negative status."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"libpa_b200 error {code}: {msg}")
        self.code = code


class AttnArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("seq_q", C.c_int32), ("seq_kv", C.c_int32),
        ("head_dim", C.c_int32), ("dtype", C.c_int32), ("is_causal", C.c_int32), ("scale", C.c_float),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("o_stride", C.c_int64 * 3),
        ("status", C.c_void_p), ("wait_limit_ns", C.c_uint64),
        ("key_bits", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
    ]


class CpAttnArgs(C.Structure):
    _fields_ = [
        ("q_stage", C.c_void_p), ("k_stage", C.c_void_p), ("v_stage", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32), ("dtype", C.c_int32),
        ("n_q_chunks", C.c_int32), ("q_rows", C.c_int32), ("q_first", C.c_int32),
        ("n_kv_chunks", C.c_int32), ("kv_rows", C.c_int32), ("kv_first", C.c_int32),
        ("scale", C.c_float),
        ("out", C.c_void_p * PA_MAX_CHUNKS), ("lse", C.c_void_p * PA_MAX_CHUNKS),
        ("o_stride", C.c_int64 * 3), ("lse_stride", C.c_int64 * 2),
        ("out_head_offset", C.c_int32),
        ("q_flag", C.c_void_p * PA_MAX_CHUNKS), ("kv_flag", C.c_void_p * PA_MAX_CHUNKS),
        ("flag_expect", C.c_uint32),
        ("done_flag", C.c_void_p * PA_MAX_CHUNKS),
        ("status", C.c_void_p), ("wait_limit_ns", C.c_uint64),
        ("fused_push", C.c_void_p),
        ("q_local", C.c_void_p), ("k_local", C.c_void_p), ("v_local", C.c_void_p),
        ("q_local_stride", C.c_int64 * 3), ("k_local_stride", C.c_int64 * 3), ("v_local_stride", C.c_int64 * 3),
        ("local_head_offset", C.c_int32), ("local_total_heads", C.c_int32),
        ("is_causal", C.c_int32), ("pad_", C.c_int32),
        ("q_pos", C.c_int64 * PA_MAX_CHUNKS), ("kv_pos", C.c_int64 * PA_MAX_CHUNKS),
        ("key_bits", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
    ]


PA_MAX_PUSH_JOBS = 24


class PushJob(C.Structure):
    _fields_ = [
        ("src", C.c_void_p), ("dst", C.c_void_p),
        ("src_stride", C.c_int64 * 3), ("dst_stride", C.c_int64 * 3),
        ("head0", C.c_int32), ("heads", C.c_int32), ("batch", C.c_int32), ("rows", C.c_int32),
        ("dest", C.c_int32), ("head_dim", C.c_int32),
    ]


class CpPushArgs(C.Structure):
    _fields_ = [
        ("jobs", PushJob * PA_MAX_PUSH_JOBS),
        ("n_jobs", C.c_int32), ("n_dest", C.c_int32),
        ("flag", C.c_void_p * PA_MAX_CHUNKS),
        ("ctas_per_dest", C.c_int32), ("first_dest", C.c_int32),
    ]


class QkvPrepArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("q_out", C.c_void_p), ("k_out", C.c_void_p), ("v_out", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("q_out_stride", C.c_int64 * 3), ("k_out_stride", C.c_int64 * 3), ("v_out_stride", C.c_int64 * 3),
        ("q_weight", C.c_void_p), ("k_weight", C.c_void_p), ("cos", C.c_void_p), ("sin", C.c_void_p),
        ("table_row0", C.c_int64),
        ("batch", C.c_int32), ("rows", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("dtype", C.c_int32), ("eps", C.c_float),
    ]


_lib = None


def load() -> C.CDLL:
    """Load the library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m paraattention_b200.build_ext` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback."
        )
    lib = C.CDLL(str(LIB_PATH))
    lib.pa_last_error.restype = C.c_char_p
    lib.pa_last_error.argtypes = []
    lib.pa_version.restype = C.c_int
    lib.pa_attn_workspace_bytes.restype = C.c_int64
    lib.pa_attn_workspace_bytes.argtypes = []
    lib.pa_attn_split_plan.restype = C.c_int
    lib.pa_attn_split_plan.argtypes = [C.c_int64, C.c_int32, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int64,
                                       C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.pa_attn_fwd.restype = C.c_int
    lib.pa_attn_fwd.argtypes = [C.POINTER(AttnArgs), C.c_void_p]
    lib.pa_qkv_prep.restype = C.c_int
    lib.pa_qkv_prep.argtypes = [C.POINTER(QkvPrepArgs), C.c_void_p]
    lib.pa_cp_attn_fwd.restype = C.c_int
    lib.pa_cp_attn_fwd.argtypes = [C.POINTER(CpAttnArgs), C.c_void_p]
    lib.pa_taylor_update.restype = C.c_int
    lib.pa_taylor_update.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int32, C.c_int32,
                                     C.c_int64, C.c_int32, C.c_void_p]
    lib.pa_taylor_approx.restype = C.c_int
    lib.pa_taylor_approx.argtypes = [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_int64,
                                     C.c_int32, C.c_void_p]
    lib.pa_pack_key_mask.restype = C.c_int
    lib.pa_pack_key_mask.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    lib.pa_cp_push.restype = C.c_int
    lib.pa_cp_push.argtypes = [C.POINTER(CpPushArgs), C.c_void_p]
    lib.pa_flag_wait.restype = C.c_int
    lib.pa_flag_wait.argtypes = [C.POINTER(C.c_void_p), C.c_int32, C.c_uint32, C.c_void_p, C.c_uint64, C.c_int32,
                                 C.c_void_p]
    lib.pa_merge_out_lse.restype = C.c_int
    lib.pa_merge_out_lse.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                     C.c_void_p]
    lib.pa_fbc_scratch_bytes.restype = C.c_int64
    lib.pa_fbc_scratch_bytes.argtypes = []
    lib.pa_fbc_residual_diff.restype = C.c_int
    lib.pa_fbc_residual_diff.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                         C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.pa_fbc_residual_diff_static.restype = C.c_int
    lib.pa_fbc_residual_diff_static.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                                C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    lib.pa_fbc_axpy.restype = C.c_int
    lib.pa_fbc_axpy.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p]
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != PA_OK:
        raise PaError(rc, load().pa_last_error().decode())
