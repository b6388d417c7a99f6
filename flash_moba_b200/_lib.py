"""ctypes binding of libflashmoba_b200.so (the C ABI declared in include/flash_moba_b200.h).

There is no fallback: if the library has not been built, importing this module raises.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libflashmoba_b200.so")

c_i32p = ctypes.c_void_p
c_ptr = ctypes.c_void_p
i64 = ctypes.c_int64
i32 = ctypes.c_int
f32 = ctypes.c_float
sz = ctypes.c_size_t

FMB_BF16, FMB_FP16 = 0, 1

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python flash_moba_b200/build.py` "
        "(needs nvcc with sm_100a support). flash_moba_b200 has no CPU or PyTorch fallback."
    )

lib = ctypes.CDLL(LIB_PATH)

_SIGS = {
    "fmb_version": (i32, []),
    "fmb_last_error": (ctypes.c_char_p, []),
    "fmb_set_engine": (i32, [i32]),
    "fmb_attn_engine": (i32, [i32, i32, i32]),
    "fmb_gate_engine": (i32, [i32, i32]),
    "fmb_gate_status": (i32, [c_ptr]),
    "fmb_attn_status": (i32, [c_ptr, c_ptr, c_ptr]),
    "fmb_attn_status_mirror": (i32, [c_ptr]),
    "fmb_attn_key_spans": (i32, [c_ptr, c_ptr]),
    "fmb_selftest_wait_expiry": (i32, [c_ptr, c_ptr, c_ptr]),
    "fmb_selftest_umma": (i32, [c_ptr, c_ptr, c_ptr, i32, i32, c_ptr, c_ptr]),
    "fmb_launch_count": (ctypes.c_ulonglong, []),
    "fmb_profile_enable": (i32, [i32]),
    "fmb_profile_read": (i32, [i32, c_ptr, i32]),
    "fmb_profile_kinds": (i32, [ctypes.c_uint]),
    "fmb_copy_rows_async": (i32, [c_ptr, sz, c_ptr, sz, sz, sz, i32, c_ptr]),
    "fmb_chunk_offsets": (i32, [c_ptr, i32, i32, c_ptr, c_ptr]),
    "fmb_mean_pool": (i32, [c_ptr, i64, i64, c_ptr, c_ptr, c_ptr, i32, i32, i32, i32, i32, i32, c_ptr]),
    "fmb_mean_pool_offsets": (i32, [c_ptr, i64, i64, c_ptr, c_ptr, c_ptr, i32, i32, i32, i32, i32, i32, c_ptr]),
    "fmb_gate_topk": (i32, [c_ptr, i64, i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, i64, i64,
                            i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, c_ptr]),
    "fmb_build_csc_workspace_bytes": (sz, [i32, i32, i32, i32]),
    "fmb_build_csc": (i32, [c_ptr, i64, i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, sz, i32, i32, i32, i32, i32, c_ptr]),
    "fmb_build_csc_rows": (i32, [c_ptr, i64, i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, sz, i32, i32, i32, i64, i32, i32,
                                 c_ptr]),
    "fmb_attn_rows_offer": (i32, [c_ptr, i64, i32, i32]),
    "fmb_build_csc_static_capacity": (sz, []),
    "fmb_build_csc_static": (i32, [c_ptr, i64, i64, c_ptr, c_ptr, c_ptr, c_ptr, i32, i32, i32, i32, i32, c_ptr]),
    "fmb_varlen_sort": (i32, [c_ptr, c_ptr, c_ptr, c_ptr, i64, i64, c_ptr]),
    "fmb_attn_fwd_workspace_bytes": (sz, [i64, i32, i32, i32, i64, i32, i32, i32, i32]),
    "fmb_attn_bwd_workspace_bytes": (sz, [i64, i32, i32, i32, i64, i32, i32, i32, i32]),
    "fmb_attn_lists_bytes": (sz, [i64, i32, i32, i32, i64, i32, i32, i32]),
    "fmb_attn_lists_save": (i32, [c_ptr, sz, i64, i32, i32, i32, i64, i32, i32, i32, c_ptr, sz, c_ptr]),
    "fmb_attn_lists_load": (i32, [c_ptr, sz, i64, i32, i32, i32, i64, i32, i32, i32, c_ptr, sz, c_ptr]),
    "fmb_attn_fwd": (i32, [c_ptr, i64, i64, c_ptr, i64, i64, c_ptr, i64, i64, c_ptr, i64, i64, c_ptr,
                           c_ptr, c_ptr, c_ptr, i64, c_ptr, c_ptr, c_ptr, sz,
                           i32, i32, i32, i32, i64, i32, i32, i32, f32, i32, i32, c_ptr]),
    "fmb_attn_bwd": (i32, [c_ptr, i64, i64, c_ptr, i64, i64, c_ptr, i64, i64, c_ptr, i64, i64, c_ptr, i64, i64,
                           c_ptr, c_ptr, i64, i64, c_ptr, i64, i64, c_ptr, i64, i64, c_ptr,
                           c_ptr, c_ptr, c_ptr, i64, c_ptr, c_ptr, c_ptr, sz,
                           i32, i32, i32, i32, i64, i64, i32, i32, i32, f32, i32, i32, c_ptr]),
}

for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args

EXPORTS = tuple(_SIGS)


def check(rc: int) -> None:
    """Turn a non-zero status into the RuntimeError the reference raises through TORCH_CHECK."""
    if rc != 0:
        raise RuntimeError(lib.fmb_last_error().decode("utf-8", "replace") or f"flash_moba_b200 error {rc}")
