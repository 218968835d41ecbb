"""ctypes binding of libmini_vllm_b200.so (the C ABI declared in include/mini_vllm_b200.h).

There is no fallback: if the library is missing, importing the kernels raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libmini_vllm_b200.so"

i32, i64, f32, u64, vp, sz = C.c_int, C.c_int64, C.c_float, C.c_uint64, C.c_void_p, C.c_size_t

# name -> (restype, argtypes); mirrors include/mini_vllm_b200.h exactly
SIGNATURES = {
    "mvb_abi_version": (i32, []),
    "mvb_status_string": (C.c_char_p, [i32]),
    "mvb_selftest_wait_timeout": (i32, [vp, i32, vp]),
    "mvb_pack_prefill": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp]),
    "mvb_pack_decode": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i32, vp, vp, vp, vp, vp, vp, vp]),
    "mvb_rope_kv_write": (i32, [vp, i64, vp, i64, vp, i64, vp, vp, i64, vp, vp, vp, i64, i32, i32, i32, i32, i32,
                                vp, vp]),
    "mvb_qk_norm_rope_kv_write": (i32, [vp, i64, vp, i64, vp, i64, vp, vp, f32, i32, vp, vp, i64, vp, vp, vp, i64,
                                        i32, i32, i32, i32, i32, vp, vp]),
    "mvb_decode_workspace_bytes": (sz, [i32, i32, i32]),
    "mvb_decode_plan": (i32, [vp, i32, i32, i32, i32, i32, vp, sz, vp]),
    "mvb_decode_plan_with_table": (i32, [vp, vp, i64, i32, i32, i32, i32, i32, i32, vp, sz, vp]),
    "mvb_decode_attn": (i32, [vp, i64, vp, vp, i64, i32, vp, vp, i64, i32, i32, i32, i32, i32, f32, i32, vp, i64,
                              vp, sz, vp, vp]),
    "mvb_decode_attn_static": (i32, [vp, i64, vp, vp, i64, i32, vp, vp, i64, i32, i32, i32, i32, i32, f32, i32, vp,
                                     i64, vp, vp]),
    "mvb_prefill_attn": (i32, [vp, i64, vp, i64, vp, i64, i64, vp, vp, vp, i64, i32, i32, i32, i32, i32, i32, i32, f32,
                               i32, vp, i64, vp, vp]),
    "mvb_prefill_item_rows": (i32, [i32, i32, i32]),
    "mvb_prefill_attn_items": (i32, [vp, i64, vp, i64, vp, i64, i64, vp, vp, vp, i64, i32, i32, i32, i32, i32, i32, i32,
                                     f32, i32, vp, i64, vp, i32, vp, vp]),
    "mvb_act_mul": (i32, [vp, i64, vp, i64, i32, i32, i32, vp]),
    "mvb_add_rmsnorm": (i32, [vp, vp, i64, vp, vp, vp, i32, i32, f32, i32, vp]),
    "mvb_add_rmsnorm_last_tokens": (i32, [vp, vp, i64, vp, vp, vp, vp, i32, i32, f32, i32, vp]),
    "mvb_lm_head_argmax_scratch_bytes": (sz, [i32]),
    "mvb_lm_head_argmax": (i32, [vp, i64, vp, i64, i32, i32, i32, vp, vp, vp, vp, sz, vp, vp]),
    "mvb_sample": (i32, [vp, i64, i32, i32, vp, vp, vp, u64, u64, vp, vp, vp, vp, vp]),
}

_lib = None


class KernelError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def load() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise KernelError(
                f"{_LIB_PATH} is missing: build it with `python -m mini_vllm_b200.csrc.build` "
                "(there is no CPU or PyTorch fallback for these kernels)")
        lib = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().mvb_status_string(status).decode()
        raise KernelError(f"{what}: {msg} (status {status})")
