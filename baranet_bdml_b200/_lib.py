"""ctypes binding of libbn_attn.so (the C ABI declared in include/bn_attn.h).

There is no fallback: if the library is missing, or a call returns a non-zero
status, a RuntimeError is raised — the reference's own error convention
(src/utils/check_error.cuh:8-14 turns every failure into std::runtime_error,
which pybind11 surfaces as RuntimeError).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# BN_ATTN_LIB names another build of the same library (e.g. an instrumented one)
LIB_PATH = os.environ.get("BN_ATTN_LIB") or os.path.join(_HERE, "libbn_attn.so")

BN_OK, BN_ERR_INVALID_ARG, BN_ERR_UNSUPPORTED, BN_ERR_CUDA, BN_ERR_ARCH, BN_ERR_TIMEOUT, BN_ERR_WORKSPACE = range(7)
BN_HEADS_COLLAPSED, BN_HEADS_PER_HEAD = 0, 1
BN_PAGE_TOKENS = 16

_i, _i64, _f, _p, _sz = C.c_int, C.c_int64, C.c_float, C.c_void_p, C.c_size_t

# name -> (restype, argtypes); mirrors include/bn_attn.h one to one
SIGNATURES = {
    "bn_last_error": (C.c_char_p, []),
    "bn_version": (_i, []),
    "bn_mm_f32": (_i, [_p, _i64, _i64, _p, _i64, _i64, _p, _i64, _i64, _i, _i, _i, _p]),
    "bn_rope_f32": (_i, [_p, _i64, _i64, _p, _i64, _i64, _i, _i, _i, _f, _i, _p]),
    "bn_embedding_gather_f32": (_i, [_p, _i64, _p, _p, _i64, _i, _i, _i, _p, _p]),
    "bn_argmax_rows_f32": (_i, [_p, _i64, _i64, _p, _i, _i, _p]),
    "bn_add_rmsnorm_bf16": (_i, [_p, _p, _p, _p, _p, _i, _i, _f, _p]),
    "bn_gemm_bf16_nt": (_i, [_p, _p, _p, _i, _i, _i, _p, _p]),
    "bn_gemm_bf16_nt_small_m_workspace_bytes": (_sz, [_i, _i, _i]),
    "bn_gemm_bf16_nt_small_m": (_i, [_p, _p, _p, _i, _i, _i, _p, _sz, _p, _p]),
    "bn_gemm_bf16_nt_skinny": (_i, [_p, _p, _i, _i, _i, _p, _i, _p, _i, _p, _p]),
    "bn_gemm_swiglu_bf16_nt_skinny": (_i, [_p, _p, _p, _p, _i, _i, _i, _p]),
    "bn_gemm_qkv_append_bf16_skinny": (_i, [_p, _p, _i, _i, _i, _i, _i, _p, _p, _i64, _p, _i, _p, _p, _f, _p]),
    "bn_gemm_swiglu_bf16_nt": (_i, [_p, _p, _p, _i, _i, _i, _p, _p]),
    "bn_rmsnorm_f32": (_i, [_p, _i64, _i64, _p, _i64, _p, _i64, _i64, _i, _i, _f, _p]),
    "bn_add_rmsnorm_f32": (_i, [_p, _i64, _i64, _p, _i64, _i64, _p, _i64, _p, _i64, _i64, _p, _i64, _i64, _i, _i, _f,
                                _p]),
    "bn_attn_prefill_f32": (_i, [_p, _i64, _i64, _p, _i64, _i64, _p, _i64, _i64, _p, _i64, _i64,
                                 _i, _i, _i, _i, _f, _f, _i, _i, _i, _i, _p]),
    "bn_attn_prefill_bf16_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "bn_attn_prefill_bf16": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _f, _i, _i, _i, _p, _sz, _p]),
    "bn_attn_prefill_bf16_table": (_i, [_i, _i, _i, _i, _f, _i, _p, _sz, _p]),
    "bn_gemm_qkv_rope_bf16": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _sz, _p, _i64, _p, _i, _p, _p]),
    "bn_kv_append": (_i, [_p, _i64, _p, _i, _p, _p, _i, _p, _p, _i64, _i, _i, _i, _f, _p]),
    "bn_attn_decode_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "bn_attn_decode_paged": (_i, [_p, _p, _i64, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _i, _f, _f, _i, _i, _i,
                                  _p, _sz, _p]),
    "bn_attn_decode_paged_static": (_i, [_p, _p, _i64, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _i, _f, _f, _i, _i, _p]),
    "bn_attn_decode_paged_static_status": (_i, [_p]),
    "bn_attn_lse_combine": (_i, [_p, _p, _i, _i64, _i, _p, _p, _p, _p]),
    "bn_attn_lse_combine_strided": (_i, [_p, _i64, _p, _i64, _i, _i64, _i, _p, _p, _p, _p]),
    "bn_workspace_status": (_i, [_p, _p]),
    "bn_selftest_wait_timeout": (_i, [_p, C.c_uint, _p]),
    "bn_exchange_create": (_i, [_i, _i, _i, _i, C.POINTER(_p)]),
    "bn_exchange_ipc_handle": (_i, [_p, _p]),
    "bn_exchange_open_peers": (_i, [_p, _p, _i]),
    "bn_exchange_combine": (_i, [_p, _p, _p, _p, C.c_uint, _p]),
    "bn_exchange_status": (_i, [_p, _p]),
    "bn_exchange_destroy": (None, [_p]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m baranet_bdml_b200.build` "
                "(there is no CPU fallback for the attention kernels)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().bn_last_error().decode()


def check(status: int) -> None:
    if status != BN_OK:
        raise RuntimeError(f"bn_attn status {status}: {last_error()}")
