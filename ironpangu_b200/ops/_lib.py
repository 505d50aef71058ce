"""ctypes binding of ``libifab_kernels.so`` (the sm_100a kernel library).

The library is built in-tree by :mod:`ironpangu_b200._build`. Loading never falls back to another
implementation: on a machine with a GPU a missing or unbuildable library is an error.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

from .. import _build


_lock = threading.Lock()
_lib = None

c_void_p, c_int, c_long, c_float, c_u64 = C.c_void_p, C.c_int, C.c_long, C.c_float, C.c_uint64
MAX_RANKS = 8


class IfabFabric(C.Structure):
    """Mirror of ``struct IfabFabric`` in ``csrc/kernels/ifab_kernels.h``."""

    _fields_ = [
        ("data", c_void_p * MAX_RANKS),
        ("flags", c_void_p * MAX_RANKS),
        ("seq", c_void_p),
        ("done", c_void_p),
        ("status", c_void_p),
        ("rank", C.c_int32),
        ("world", C.c_int32),
        ("spin_limit", C.c_uint32),
        ("data_half_bytes", C.c_uint32),
        ("flag_half_words", C.c_uint32),
        ("ll_half_bytes", C.c_uint32),
        ("ll_offset", C.c_uint64),
        ("mc", c_void_p),
    ]


_P = c_void_p
_SIGS = {
    "ifab_device_alloc": [C.POINTER(c_void_p), c_u64],
    "ifab_device_free": [_P],
    "ifab_ipc_export": [_P, C.c_char_p],
    "ifab_ipc_import": [C.c_char_p, C.POINTER(c_void_p)],
    "ifab_ipc_close": [_P],
    "ifab_set_device": [c_int],
    "ifab_set_pdl": [c_int],
    "ifab_peek": [_P, _P, c_u64],
    "ifab_poke": [_P, _P, c_u64],
    "ifab_embedding_bf16": [_P, _P, _P, c_int, c_int, c_int, _P, _P],
    "ifab_swiglu_rows_bf16": [_P, c_long, _P, c_long, c_int, c_int, _P],
    "ifab_rmsnorm_bf16": [_P, c_long, _P, _P, c_long, c_int, c_int, c_float, c_int, _P],
    "ifab_gemv_bf16": [_P, c_long, _P, _P, c_float, c_int, _P, c_long, _P, c_long, c_int, c_int, c_int, c_int, c_int, _P],
    "ifab_gemv_allreduce_bf16": [_P, c_long, _P, _P, c_long, _P, c_long, _P, c_int, c_int, c_int, C.POINTER(IfabFabric), _P],
    "ifab_gemm_bf16": [_P, c_long, _P, c_long, _P, c_long, c_int, _P, c_long, c_int, c_int, c_int, _P, _P],
    "ifab_gemm_bf16_2sm": [_P, c_long, _P, c_long, _P, c_long, c_int, _P, c_long, c_int, c_int, c_int, _P, _P],
    "ifab_gemm_swiglu_bf16_2sm": [_P, c_long, _P, c_long, _P, c_long, c_int, c_int, c_int, _P, _P],
    "ifab_gemm_bf16_2sm_persistent": [_P, c_long, _P, c_long, _P, c_long, c_int, _P, c_long, c_int, c_int, c_int, _P, _P],
    "ifab_gemm_allreduce_bf16": [_P, c_long, _P, c_long, _P, c_long, _P, c_long, c_int, c_int, c_int, C.POINTER(IfabFabric), _P],
    "ifab_gemm_reduce_scatter_bf16": [_P, c_long, _P, c_long, _P, c_long, _P, c_long, c_int, c_int, c_int, C.POINTER(IfabFabric), _P],
    "ifab_router_topk": [_P, c_long, _P, c_float, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_float, _P, _P, c_long, _P],
    "ifab_moe_gate_up_decode": [_P, c_long, _P, c_float, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, c_int, _P, _P],
    "ifab_moe_down_allreduce_decode": [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, c_int, _P, c_long, _P,
                                       c_long, C.POINTER(IfabFabric), _P],
    "ifab_moe_block_decode": [_P, c_long, _P, c_float, _P, _P, c_int, c_int, c_int, c_int, c_float, _P, _P, _P, _P, c_int, c_int,
                              c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P, c_long, _P, C.POINTER(IfabFabric), _P],
    "ifab_mla_head_decode": [_P, c_long, _P, _P, c_float, c_float, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, _P, c_int, c_int, c_float,
                             c_int, c_int, c_int, c_int, c_int, _P, c_long, _P, _P],
    "ifab_mla_head_decode_pf": [_P, c_long, _P, _P, c_float, c_float, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, _P, c_int, c_int, c_float,
                                c_int, c_int, c_int, c_int, c_int, _P, c_long, _P, _P, C.c_uint64, _P, C.c_uint64, _P, C.c_uint64, _P],
    "ifab_quantize_fp8_block": [_P, c_long, c_long, c_int, _P, _P, _P],
    "ifab_dequantize_fp8_block": [_P, _P, c_long, c_int, _P, _P],
    "ifab_moe_gate_up_decode_fp8": [_P, c_long, _P, c_float, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P, c_int, _P, _P],
    "ifab_moe_down_allreduce_decode_fp8": [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P, c_int, _P, c_long, _P,
                                           c_long, C.POINTER(IfabFabric), _P],
    "ifab_lm_head_argmax": [_P, c_long, _P, c_float, _P, _P, c_int, c_int, c_int, c_int, _P, c_u64, _P, _P,
                            C.POINTER(IfabFabric), _P],
    "ifab_sample_topk": [_P, c_long, c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P, c_long, _P, _P, _P, _P, c_u64, _P, _P,
                         C.POINTER(IfabFabric), _P],
    "ifab_mla_kv_write": [_P, c_long, _P, c_float, c_float, _P, _P, _P, c_int, c_int, _P, c_int, c_int, c_int, c_int, _P, _P],
    "ifab_mla_kv_write_split": [_P, c_long, _P, c_long, _P, c_float, c_float, _P, _P, _P, c_int, c_int, _P, c_int, c_int, c_int, c_int, _P, _P],
    "ifab_mla_q_absorb": [_P, c_long, _P, c_float, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P],
    "ifab_mla_decode_attention": [_P, _P, _P, _P, _P, c_int, c_int, c_int, _P, c_int, c_int, c_float, c_int, c_int, c_int,
                                  c_int, c_int, c_int, _P, c_u64, _P, c_int, c_int, _P, c_long, _P, _P],
    "ifab_mla_decode_attention_indexed": [_P, _P, _P, _P, _P, c_int, c_int, c_int, _P, c_int, c_int, c_float, c_int, c_int, c_int,
                                          c_int, c_int, c_int, _P, c_u64, _P, c_int, c_int, _P, c_long, _P, _P, c_int, _P],
    "ifab_gqa_rope_kv_write": [_P, c_long, _P, _P, _P, c_int, c_int, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_float, _P, _P],
    "ifab_mome": [_P, c_long, _P, _P, _P, _P, _P, c_long, c_int, c_int, c_int, c_int, _P],
    "ifab_mhc_pre": [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_float, _P],
    "ifab_mhc_pre_ticketed": [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_float, _P, _P],
    "ifab_mhc_post": [_P, _P, c_long, _P, _P, _P, c_int, c_int, c_int, _P],
    "ifab_mhc_post_norm": [_P, _P, c_long, _P, c_float, _P, _P, _P, c_int, c_int, c_int, _P],
    "ifab_rope_prefix": [_P, c_long, _P, _P, c_long, c_int, c_int, c_int, c_int, c_float, _P],
    "ifab_index_cache_append": [_P, c_long, _P, _P, _P, c_int, c_int, c_int, _P, c_int, c_int, _P, _P],
    "ifab_index_cache_append_q8": [_P, c_long, _P, _P, _P, c_int, c_int, c_int, _P, _P, c_int, c_int, _P, _P],
    "ifab_add_rows": [_P, c_long, _P, c_long, _P, c_long, c_int, c_int, _P],
    "ifab_swiglu_pair": [_P, c_long, _P, c_long, _P, c_long, c_int, c_int, _P],
    "ifab_zc_rmsnorm": [_P, c_long, _P, c_float, _P, c_long, c_int, c_int, c_int, _P],
    "ifab_hybrid_qk_prepare": [_P, c_long, _P, c_long, _P, _P, c_float, _P, c_long, _P, c_long, c_int, c_int, c_int, c_int, _P],
    "ifab_sigmoid_mul": [_P, c_long, _P, c_long, _P, c_long, c_int, c_int, _P],
    "ifab_conv_silu": [_P, c_long, _P, _P, _P, _P, _P, c_long, c_int, c_int, c_int, _P],
    "ifab_delta_prepare": [_P, c_long, _P, c_long, _P, _P, c_float, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, _P],
    "ifab_gated_rmsnorm": [_P, _P, c_long, _P, c_float, _P, c_long, c_int, c_int, c_int, _P],
    "ifab_delta_rule_decode": [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P],
    "ifab_sparse_index": [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, _P, c_int, c_int, c_int, c_int, c_int, _P, _P, _P],
    "ifab_sparse_index_general": [_P, _P, c_long, c_int, _P, _P, _P, _P, _P, c_int, c_int, c_int, _P, c_int, c_int, c_int, c_int, c_int, _P, _P, _P],
    "ifab_sparse_index_q8": [_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, _P, c_int, c_int, c_int, c_int, c_int, _P, _P, _P],
    "ifab_mla_kv_write_q8": [_P, c_long, _P, c_float, c_float, _P, _P, _P, c_int, c_int, _P, c_int, c_int, _P, _P],
    "ifab_mla_kv_write_q8_split": [_P, c_long, _P, c_long, _P, c_float, c_float, _P, _P, _P, c_int, c_int, _P, c_int, c_int, _P, _P],
    "ifab_kv_dequantize_q8": [_P, _P, c_long, _P],
    "ifab_quantize_int8": [_P, c_long, _P, c_long, _P, c_long, c_int, c_int, c_int, _P],
    "ifab_grouped_gemm_bf16": [_P, c_long, c_int, _P, c_int, c_int, c_int, _P, _P, c_int, _P, c_long, c_int, _P, _P],
    "ifab_router_block": [_P, c_long, _P, c_float, _P, _P, _P, _P, _P, _P, c_long, c_int, c_int, c_int, c_int, c_int, c_int,
                          c_float, _P],
    "ifab_moe_dispatch": [_P, c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, c_int, _P],
    "ifab_moe_gather": [_P, c_long, _P, _P, _P, c_long, c_int, c_int, _P],
    "ifab_moe_combine": [_P, c_long, _P, _P, c_int, c_int, c_int, _P, c_long, _P, c_long, _P, _P, c_long, _P],
    "ifab_mla_q_rope": [_P, c_long, _P, _P, c_int, c_int, c_int, c_int, c_float, _P],
    "ifab_mla_merge": [_P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P],
    "ifab_allreduce_rows": [_P, _P, c_long, _P, c_long, c_long, c_int, C.POINTER(IfabFabric), _P],
    "ifab_fa_prefill_bf16": [_P, c_long, c_int, _P, c_long, c_int, _P, c_long, _P, c_long, c_int, c_int, c_int, _P, c_long, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_float, _P, _P],
    "ifab_mla_q_rope_inplace": [_P, c_long, _P, c_int, c_int, c_int, c_int, c_float, _P],
    "ifab_mla_ctx_gather": [_P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P],
    "ifab_gqa_ctx_gather": [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, c_long, _P, _P],
    "ifab_allreduce_rows_nvls": [_P, _P, _P, c_long, _P, c_long, c_long, c_int, _P, C.POINTER(IfabFabric), _P],
    "ifab_gqa_decode_attention": [_P, c_long, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int,
                                  c_int, c_int, _P, c_u64, _P, c_long, _P, _P],
}


def lib_path() -> Path:
    return _build.KERNEL_LIB


def load(build: bool = True):
    """Return the loaded kernel library, building it first when the sources changed."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.KERNEL_LIB
        if build:
            try:
                path = _build.build_kernels()
            except Exception:
                if not path.exists():
                    raise
        if not path.exists():
            raise RuntimeError(f"{path} is missing: run `python -m ironpangu_b200._build`")
        lib = C.CDLL(str(path))
        lib.ifab_error_string.restype = C.c_char_p
        lib.ifab_error_string.argtypes = [c_int]
        for name, sig in _SIGS.items():
            fn = getattr(lib, name, None)
            if fn is None:
                continue
            fn.argtypes = sig
            fn.restype = c_int
        import os
        if os.environ.get("IFAB_PDL", "1") == "0":  # A/B switch: plain stream-ordered launches
            lib.ifab_set_pdl(0)
        _lib = lib
        return lib


launch_count = 0          # launches of this library's kernels since the process started (every entry point reports here)


def check(rc: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if rc != 0:
        msg = load().ifab_error_string(rc).decode()
        raise RuntimeError(f"{what} failed: {msg} (code {rc})")
