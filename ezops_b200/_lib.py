"""ctypes binding of ``libezb200.so`` (the C ABI declared in include/ezb200.h).

The library is the only implementation of the kernels: if it is missing or does
not load, importing the kernel backends raises -- there is no fallback path.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_size_t, c_uint, c_void_p, POINTER
from pathlib import Path

import os

# EZB200_LIBRARY points at an alternative build of the same library (used to A/B kernel variants).
LIB_PATH = Path(os.environ.get("EZB200_LIBRARY") or Path(__file__).resolve().parent / "libezb200.so")

EZB_OK = 0
EZB_ERR_INVALID_ARGUMENT = -1
EZB_ERR_UNSUPPORTED_SHAPE = -2
EZB_ERR_CUDA = -3
EZB_ERR_WORKSPACE = -4
EZB_ERR_DEVICE_FAULT = -5

TUNE = {
    "pdl": 0,
    "gemv_smem_kb": 1,
    "gemv_prefetch": 2,
    "gemv_ctas_per_sm": 3,
    "attn_min_chunk": 4,
    "attn_waves": 5,
    "gemv_kc": 6,
    "gemv_rows8": 7,
    "pdl_across_calls": 8,
    "l2_prefetch": 9,
    "l2_prefetch_kb": 10,
    "gemv_window": 11,
    "l2_prefetch_attn_kb": 12,
    "tc": 13, "attn_waves_uniform": 14, "tp_poll_all": 15, "tp_pull": 16,
    "mega": 17, "mega_l2_stages": 18, "wait_limit_ms": 19, "mega_stages": 20, "mega_inflight": 21, "mega_gate": 22,
    "tp_wait_limit_ms": 23, "tp_strong_stores": 24, "stream_evict_first": 25,
}

# name -> (restype, argtypes); every symbol include/ezb200.h declares
SIGNATURES = {
    "ezb_version": (c_int, []),
    "ezb_strerror": (c_char_p, [c_int]),
    "ezb_last_error_message": (c_char_p, []),
    "ezb_set_tuning": (c_int, [c_int, c_int]),
    "ezb_get_tuning": (c_int, [c_int]),
    "ezb_device_status": (c_int, [POINTER(c_uint), c_int]),
    "ezb_trace_enable": (c_int, [c_void_p, c_void_p, c_uint]),
    "ezb_gemv_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "ezb_gemv_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "ezb_gemv_batched_bf16": (c_int, [c_void_p] * 4 + [c_size_t] + [c_int] * 3 + [c_void_p]),
    "ezb_rmsnorm_f32": (c_int, [c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "ezb_rmsnorm_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "ezb_qk_norm_rope": (c_int, [c_void_p] * 11 + [c_int] * 6 + [c_void_p, c_float, c_void_p]),
    "ezb_attn_decode_workspace_bytes": (c_size_t, [c_int] * 5),
    "ezb_attn_decode": (c_int, [c_void_p] * 5 + [c_size_t] + [c_int] * 5 + [c_void_p, c_void_p]),
    "ezb_attn_decode_static": (c_int, [c_void_p] * 4 + [c_int] * 5 + [c_void_p, c_void_p]),
    "ezb_o_proj_ffn_workspace_bytes": (c_size_t, [c_int] * 4),
    "ezb_o_proj_ffn": (c_int, [c_void_p] * 9 + [c_size_t] + [c_int] * 4 + [c_float, c_void_p]),
    "ezb_qwen3_decode_layer_workspace_bytes": (c_size_t, [c_int] * 7),
    "ezb_qwen3_decode_layer": (c_int, [c_void_p] * 9 + [c_size_t] + [c_int] * 7 + [c_float, c_void_p]),
    "ezb_qwen3_decode_layer_tp_attn": (c_int, [c_void_p] * 7 + [c_size_t] + [c_int] * 6 + [c_float, c_void_p]),
    "ezb_qwen3_decode_layer_tp_ffn": (c_int, [c_void_p] * 7 + [c_size_t] + [c_int] * 3 + [c_float, c_void_p]),
    "ezb_residual_add_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "ezb_copy_pinned": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "ezb_tp_allreduce_f32": (c_int, [c_void_p, POINTER(c_void_p), c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "ezb_attn_decode_paged": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t] + [c_int] * 7
                              + [c_void_p, c_void_p]),
    "ezb_qwen3_decode_stack_paged": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                             c_int, c_void_p, c_size_t] + [c_int] * 6 + [c_float, c_void_p]),
    "ezb_qwen3_decode_stack_workspace_bytes": (c_size_t, [c_int] * 7),
    "ezb_qwen3_decode_stack": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_size_t]
                               + [c_int] * 7 + [c_float, c_void_p]),
    "ezb_qwen3_decode_stack_tp_fused_workspace_bytes": (c_size_t, [c_int] * 7),
    "ezb_qwen3_decode_stack_tp_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                c_size_t, POINTER(c_void_p)] + [c_int] * 9 + [c_float, c_void_p]),
    "ezb_vector_add_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p]),
    "ezb_softmax_f32": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "ezb_reduce_workspace_bytes": (c_size_t, []),
    "ezb_reduce_sum_f32": (c_int, [c_void_p, c_void_p, c_longlong, c_void_p, c_size_t, c_void_p]),
    "ezb_pdl_gemm_f32": (c_int, [c_void_p] * 5 + [c_int] * 5 + [c_void_p]),
    "ezb_launch_count": (ctypes.c_ulonglong, []),
    "ezb_hbm_stream": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_float, c_int, c_int, c_void_p]),
    "ezb_tp_comm_bytes": (c_size_t, [c_int, c_int]),
    "ezb_tp_comm_alloc": (c_int, [c_size_t, POINTER(c_void_p)]),
    "ezb_tp_comm_free": (c_int, [c_void_p]),
    "ezb_ipc_export": (c_int, [c_void_p, c_void_p]),
    "ezb_ipc_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "ezb_ipc_close": (c_int, [c_void_p]),
    "ezb_qwen3_decode_layer_tp_fused": (c_int, [c_void_p] * 9 + [c_size_t, POINTER(c_void_p)] + [c_int] * 9 + [c_float, c_void_p]),
}

_lib = None


class EzbError(RuntimeError):
    """A CUDA-side or workspace failure reported by libezb200."""


def load() -> ctypes.CDLL:
    """Load the shared library and bind every declared entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: the sm_100a kernels are not built. Run `python -m ezops_b200.build` "
            "(needs nvcc); there is no fallback implementation."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the header and the library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


class LayerStruct(ctypes.Structure):
    """``ezb_layer_t``: one decoder layer's device pointers (0 for an absent norm weight)."""

    _fields_ = [(name, c_void_p) for name in ("K_cache", "V_cache", "Wqkv", "Wo", "Wgu", "Wd", "input_norm_w", "post_norm_w",
                                              "q_norm_w", "k_norm_w")]


def check(rc: int) -> None:
    """Turn a return code into the exception the operator API documents:
    ``ValueError`` for rejected arguments / shapes, ``EzbError`` otherwise."""
    if rc == EZB_OK:
        return
    lib = load()
    detail = lib.ezb_last_error_message().decode()
    name = lib.ezb_strerror(rc).decode()
    msg = f"libezb200: {name}: {detail}"
    if rc in (EZB_ERR_INVALID_ARGUMENT, EZB_ERR_UNSUPPORTED_SHAPE):
        raise ValueError(msg)
    raise EzbError(msg)


def set_tuning(**knobs: int) -> None:
    lib = load()
    for key, value in knobs.items():
        check(lib.ezb_set_tuning(TUNE[key], int(value)))


def get_tuning(key: str) -> int:
    return load().ezb_get_tuning(TUNE[key])


def device_status(clear: bool = True) -> int:
    """Synchronise the current device and return its status word (0 = healthy)."""
    word = c_uint(0)
    rc = load().ezb_device_status(ctypes.byref(word), 1 if clear else 0)
    if rc not in (EZB_OK, EZB_ERR_DEVICE_FAULT):
        check(rc)
    return int(word.value)
