"""ctypes binding of ``libeasymlx_b200.so`` (the C ABI in ``include/easymlx_b200.h``).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  PyTorch is used only for device memory and streams.
"""

from __future__ import annotations

import ctypes as C
import os
import threading

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libeasymlx_b200.so")

EMLX_OK, EMLX_ERR_INVALID, EMLX_ERR_UNSUPPORTED, EMLX_ERR_CUDA, EMLX_ERR_WORKSPACE, EMLX_ERR_DEVICE = range(6)
F16, BF16, F32 = 0, 1, 2
KV_FLOAT, KV_AFFINE8, KV_AFFINE4 = 0, 8, 4

_DTYPE_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}


class Pool(C.Structure):
    _fields_ = [
        ("key_cache", C.c_void_p), ("value_cache", C.c_void_p),
        ("k_scale", C.c_void_p), ("k_bias", C.c_void_p), ("v_scale", C.c_void_p), ("v_bias", C.c_void_p),
        ("num_blocks", C.c_int64), ("block_size", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("kv_format", C.c_int32), ("kv_dtype", C.c_int32), ("reserved", C.c_int32),
    ]


class Rope(C.Structure):
    _fields_ = [("inv_freq", C.c_void_p), ("dims", C.c_int32), ("traditional", C.c_int32),
                ("position_scale", C.c_float), ("mscale", C.c_float), ("head_dim_if_no_pool", C.c_int32),
                ("reserved", C.c_int32)]


class AttnArgs(C.Structure):
    _fields_ = [
        ("queries", C.c_void_p), ("out", C.c_void_p), ("block_tables", C.c_void_p), ("kv_lens", C.c_void_p),
        ("query_start_loc", C.c_void_p),
        ("total_tokens", C.c_int32), ("num_seqs", C.c_int32), ("num_q_heads", C.c_int32),
        ("max_blocks_per_seq", C.c_int32), ("q_dtype", C.c_int32), ("sliding_window", C.c_int32),
        ("softmax_scale", C.c_float), ("max_query_len", C.c_int32), ("row_class_mask", C.c_int32),
        ("plan_flags", C.c_int32),
        ("plan", C.c_void_p), ("plan_bytes", C.c_size_t), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p),
    ]


# name -> (restype, argtypes); every symbol declared in include/easymlx_b200.h
_I32, _I64, _P = C.c_int32, C.c_int64, C.c_void_p
SIGNATURES = {
    "emlx_last_error": (C.c_char_p, []),
    "emlx_abi_version": (C.c_int, []),
    "emlx_launch_count": (C.c_int64, []),
    "emlx_read_status": (C.c_int, [_P, _P]),
    "emlx_build_metadata": (C.c_int, [_P, _P, _I32, _I32, _P, _I32, _I32, _P, _I32, _I32, _P, _P, _P, _P, _P, _I64, _P,
                                     _I32, _I32, _I32, _I32, _I32, _P, C.c_size_t, _P]),
    "emlx_kv_write": (C.c_int, [_P, _P, _I32, _I32, _P, C.POINTER(Pool), _P, _P]),
    "emlx_kv_write_rope": (C.c_int, [_P, _P, _I32, _P, _P, _I32, _I32, _P, _P, C.POINTER(Rope), C.POINTER(Pool), _P, _P]),
    "emlx_kv_write_step": (C.c_int, [_P, _P, _P, _P, _I32, _P, _P, _I32, _I32, _P, _I32, _I32, _P, _I32, C.POINTER(Pool),
                                    C.POINTER(Rope), _P, _P, _P, _I32, _I32, _I32, _I32, _P, C.c_size_t, _P, _P, _P]),
    "emlx_kv_write_decode": (C.c_int, [_P, _P, _P, _P, _I32, _P, _I32, _P, _I32, _I32, _P, _I32, C.POINTER(Pool),
                                      C.POINTER(Rope), _P, _P, _P, _I32, _I32, _I32, _P, C.c_size_t, _P, _P, _P]),
    "emlx_attn_plan_bytes": (C.c_size_t, [_I32, _I32, _I32, _I32]),
    "emlx_attn_workspace_bytes": (C.c_size_t, [_I32, _I32, _I32, _I32, _I32]),
    "emlx_attn_plan": (C.c_int, [_P, _P, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _P, C.c_size_t, _P]),
    "emlx_attn_plan_flags": (C.c_int, [_I32, _I32, _I32, _I32]),
    "emlx_attn_dequant_bytes": (C.c_size_t, [C.POINTER(Pool), _I32, _I32, _I32, _I32, _I32, _I32]),
    "emlx_attn_unified": (C.c_int, [C.POINTER(AttnArgs), C.POINTER(Pool), _P]),
    "emlx_attn_decode": (C.c_int, [C.POINTER(AttnArgs), C.POINTER(Pool), _P]),
    "emlx_attn_prefill": (C.c_int, [C.POINTER(AttnArgs), C.POINTER(Pool), _P]),
    "emlx_attn_generic": (C.c_int, [C.POINTER(AttnArgs), C.POINTER(Pool), _P]),
    "emlx_selftest_device_once": (C.c_int, []),
    "emlx_selftest_wait_timeout": (C.c_int, [_P, C.c_uint32, _P]),
    "emlx_attn_decode_static": (C.c_int, [C.POINTER(AttnArgs), C.POINTER(Pool), _P]),
    "emlx_attn_row_class": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "emlx_peer_buffer_create": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p), _P]),
    "emlx_peer_buffer_open": (C.c_int, [_P, C.POINTER(C.c_void_p)]),
    "emlx_peer_buffer_close": (C.c_int, [_P]),
    "emlx_peer_buffer_free": (C.c_int, [_P]),
    "emlx_gather_init": (C.c_int, [_P, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), _I32, _I32, _I32, _P]),
    "emlx_attn_decode_gather": (C.c_int, [C.POINTER(AttnArgs), C.POINTER(Pool), _P, _I32, _I32, _P]),
    "emlx_gather_last_tokens": (C.c_int, [_P, C.c_int32, C.c_int64, _P, C.c_int32, _P, _P, _P]),
    "emlx_pad_token_ids": (C.c_int, [_P, C.c_int32, _P, C.c_int32, C.c_int32, _P, _P]),
    "emlx_page_staging_bytes": (C.c_int64, [C.POINTER(Pool)]),
    "emlx_copy_blocks": (C.c_int, [C.POINTER(Pool), _P, C.c_int32, _P, C.c_int64, _P, _P]),
    "emlx_zero_pages": (C.c_int, [C.POINTER(Pool), _P, C.c_int32, _P]),
    "emlx_gather_kv_cache": (C.c_int, [C.POINTER(Pool), _P, C.c_int32, C.c_int32, _P, C.c_int32, C.c_int32, _P, _P, _P, _P]),
    "emlx_rows_assign": (C.c_int, [_P, _P, C.c_int32, C.c_int32, C.c_int32, _P, C.c_int32, C.c_int32, _P]),
    "emlx_rows_update": (C.c_int, [_P, _P, C.c_int32, C.c_int32, _P, C.c_int32, C.c_int32, _P, _P]),
}

_lib = None
_lock = threading.Lock()


def library_path() -> str:
    return _LIB_PATH


def lib() -> C.CDLL:
    """Load the CUDA library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(_LIB_PATH):
                    raise RuntimeError(
                        f"{_LIB_PATH} is missing: build it with `python -m easymlx_b200.build` "
                        "(there is no CPU or PyTorch fallback for this path)"
                    )
                handle = C.CDLL(_LIB_PATH)
                for name, (restype, argtypes) in SIGNATURES.items():
                    fn = getattr(handle, name)
                    fn.restype = restype
                    fn.argtypes = argtypes
                _lib = handle
    return _lib


def last_error() -> str:
    return (lib().emlx_last_error() or b"unknown error").decode(errors="replace")


def check(rc: int) -> None:
    """Turn a status code into the exception the reference would raise for the same fault."""
    if rc == EMLX_OK:
        return
    msg = last_error()
    if rc == EMLX_ERR_INVALID:
        raise ValueError(msg)
    if rc == EMLX_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(msg)


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}; expected float16, bfloat16 or float32") from None


def ptr(t: torch.Tensor | None):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr(device=None):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("easymlx_b200 runs on CUDA tensors only; there is no CPU path")


def launch_count() -> int:
    return int(lib().emlx_launch_count())
