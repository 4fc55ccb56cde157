"""ctypes binding of ``libnvfp4_b200.so`` (the C ABI in ``include/nvfp4_b200.h``).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnvfp4_b200.so")

IMPL_AUTO, IMPL_GENERIC, IMPL_SM100 = 0, 1, 2
DECODE_PROGRAMMATIC_LAUNCH = 1
DECODE_REUSE_WORK_LIST = 2
DECODE_PERSISTENT = 4
DECODE_WIDE_FORM = 8
DECODE_MERGE_IN_LAUNCH = 16
DECODE_HOST_IO_DIRECT = 32
STATUS_BAD_PAGE_ID, STATUS_BAD_TAIL_ID, STATUS_WAIT_TIMEOUT, STATUS_BAD_LENGTH = 1, 2, 4, 8
ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED = 1, 2, 3

EXPORTS = (
    "nvfp4_last_error",
    "nvfp4_version",
    "nvfp4_device_supported",
    "nvfp4_quantize_q",
    "nvfp4_quantize_kv_pages",
    "nvfp4_tail_append",
    "nvfp4_tail_reset",
    "nvfp4_tail_flush",
    "nvfp4_decode",
    "nvfp4_decode_workspace_bytes",
    "nvfp4_decode_impl_available",
    "nvfp4_lse_merge",
    "nvfp4_lse_merge_ptrs",
    "nvfp4_peer_merge",
    "nvfp4_control_step",
    "nvfp4_control_step_balanced",
    "nvfp4_work_table",
    "nvfp4_write_kv",
    "nvfp4_key_sum_accumulate",
    "nvfp4_push_merge",
    "nvfp4_decode_exchange",
    "nvfp4_push_merge_inbox_floats",
    "nvfp4_decode_split_static",
    "nvfp4_decode_balanced",
    "nvfp4_decode_balanced_capacity",
    "nvfp4_decode_balanced_workspace_bytes",
    "nvfp4_static_workspace_bytes",
    "nvfp4_decode_split_static_error",
    "nvfp4_decode_persistent_workspace_bytes",
    "nvfp4_decode_persistent_supported",
    "nvfp4_decode_host_io",
)


class DecodeArgs(ctypes.Structure):
    """Mirror of ``struct nvfp4_decode_args``."""

    _fields_ = [
        ("q_fp4", c_void_p),
        ("q_sf", c_void_p),
        ("q_bf16", c_void_p),
        ("q_bf16_row_stride", c_int64),
        ("q_bf16_head_stride", c_int64),
        ("k_packed", c_void_p),
        ("k_pitch", c_int64),
        ("k_sf", c_void_p),
        ("k_sf_pitch", c_int64),
        ("v_packed", c_void_p),
        ("v_pitch", c_int64),
        ("v_sf", c_void_p),
        ("v_sf_pitch", c_int64),
        ("num_pages", c_int64),
        ("page_table", c_void_p),
        ("page_table_row_stride", c_int64),
        ("max_pages", c_int32),
        ("seqused_fp4", c_void_p),
        ("tail_key", c_void_p),
        ("tail_value", c_void_p),
        ("tail_pages", c_int64),
        ("tail_ids", c_void_p),
        ("seqused_tail", c_void_p),
        ("out", c_void_p),
        ("out_indices", c_void_p),
        ("o_partial", c_void_p),
        ("lse_partial", c_void_p),
        ("rows", c_int32),
        ("heads_q", c_int32),
        ("heads_kv", c_int32),
        ("softmax_scale", c_float),
        ("num_splits", c_int32),
        ("impl", c_int32),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
        ("status", c_void_p),
        ("flags", ctypes.c_uint32),
        ("append_key", c_void_p),
        ("append_value", c_void_p),
        ("append_key_token_stride", c_int64),
        ("append_value_token_stride", c_int64),
        ("key_shift", c_void_p),
    ]


class LibraryNotBuiltError(RuntimeError):
    """``libnvfp4_b200.so`` is missing: run ``python -m nvfp4_attn_kernel_b200.build``."""


_lib = None


def _declare(lib) -> None:
    lib.nvfp4_last_error.restype = c_char_p
    lib.nvfp4_last_error.argtypes = []
    lib.nvfp4_version.restype = c_int
    lib.nvfp4_device_supported.restype = c_int
    lib.nvfp4_device_supported.argtypes = [c_int]
    lib.nvfp4_quantize_q.restype = c_int
    lib.nvfp4_quantize_q.argtypes = [
        c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_int, c_void_p,
    ]
    lib.nvfp4_quantize_kv_pages.restype = c_int
    lib.nvfp4_quantize_kv_pages.argtypes = [
        c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int64,
        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_void_p,
    ]
    lib.nvfp4_tail_append.restype = c_int
    lib.nvfp4_tail_append.argtypes = [
        c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int64,
        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
    ]
    lib.nvfp4_tail_reset.restype = c_int
    lib.nvfp4_tail_reset.argtypes = [
        c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p,
        c_int, c_int, c_void_p,
    ]
    lib.nvfp4_tail_flush.restype = c_int
    lib.nvfp4_tail_flush.argtypes = [
        c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
        c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_void_p,
    ]
    lib.nvfp4_decode.restype = c_int
    lib.nvfp4_decode.argtypes = [ctypes.POINTER(DecodeArgs), c_void_p]
    lib.nvfp4_decode_workspace_bytes.restype = c_size_t
    lib.nvfp4_decode_workspace_bytes.argtypes = [c_int, c_int, c_int]
    lib.nvfp4_decode_impl_available.restype = c_int
    lib.nvfp4_decode_impl_available.argtypes = [c_int, c_int, c_int]
    lib.nvfp4_lse_merge.restype = c_int
    lib.nvfp4_lse_merge.argtypes = [
        c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p,
    ]
    lib.nvfp4_lse_merge_ptrs.restype = c_int
    lib.nvfp4_lse_merge_ptrs.argtypes = [
        c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
        c_void_p,
    ]


def _declare_peer(lib) -> None:
    lib.nvfp4_peer_merge.restype = c_int
    lib.nvfp4_peer_merge.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int,
        c_void_p, c_void_p,
    ]


class ExchangeArgs(ctypes.Structure):
    """Mirror of ``struct nvfp4_exchange_args``."""

    _fields_ = [
        ("inbox_ptrs", c_void_p),
        ("flag_ptrs", c_void_p),
        ("epoch_state", c_void_p),
        ("tile_counters", c_void_p),
        ("out", c_void_p),
        ("out_is_f32", c_int32),
        ("rank", c_int32),
        ("world", c_int32),
    ]


def _declare_control(lib) -> None:
    lib.nvfp4_control_step.restype = c_int
    lib.nvfp4_control_step.argtypes = [c_void_p, c_int64, c_int] + [c_void_p] * 13 + [c_int, c_int, c_int, c_void_p]
    lib.nvfp4_control_step_balanced.restype = c_int
    lib.nvfp4_control_step_balanced.argtypes = ([c_void_p, c_int64, c_int] + [c_void_p] * 13 + [c_int] * 7
                                                + [c_void_p, c_size_t, c_void_p])
    lib.nvfp4_decode_exchange.restype = c_int
    lib.nvfp4_decode_exchange.argtypes = [ctypes.POINTER(DecodeArgs), ctypes.POINTER(ExchangeArgs), c_void_p]
    lib.nvfp4_push_merge.restype = c_int
    lib.nvfp4_push_merge.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int,
                                     c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p]
    lib.nvfp4_push_merge_inbox_floats.restype = c_size_t
    lib.nvfp4_push_merge_inbox_floats.argtypes = [c_int, c_int, c_int]
    lib.nvfp4_write_kv.restype = c_int
    lib.nvfp4_write_kv.argtypes = ([c_void_p, c_void_p, c_int64, c_int64, c_void_p]
                                   + [c_void_p, c_int64] * 4 + [c_void_p, c_void_p, c_int]
                                   + [c_void_p, c_void_p, c_int64] + [c_void_p] * 4
                                   + [c_int, c_int, c_int, c_void_p])
    lib.nvfp4_key_sum_accumulate.restype = c_int
    lib.nvfp4_key_sum_accumulate.argtypes = [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]
    lib.nvfp4_work_table.restype = c_int
    lib.nvfp4_work_table.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                     c_int, c_int, c_void_p]


def _declare_static(lib) -> None:
    lib.nvfp4_decode_split_static.restype = c_int
    lib.nvfp4_decode_split_static.argtypes = [ctypes.POINTER(DecodeArgs), c_void_p]
    lib.nvfp4_decode_balanced.restype = c_int
    lib.nvfp4_decode_balanced.argtypes = [ctypes.POINTER(DecodeArgs), c_int, c_void_p]
    lib.nvfp4_decode_balanced_capacity.restype = ctypes.c_int64
    lib.nvfp4_decode_balanced_capacity.argtypes = [c_int, c_int, c_int]
    lib.nvfp4_decode_balanced_workspace_bytes.restype = c_size_t
    lib.nvfp4_decode_balanced_workspace_bytes.argtypes = [c_int, c_int, c_int, c_int]
    lib.nvfp4_decode_persistent_workspace_bytes.restype = c_size_t
    lib.nvfp4_decode_persistent_workspace_bytes.argtypes = [c_int, c_int, c_int]
    lib.nvfp4_decode_persistent_supported.restype = c_int
    lib.nvfp4_decode_persistent_supported.argtypes = [c_int, c_int, c_int]
    lib.nvfp4_decode_host_io.restype = c_int
    lib.nvfp4_decode_host_io.argtypes = [ctypes.POINTER(DecodeArgs), c_void_p, c_size_t, c_void_p, c_size_t, c_void_p]
    lib.nvfp4_static_workspace_bytes.restype = c_size_t
    lib.nvfp4_static_workspace_bytes.argtypes = []
    lib.nvfp4_decode_split_static_error.restype = c_char_p
    lib.nvfp4_decode_split_static_error.argtypes = []


def load():
    """Load the shared library once and return the ctypes handle."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryNotBuiltError(
                f"{LIB_PATH} does not exist; build it with "
                "`python -m nvfp4_attn_kernel_b200.build` (needs nvcc). There is no "
                "CPU or PyTorch fallback for these kernels."
            )
        lib = ctypes.CDLL(LIB_PATH)
        _declare(lib)
        _declare_peer(lib)
        _declare_static(lib)
        _declare_control(lib)
        _lib = lib
    return _lib


def last_error() -> str:
    return load().nvfp4_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    """Turn a non-zero return code into the matching Python exception."""
    if code == 0:
        return
    message = last_error()
    if code == ERR_INVALID:
        raise ValueError(message)
    if code == ERR_UNSUPPORTED:
        raise NotImplementedError(message)
    raise RuntimeError(message)


def ptr(tensor) -> int | None:
    return None if tensor is None else tensor.data_ptr()
