"""ctypes binding of ``librustorch_attn.so`` — the only way this package computes anything.

There is no fallback: if the shared library is missing (or its CUDA kernels cannot be
launched) the calls raise.  ``include/rustorch_attn.h`` is the authoritative declaration
of every symbol bound here.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint8, c_void_p

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "librustorch_attn.so")

# status codes (include/rustorch_attn.h)
RT_OK = 0
RT_ERR_ZERO_DIM = -1
RT_ERR_BUFFER_SHAPE = -2
RT_ERR_OUTPUT_SHAPE = -3
RT_ERR_MASK_LEN = -4
RT_ERR_HEAD_COUNT = -5
RT_ERR_WRONG_INPUT_LEN = -6
RT_ERR_UNSUPPORTED = -7
RT_ERR_NULL_POINTER = -8
RT_ERR_BAD_LENGTH = -9
RT_ERR_WORKSPACE = -10
RT_ERR_ALIGNMENT = -11
RT_ERR_DEVICE_TIMEOUT = -12
RT_ERR_STATIC_SCRATCH = -13

RT_MASK_NONE, RT_MASK_CAUSAL = 0, 1
RT_MASKKIND_NONE, RT_MASKKIND_CAUSAL, RT_MASKKIND_PADDING = 0, 1, 2
RT_PRECISION_F32, RT_PRECISION_BF16 = 0, 1
RT_ROPE_HALF_SPLIT, RT_ROPE_ADJACENT = 0, 1

_fp = POINTER(c_float)
_i32p = POINTER(c_int32)
_u8p = POINTER(c_uint8)

# name -> (restype, argtypes); mirrors include/rustorch_attn.h one to one
PROTOTYPES = {
    "rt_attn_version": (c_int, []),
    "rt_attn_error_string": (c_char_p, [c_int]),
    "rt_attn_device_status": (c_int, [POINTER(c_int)]),
    "rt_attn_prefill_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                     c_int, c_int, c_void_p, c_void_p, c_int64, c_float, c_void_p]),
    "rt_attn_prefill_gqa_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                         c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64,
                                         c_float, c_void_p]),
    "rt_attn_prefill_strided_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                             c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_int, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_void_p]),
    "rt_attn_prefill_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                    c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_float,
                                    c_void_p]),
    "rt_attn_backward_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "rt_attn_backward_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_float, c_void_p, c_size_t,
                                     c_void_p]),
    "rt_attn_backward_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_float, c_void_p, c_size_t,
                                      c_void_p]),
    "rt_flash_backward_f32_host": (c_int, [_fp, c_size_t, _fp, c_size_t, _fp, c_size_t, _fp, c_size_t, _fp, c_size_t,
                                           _fp, c_size_t, _fp, c_size_t, c_int64, c_int64, c_int64, c_int64, c_int]),
    "rt_flash_forward_f32_host": (c_int, [_fp, c_size_t, _fp, c_size_t, _fp, c_size_t, _fp, c_size_t, c_int64,
                                          c_int64, c_int64, c_int64, c_int, _u8p, c_size_t, c_int]),
    "rt_attn_prefill_bf16_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                          c_int64, c_int, c_int, c_void_p, c_float]),
    "rt_gqa_decode_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int, c_int64]),
    "rt_gqa_decode_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                   c_int64, c_int, c_int64, c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p,
                                   c_size_t, c_void_p]),
    "rt_gqa_decode_record_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                                          c_int64, c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p, c_size_t,
                                          c_void_p]),
    "rt_splitkv_push_record": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, ctypes.c_uint32, c_void_p]),
    "rt_gqa_decode_record_push_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                               ctypes.c_uint32, c_void_p, c_int64, c_int64, c_int64, c_int, c_int64,
                                               c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p, c_size_t,
                                               c_void_p]),
    "rt_attn_merge_records_after": (c_int, [c_void_p, c_void_p, ctypes.c_uint32, c_int64, c_int64, c_int64, c_int,
                                            c_void_p, c_void_p, c_void_p, c_void_p]),
    "rt_gqa_decode_exchange_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_void_p, c_int, c_int, ctypes.c_uint32, c_int64, c_int, c_int64,
                                            c_int64, c_int64, c_int, c_int64, c_void_p, c_int64, c_int64, c_int64, c_float,
                                            c_void_p, c_size_t, c_void_p]),
    "rt_attn_merge_records_after_rows": (c_int, [c_void_p, c_void_p, ctypes.c_uint32, c_int64, c_int64, c_int64, c_int,
                                                 c_void_p, c_void_p, c_void_p, c_void_p]),
    "rt_gqa_decode_exchange_ll_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_int, c_int, ctypes.c_uint32, c_int64, c_int, c_int64, c_int64,
                                               c_int64, c_int, c_int64, c_void_p, c_int64, c_int64, c_int64, c_float,
                                               c_void_p, c_size_t, c_void_p]),
    "rt_attn_merge_ll_rows": (c_int, [c_void_p, ctypes.c_uint32, c_int64, c_int, c_int64, c_int, c_void_p, c_void_p,
                                      c_void_p, c_void_p]),
    "rt_attn_merge_records": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "rt_gqa_decode_online_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                          c_void_p, c_size_t, c_void_p]),
    "rt_gqa_decode_online_bf16_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                 c_int, c_void_p]),
    "rt_attn_merge_partials": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                       c_void_p]),
    "rt_gqa_forward_f32_host": (c_int, [_fp, c_size_t, _fp, c_size_t, _fp, c_size_t, _fp, c_size_t, c_int64, c_int64,
                                        c_int64, c_int64, c_int64, c_int64]),
    "rt_kv_append_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, c_int64,
                                  c_void_p, c_void_p]),
    "rt_rope_kv_append_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                       c_int, c_int64, c_int64, c_void_p, c_int, c_void_p]),
    "rt_convert_f32_to_bf16": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "rt_convert_bf16_to_f32": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "rt_debug_tc_selftest": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """Loads the C-ABI library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m rustorch_b200.build`. "
                "This package has no CPU or PyTorch fallback.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)  # AttributeError if the library does not export it
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def error_string(status: int) -> str:
    return lib().rt_attn_error_string(int(status)).decode()


class CudaError(RuntimeError):
    """Mirror of the reference's ``CudaError::Driver{code, location}`` (rustorch-cuda/src/error.rs:8-62)."""

    def __init__(self, code: int, location: str):
        self.code, self.location = code, location
        super().__init__(f"{location}: status {code}: {error_string(code)}")


class Unsupported(CudaError):
    """Mirror of ``CudaError::Unsupported{msg}``."""


def check(status: int, location: str) -> None:
    if status == RT_OK:
        return
    if status == RT_ERR_UNSUPPORTED:
        raise Unsupported(status, location)
    raise CudaError(status, location)


def device_status() -> int:
    """Synchronises and returns the device status word (0 = clean); clears it."""
    v = c_int(0)
    rc = lib().rt_attn_device_status(ctypes.byref(v))
    if rc not in (RT_OK, RT_ERR_DEVICE_TIMEOUT):
        raise CudaError(rc, "rt_attn_device_status")
    return v.value
