"""ctypes front-end of oracle/_ref/libref_llm_kernels.so.  TEST INFRASTRUCTURE ONLY.

The library holds the reference's own CUDA C decode kernels (see build_ref.py), compiled unchanged.
It pins the decode path to outputs of the reference itself and gives the batch-1 decode call its
same-machine baseline.  Only tests and the benchmark's baseline rows may import this module.

Arguments are torch CUDA tensors laid out as the reference's wrappers expect:
q / out [n_heads, head_dim] bf16, caches [n_kv, max_seq, head_dim] bf16, one sequence.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_void_p

from . import build_ref

_lib = None


def available() -> bool:
    return build_ref.available()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError("oracle/_ref/libref_llm_kernels.so is missing: run `python -m oracle.build_ref` "
                               "on a machine that has the reference checkout")
        h = ctypes.CDLL(build_ref.REF_SO)
        h.ref_gqa_decode_online_bf16.restype = c_int
        h.ref_gqa_decode_online_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                 c_int, c_void_p]
        h.ref_kv_append_bf16.restype = c_int
        h.ref_kv_append_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        h.ref_rope_half_split_bf16.restype = c_int
        h.ref_rope_half_split_bf16.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        _lib = h
    return _lib


def _stream():
    import torch
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check_bf16(*tensors):
    import torch
    for t in tensors:
        assert t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()


def gqa_decode_online_bf16(q, k_cache, v_cache, kv_len: int, out=None):
    """The reference kernel on one sequence: q [Hq, D], caches [Hkv, max_seq, D] -> out [Hq, D] bf16."""
    import torch
    _check_bf16(q, k_cache, v_cache)
    n_heads, head_dim = q.shape
    n_kv, max_seq, _ = k_cache.shape
    if out is None:
        out = torch.empty_like(q)
    rc = lib().ref_gqa_decode_online_bf16(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), n_heads,
                                          n_kv, int(kv_len), head_dim, max_seq, _stream())
    if rc != 0:
        raise RuntimeError(f"ref_gqa_decode_online_bf16: status {rc}")
    return out


def kv_append_bf16(k_cache, v_cache, k_in, v_in, pos: int) -> None:
    _check_bf16(k_cache, v_cache, k_in, v_in)
    n_kv, max_seq, head_dim = k_cache.shape
    rc = lib().ref_kv_append_bf16(k_cache.data_ptr(), v_cache.data_ptr(), k_in.data_ptr(), v_in.data_ptr(), int(pos),
                                  n_kv, head_dim, max_seq, _stream())
    if rc != 0:
        raise RuntimeError(f"ref_kv_append_bf16: status {rc}")


def rope_half_split_bf16(x, inv_freq, pos: int) -> None:
    """In place on x [n_heads, head_dim] bf16; rotates ADJACENT pairs (2p, 2p+1) despite the name."""
    import torch
    _check_bf16(x)
    assert inv_freq.is_cuda and inv_freq.dtype == torch.float32 and inv_freq.is_contiguous()
    n_heads, head_dim = x.shape
    rc = lib().ref_rope_half_split_bf16(x.data_ptr(), inv_freq.data_ptr(), int(pos), n_heads, head_dim, _stream())
    if rc != 0:
        raise RuntimeError(f"ref_rope_half_split_bf16: status {rc}")
