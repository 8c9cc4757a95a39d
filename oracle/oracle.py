"""ctypes front-end of the CPU oracle (``oracle.c``).  TEST INFRASTRUCTURE ONLY.

The oracle is the checker for the CUDA kernels and the timed CPU baseline of the
benchmark.  Nothing in the shipped package imports this module; only the tests,
the smoke check and the benchmark's cpu-baseline / reference arm do.

Every function mirrors one C entry point; see ``oracle.c`` for the reference
file:line each one follows.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_float, c_int, c_int32, c_int64, c_uint8, c_uint16, c_uint32, c_uint64

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

MASK_NONE, MASK_CAUSAL, MASK_PADDING = 0, 1, 2
ERR_ZERO_DIM, ERR_MASK_LEN, ERR_HEADS = -1, -4, -5


def build(force: bool = False) -> str:
    """Compile ``oracle.c`` into ``liboracle.so`` next to it (gcc + OpenMP)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        fp, u8p, i32p = POINTER(c_float), POINTER(c_uint8), POINTER(c_int32)
        _lib.orc_flash_forward_ext.argtypes = [c_int64, c_int64, c_int64, c_int, c_int, c_int, fp, fp, fp,
                                               c_int, u8p, c_int64, c_int64, i32p, c_float, c_int, fp, fp]
        _lib.orc_flash_forward_masked.argtypes = [c_int64, c_int64, c_int64, c_int, c_int, c_int, fp, fp, fp,
                                                  c_int, u8p, c_int64, fp]
        _lib.orc_naive_forward_ext.argtypes = [c_int64, c_int64, c_int64, c_int, fp, fp, fp, c_int, u8p,
                                               c_int64, c_int64, i32p, c_float, fp, fp]
        _lib.orc_naive_forward_masked.argtypes = [c_int64, c_int64, c_int64, c_int, fp, fp, fp, c_int, u8p,
                                                  c_int64, fp]
        _lib.orc_attention_general.argtypes = [fp, fp, fp, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int,
                                               i32p, i32p, c_float, fp, fp]
        _lib.orc_flash_backward_ext.argtypes = [c_int64, c_int64, c_int64, c_int, fp, fp, fp, fp, c_int, c_float,
                                                fp, fp, fp, fp]
        _lib.orc_flash_backward.argtypes = [c_int64, c_int64, c_int64, c_int, fp, fp, fp, fp, fp, fp, fp]
        _lib.orc_online_softmax_full.argtypes = [fp, c_int64, fp, fp]
        _lib.orc_combine_tiles.argtypes = [c_float, c_float, c_float, c_float, fp, fp]
        _lib.orc_gqa_forward_f32.argtypes = [fp, fp, fp, fp, c_int64, c_int64, c_int64, c_int64, c_int64, c_int]
        _lib.orc_gqa_decode_cache.argtypes = [fp, fp, fp, i32p, c_int64, c_int64, c_int64, c_int, c_int64,
                                              c_int64, c_int64, c_float, c_int, fp, fp]
        _lib.orc_merge_partials.argtypes = [fp, fp, c_int64, c_int64, c_int, fp, fp]
        _lib.orc_kv_cache_append.argtypes = [fp, fp, fp, fp, c_int64, c_int64, c_int64, c_int, c_int64, c_int64]
        _lib.orc_kv_cache_append.restype = c_int64
        _lib.orc_rope_token.argtypes = [fp, c_int64, c_int64, c_int, i32p, c_float, c_int]
        _lib.orc_f32_to_bf16.argtypes = [fp, POINTER(c_uint16), c_int64]
        _lib.orc_bf16_to_f32.argtypes = [POINTER(c_uint16), fp, c_int64]
        _lib.orc_round_to_bf16.argtypes = [fp, c_int64]
        _lib.orc_fill_normal.argtypes = [fp, c_int64, c_uint64, c_uint64]
        _lib.orc_fill_uniform_int.argtypes = [i32p, c_int64, c_uint64, c_int32, c_int32]
        _lib.orc_fill_lcg.argtypes = [fp, c_int64, c_uint32, c_float]
        _lib.orc_set_threads.argtypes = [c_int]
        _lib.orc_set_gemm_kernel.argtypes = [c_int]
        _lib.orc_get_gemm_kernel.restype = c_int
        _lib.orc_micro_isa.restype = c_int
        _lib.orc_fma_peak_gflops.restype = ctypes.c_double
        _lib.orc_tile_gemm_gflops.restype = ctypes.c_double
        _lib.orc_tile_gemm_gflops.argtypes = [c_int, c_int]
        _lib.orc_get_threads.restype = c_int
    return _lib


def _f(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(POINTER(c_float))


def _opt(a, ty):
    return a.ctypes.data_as(POINTER(ty)) if a is not None else None


def set_threads(n: int) -> None:
    lib().orc_set_threads(int(n))


def get_threads() -> int:
    return int(lib().orc_get_threads())


def set_gemm_kernel(kind: int) -> None:
    """0: the tile products run as plain loop nests (the parity oracle).  1: they run on the register-blocked
    FMA micro-kernels that stand in for the reference's `gemm` crate when the CPU path is timed."""
    lib().orc_set_gemm_kernel(int(kind))


def get_gemm_kernel() -> int:
    return int(lib().orc_get_gemm_kernel())


def micro_isa() -> str:
    return {0: "none", 1: "avx2+fma", 2: "avx512f"}[int(lib().orc_micro_isa())]


def fma_peak_gflops() -> float:
    """One core's measured f32 FMA throughput on the ISA the micro-kernels use (GFLOP/s)."""
    return float(lib().orc_fma_peak_gflops())


def tile_gemm_gflops(dim: int, reps: int = 20000) -> float:
    """Throughput of the two tile products alone (64x64xdim and 64xdimx64) on one core (GFLOP/s)."""
    return float(lib().orc_tile_gemm_gflops(int(dim), int(reps)))


# ----------------------------------------------------------------- inputs

def fill_normal(shape, seed: int, first_index: int = 0) -> np.ndarray:
    out = np.empty(shape, dtype=np.float32)
    lib().orc_fill_normal(_f(out), out.size, seed, first_index)
    return out


def fill_uniform_int(n: int, seed: int, lo: int, hi: int) -> np.ndarray:
    out = np.empty(n, dtype=np.int32)
    lib().orc_fill_uniform_int(out.ctypes.data_as(POINTER(c_int32)), n, seed, lo, hi)
    return out


def fill_lcg(n: int, seed: int, width: float) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().orc_fill_lcg(_f(out), n, seed & 0xFFFFFFFF, width)
    return out


def round_to_bf16(a: np.ndarray) -> np.ndarray:
    out = np.ascontiguousarray(a, dtype=np.float32).copy()
    lib().orc_round_to_bf16(_f(out), out.size)
    return out


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16(_f(a), out.ctypes.data_as(POINTER(c_uint16)), a.size)
    return out


def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().orc_bf16_to_f32(a.ctypes.data_as(POINTER(c_uint16)), _f(out), a.size)
    return out


# ----------------------------------------------------------------- prefill

def flash_forward_masked(q, k, v, mask_kind=MASK_NONE, keep=None, br=64, bc=64):
    """The reference API: q,k,v [B,H,N,D] f32 -> out. Returns (rc, out)."""
    B, H, N, D = q.shape
    out = np.zeros_like(q)
    keep_a = None if keep is None else np.ascontiguousarray(keep, dtype=np.uint8)
    rc = lib().orc_flash_forward_masked(B, H, N, D, br, bc, _f(q), _f(k), _f(v), mask_kind,
                                        _opt(keep_a, c_uint8), 0 if keep_a is None else keep_a.size, _f(out))
    return rc, out


def naive_forward_masked(q, k, v, mask_kind=MASK_NONE, keep=None):
    B, H, N, D = q.shape
    out = np.zeros_like(q)
    keep_a = None if keep is None else np.ascontiguousarray(keep, dtype=np.uint8)
    rc = lib().orc_naive_forward_masked(B, H, N, D, _f(q), _f(k), _f(v), mask_kind,
                                        _opt(keep_a, c_uint8), 0 if keep_a is None else keep_a.size, _f(out))
    return rc, out


def flash_forward_ext(q, k, v, causal=False, keep=None, kv_lens=None, scale=-1.0, br=64, bc=64,
                      fix_leading_masked_tile=True):
    """Extended tiled forward. keep: None, [N] (shared) or [B,N]. Returns (rc, out, lse)."""
    B, H, N, D = q.shape
    out = np.zeros_like(q)
    lse = np.zeros((B, H, N), dtype=np.float32)
    keep_a, stride, klen = None, 0, 0
    if keep is not None:
        keep_a = np.ascontiguousarray(keep, dtype=np.uint8)
        klen = keep_a.shape[-1]
        stride = klen if keep_a.ndim == 2 else 0
    lens_a = None if kv_lens is None else np.ascontiguousarray(kv_lens, dtype=np.int32)
    rc = lib().orc_flash_forward_ext(B, H, N, D, br, bc, _f(q), _f(k), _f(v), int(causal),
                                     _opt(keep_a, c_uint8), klen, stride, _opt(lens_a, c_int32),
                                     scale, int(fix_leading_masked_tile), _f(out), _f(lse))
    return rc, out, lse


def naive_forward_ext(q, k, v, causal=False, keep=None, kv_lens=None, scale=-1.0):
    B, H, N, D = q.shape
    out = np.zeros_like(q)
    lse = np.zeros((B, H, N), dtype=np.float32)
    keep_a, stride, klen = None, 0, 0
    if keep is not None:
        keep_a = np.ascontiguousarray(keep, dtype=np.uint8)
        klen = keep_a.shape[-1]
        stride = klen if keep_a.ndim == 2 else 0
    lens_a = None if kv_lens is None else np.ascontiguousarray(kv_lens, dtype=np.int32)
    rc = lib().orc_naive_forward_ext(B, H, N, D, _f(q), _f(k), _f(v), int(causal), _opt(keep_a, c_uint8),
                                     klen, stride, _opt(lens_a, c_int32), scale, _f(out), _f(lse))
    return rc, out, lse


def attention_general(q, k, v, causal=False, kv_lens=None, q_offsets=None, scale=-1.0):
    """q [B,Hq,Nq,D], k/v [B,Hkv,Nkv,D] -> (rc, out [B,Hq,Nq,D], lse [B,Hq,Nq]); see orc_attention_general."""
    B, Hq, Nq, D = q.shape
    _, Hkv, Nkv, _ = k.shape
    out = np.zeros_like(q)
    lse = np.zeros((B, Hq, Nq), dtype=np.float32)
    lens_a = None if kv_lens is None else np.ascontiguousarray(kv_lens, dtype=np.int32)
    offs_a = None if q_offsets is None else np.ascontiguousarray(q_offsets, dtype=np.int32)
    rc = lib().orc_attention_general(_f(q), _f(k), _f(v), B, Hq, Hkv, Nq, Nkv, D, int(causal),
                                     _opt(lens_a, c_int32), _opt(offs_a, c_int32), scale, _f(out), _f(lse))
    return rc, out, lse


# ----------------------------------------------------------------- online softmax

def flash_backward(q, k, v, d_out, causal=False, scale=-1.0, with_lse=False):
    """cpu_backward.rs:46-185 (+ causal extension): returns (rc, dq, dk, dv[, lse])."""
    B, H, N, D = q.shape
    dq, dk, dv = np.zeros_like(q), np.zeros_like(q), np.zeros_like(q)
    lse = np.zeros((B, H, N), dtype=np.float32) if with_lse else None
    rc = lib().orc_flash_backward_ext(B, H, N, D, _f(q), _f(k), _f(v), _f(d_out), int(causal), scale, _f(dq), _f(dk),
                                      _f(dv), _opt(lse, c_float))
    return (rc, dq, dk, dv, lse) if with_lse else (rc, dq, dk, dv)


def online_softmax_full(xs):
    xs = np.ascontiguousarray(xs, dtype=np.float32)
    m, l = c_float(), c_float()
    lib().orc_online_softmax_full(_f(xs), xs.size, ctypes.byref(m), ctypes.byref(l))
    return m.value, l.value


def combine_tiles(a, b):
    m, l = c_float(), c_float()
    lib().orc_combine_tiles(a[0], a[1], b[0], b[1], ctypes.byref(m), ctypes.byref(l))
    return m.value, l.value


# ----------------------------------------------------------------- GQA / decode

def gqa_forward_f32(q, k, v, batch, n_heads, n_kv_heads, seq_q, seq_kv, head_dim):
    """The reference API over flat f32 buffers. Returns (rc, out)."""
    out = np.zeros(batch * n_heads * seq_q * head_dim, dtype=np.float32)
    rc = lib().orc_gqa_forward_f32(_f(q), _f(k), _f(v), _f(out), batch, n_heads, n_kv_heads, seq_q, seq_kv,
                                   head_dim)
    return rc, out


def gqa_decode_cache(q, k_cache, v_cache, kv_lens, kv_begin=0, kv_end=-1, scale=-1.0, parallel=True):
    """q [B,Hq,D]; caches [B,Hkv,max_seq,D]; kv_lens [B] -> (rc, out [B,Hq,D], lse [B,Hq])."""
    B, Hq, D = q.shape
    _, Hkv, max_seq, _ = k_cache.shape
    out = np.zeros_like(q)
    lse = np.zeros((B, Hq), dtype=np.float32)
    lens = np.ascontiguousarray(kv_lens, dtype=np.int32)
    rc = lib().orc_gqa_decode_cache(_f(q), _f(k_cache), _f(v_cache), lens.ctypes.data_as(POINTER(c_int32)),
                                    B, Hq, Hkv, D, max_seq, kv_begin, kv_end, scale, int(parallel),
                                    _f(out), _f(lse))
    return rc, out, lse


def merge_partials(o_parts, lse_parts):
    """o_parts [R,rows,D], lse_parts [R,rows] -> (out [rows,D], lse [rows])."""
    R, rows, D = o_parts.shape
    out = np.zeros((rows, D), dtype=np.float32)
    lse = np.zeros(rows, dtype=np.float32)
    lib().orc_merge_partials(_f(np.ascontiguousarray(o_parts)), _f(np.ascontiguousarray(lse_parts)), R, rows,
                             D, _f(out), _f(lse))
    return out, lse


def kv_cache_append(k_cache, v_cache, k_new, v_new, cur_len):
    B, Hkv, max_seq, D = k_cache.shape
    n_new = k_new.shape[2]
    return int(lib().orc_kv_cache_append(_f(k_cache), _f(v_cache), _f(np.ascontiguousarray(k_new)),
                                         _f(np.ascontiguousarray(v_new)), B, Hkv, max_seq, D, cur_len, n_new))


def rope_token(x, positions, base=10000.0, style=0):
    """x [B, n_heads, D] f32 -> rotated copy; token b at positions[b]. style 0 half-split, 1 adjacent pairs."""
    B, H, D = x.shape
    out = np.ascontiguousarray(x, dtype=np.float32).copy()
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    lib().orc_rope_token(_f(out), B, H, D, pos.ctypes.data_as(POINTER(c_int32)), base, style)
    return out
