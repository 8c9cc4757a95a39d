"""Host-side mirror of the reference's GQA / KV-cache decode API on top of the C ABI.

* ``gqa_forward_f32``   — rustorch_nn::gqa::gqa_forward_f32 (crates/rustorch-nn/src/gqa.rs:94-105),
                          host f32 buffers, ``GQAError`` variants.
* ``LlmKernels``        — the attention part of rustorch_cuda::llm_kernels::LlmKernels
                          (crates/rustorch-cuda/src/llm_kernels.rs:872-958, 1000-1042): raw device
                          pointers as integers, one sequence, bf16.
* ``gqa_decode``        — batched split-KV decode over a [B,Hkv,max_seq,D] cache with per-sequence
                          lengths (what a batched server needs; the reference has batch 1 only).
* ``merge_partials``    — (O, LSE) merge of KV shards (combine_tiles, online_softmax.rs:105-131).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_float
from typing import Optional

import numpy as np

from . import _lib


# ---------------------------------------------------------------- errors (gqa.rs:37-78)
class GQAError(Exception):
    pass


class HeadCountMismatch(GQAError):
    def __init__(self, n_heads: int, n_kv_heads: int):
        self.n_heads, self.n_kv_heads = n_heads, n_kv_heads
        super().__init__(f"gqa: n_heads {n_heads} not divisible by n_kv_heads {n_kv_heads}")


class WrongInputLen(GQAError):
    def __init__(self, which: str, expected: int, got: int):
        self.which, self.expected, self.got = which, expected, got
        super().__init__(f"gqa: {which} expected {expected} f32, got {got}")


def _f32(a, name):
    if not isinstance(a, np.ndarray) or a.dtype != np.float32 or not a.flags["C_CONTIGUOUS"]:
        raise TypeError(f"{name} must be a C-contiguous float32 numpy array")
    return a.ctypes.data_as(POINTER(c_float))


def gqa_forward_f32(q, k, v, out, batch: int, n_heads: int, n_kv_heads: int, seq_q: int, seq_kv: int,
                    head_dim: int) -> None:
    """gqa.rs:94-210 on the GPU (f32 arithmetic).  Buffers are flat host f32 arrays."""
    if n_kv_heads == 0 or n_heads % n_kv_heads != 0:
        raise HeadCountMismatch(n_heads, n_kv_heads)
    q_len = batch * n_heads * seq_q * head_dim
    kv_len = batch * n_kv_heads * seq_kv * head_dim
    for which, buf, exp in (("q", q, q_len), ("k", k, kv_len), ("v", v, kv_len), ("out", out, q_len)):
        if buf.size != exp:
            raise WrongInputLen(which, exp, buf.size)
    rc = _lib.lib().rt_gqa_forward_f32_host(_f32(q, "q"), q.size, _f32(k, "k"), k.size, _f32(v, "v"), v.size,
                                            _f32(out, "out"), out.size, batch, n_heads, n_kv_heads, seq_q, seq_kv,
                                            head_dim)
    if rc == _lib.RT_ERR_HEAD_COUNT:
        raise HeadCountMismatch(n_heads, n_kv_heads)
    if rc == _lib.RT_ERR_WRONG_INPUT_LEN:  # unreachable after the checks above; keep the variant's fields meaningful
        raise WrongInputLen("q", q_len, q.size)
    _lib.check(rc, "rt_gqa_forward_f32_host")


def _stream_ptr(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def _guard(name: str, t, dtype, like=None, shape=None):
    """Refuses, before anything is launched, a tensor the kernels would misread: they take raw device
    pointers, so a CPU tensor would hand them a host address (an illegal-address fault on the GPU), and a
    tensor of another dtype or with gaps would silently be read as dense data of the expected type."""
    import torch
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA tensor (got device {t.device})")
    if like is not None and t.device != like.device:
        raise TypeError(f"{name} is on {t.device}, expected {like.device}")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise TypeError(f"{name} must be contiguous")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise TypeError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


def _guard_decode_args(q, k_cache, v_cache, kv_lens=None, workspace=None):
    """Shape / dtype / device checks shared by the decode wrappers; returns (B, Hq, Hkv, D, max_seq).
    One combined test on the hot path; the per-argument diagnosis only runs when it fails."""
    import torch
    try:
        B, Hq, D = q.shape
        Bk, Hkv, max_seq, Dk = k_cache.shape
        bf16, dev = torch.bfloat16, q.device
        if (q.is_cuda and q.dtype is bf16 and k_cache.dtype is bf16 and v_cache.dtype is bf16 and k_cache.device == dev
                and v_cache.device == dev and Bk == B and Dk == D and v_cache.shape == k_cache.shape
                and q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
                and (kv_lens is None or (kv_lens.dtype is torch.int32 and kv_lens.device == dev
                                         and kv_lens.shape == (B,) and kv_lens.is_contiguous()))
                and (workspace is None or (workspace.dtype is torch.uint8 and workspace.device == dev
                                           and workspace.is_contiguous()))):
            return B, Hq, Hkv, D, max_seq
    except (AttributeError, ValueError, TypeError):
        pass
    _guard("q", q, torch.bfloat16)
    if q.dim() != 3:
        raise TypeError(f"q must be [B, Hq, D], got {tuple(q.shape)}")
    B, Hq, D = q.shape
    _guard("k_cache", k_cache, torch.bfloat16, like=q)
    if k_cache.dim() != 4 or k_cache.shape[0] != B or k_cache.shape[3] != D:
        raise TypeError(f"k_cache must be [B={B}, Hkv, max_seq, D={D}], got {tuple(k_cache.shape)}")
    _guard("v_cache", v_cache, torch.bfloat16, like=q, shape=k_cache.shape)
    if kv_lens is not None:
        _guard("kv_lens", kv_lens, torch.int32, like=q, shape=(B,))
    if workspace is not None:
        _guard("workspace", workspace, torch.uint8, like=q)
    raise TypeError("decode arguments are inconsistent")


def decode_workspace_bytes(batch: int, n_heads: int, n_kv_heads: int, head_dim: int, max_seq: int) -> int:
    return int(_lib.lib().rt_gqa_decode_workspace_bytes(batch, n_heads, n_kv_heads, head_dim, max_seq))


class LlmKernels:
    """Attention subset of the reference's ``LlmKernels`` (llm_kernels.rs:540-641 holds compiled
    modules; this holds the split-KV scratch instead).  Pointers are device addresses as ints,
    like the reference's ``u64`` arguments."""

    def __init__(self):
        self._ws = None

    def _workspace(self, nbytes: int):
        import torch
        if nbytes == 0:
            return None, 0
        if self._ws is None or self._ws.numel() < nbytes:
            self._ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        return self._ws.data_ptr(), self._ws.numel()

    def gqa_decode_online_bf16(self, stream, q: int, k_cache: int, v_cache: int, out: int, n_heads: int, n_kv: int,
                               kv_len: int, head_dim: int, max_seq: int) -> None:
        """llm_kernels.rs:915-958."""
        ws, ws_bytes = self._workspace(decode_workspace_bytes(1, n_heads, max(n_kv, 1), head_dim, max_seq))
        rc = _lib.lib().rt_gqa_decode_online_bf16(q, k_cache, v_cache, out, n_heads, n_kv, kv_len, head_dim, max_seq,
                                                  ws, ws_bytes, _stream_ptr(stream))
        _lib.check(rc, "gqa_decode_online_bf16::launch")

    # llm_kernels.rs:1000-1042: same contract, same result.
    gqa_decode_naive_bf16 = gqa_decode_online_bf16

    def kv_append_bf16(self, stream, k_cache: int, v_cache: int, k_in: int, v_in: int, pos: int, n_kv: int,
                       head_dim: int, max_seq: int) -> None:
        """llm_kernels.rs:872-911."""
        rc = _lib.lib().rt_kv_append_bf16(k_cache, v_cache, k_in, v_in, 1, n_kv, head_dim, max_seq, pos, None,
                                          _stream_ptr(stream))
        _lib.check(rc, "kv_append_bf16::launch")


STATIC_SCRATCH_BYTES = 8 << 20  # RT_DECODE_STATIC_SCRATCH_BYTES


def gqa_decode_online_bf16_static(stream, q: int, k_cache: int, v_cache: int, out: int, n_heads: int, n_kv: int,
                                  kv_len: int, head_dim: int, max_seq: int) -> None:
    """``rt_gqa_decode_online_bf16_static``: the reference's exact ten-argument decode call for callers
    that cannot pass scratch memory (a fixed FFI signature, or a runtime that forbids allocation once
    its pools are set up).  Uses an 8 MiB scratch array built into the library, allocates nothing, and
    gives the same result as ``LlmKernels.gqa_decode_online_bf16``.  Calls share that array, so calls
    that overlap on the GPU race; the first call on a device should precede any stream capture."""
    rc = _lib.lib().rt_gqa_decode_online_bf16_static(q, k_cache, v_cache, out, n_heads, n_kv, kv_len, head_dim,
                                                     max_seq, _stream_ptr(stream))
    if rc == _lib.RT_ERR_STATIC_SCRATCH:
        need = decode_workspace_bytes(1, n_heads, max(n_kv, 1), head_dim, max_seq)
        raise _lib.CudaError(rc, f"gqa_decode_online_bf16_static: needs {need} bytes of scratch, the built-in "
                                 f"buffer holds {STATIC_SCRATCH_BYTES}")
    _lib.check(rc, "gqa_decode_online_bf16_static::launch")


_default_ws = {}
_ws_bytes_cache: dict = {}


def _implicit_workspace(device, nbytes: int, stream: Optional[int] = None):
    """The split-KV scratch used when the caller passes no ``workspace=``: one buffer per (device, CUDA
    stream, size).  Two decodes of equal shape on different streams therefore never share chunk partials
    and completion counters; calls on ONE stream run in order and may share them."""
    import torch
    key = (device.index, stream if stream is not None else torch.cuda.current_stream(device).cuda_stream, nbytes)
    ws = _default_ws.get(key)
    if ws is None:
        ws = _default_ws[key] = torch.empty(nbytes, dtype=torch.uint8, device=device)
    return ws


def gqa_decode(q, k_cache, v_cache, kv_lens=None, kv_len: Optional[int] = None, kv_begin: int = 0, kv_end: int = -1,
               scale: Optional[float] = None, out_dtype=None, return_lse: bool = True, workspace=None, out=None,
               lse=None):
    """Batched single-token GQA decode via ``rt_gqa_decode_bf16``.

    q [B,Hq,D] bf16, caches [B,Hkv,max_seq,D] bf16 (CUDA, contiguous); kv_lens int32 CUDA [B] or a
    uniform ``kv_len``.  Returns (out [B,Hq,D] in ``out_dtype`` (bf16 default, or float32), lse or None).
    ``out`` / ``lse`` may be passed in (a decode loop reuses them: nothing is allocated per step).
    """
    import torch
    B, Hq, Hkv, D, max_seq = _guard_decode_args(q, k_cache, v_cache, kv_lens, workspace)
    if out is None:
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((B, Hq, D), dtype=out_dtype, device=q.device)
    else:
        out_dtype = out.dtype
        if out_dtype not in (torch.bfloat16, torch.float32):
            raise TypeError(f"out must be bfloat16 or float32, got {out_dtype}")
        _guard("out", out, out_dtype, like=q, shape=(B, Hq, D))
    if lse is None and return_lse:
        lse = torch.empty((B, Hq), dtype=torch.float32, device=q.device)
    elif lse is not None:
        _guard("lse", lse, torch.float32, like=q, shape=(B, Hq))
    key = (B, Hq, Hkv, D, max_seq)
    need = _ws_bytes_cache.get(key)
    if need is None:
        need = _ws_bytes_cache[key] = decode_workspace_bytes(B, Hq, Hkv, D, max_seq)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    if workspace is None and need:
        workspace = _implicit_workspace(q.device, need, stream)
    rc = _lib.lib().rt_gqa_decode_bf16(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
        out.data_ptr() if out_dtype == torch.bfloat16 else None,
        out.data_ptr() if out_dtype == torch.float32 else None,
        lse.data_ptr() if lse is not None else None, B, Hq, Hkv, D, max_seq,
        kv_lens.data_ptr() if kv_lens is not None else None, 0 if kv_len is None else int(kv_len), kv_begin, kv_end,
        -1.0 if scale is None else float(scale), workspace.data_ptr() if workspace is not None else None,
        workspace.numel() if workspace is not None else 0, stream)
    if rc == _lib.RT_ERR_HEAD_COUNT:
        raise HeadCountMismatch(Hq, Hkv)
    if rc:
        _lib.check(rc, "rt_gqa_decode_bf16")
    return out, lse


def gqa_decode_record(q, k_cache, v_cache, kv_lens=None, kv_len: Optional[int] = None, kv_begin: int = 0,
                      kv_end: int = -1, scale: Optional[float] = None, record=None, workspace=None):
    """Decode one KV shard into a packed partial record f32 [B*Hq, D+1] (O | LSE) via
    ``rt_gqa_decode_record_bf16`` — the unit the ranks of a split-KV decode all-gather."""
    import torch
    B, Hq, Hkv, D, max_seq = _guard_decode_args(q, k_cache, v_cache, kv_lens, workspace)
    if record is None:
        record = torch.empty((B * Hq, D + 1), dtype=torch.float32, device=q.device)
    else:
        _guard("record", record, torch.float32, like=q, shape=(B * Hq, D + 1))
    need = decode_workspace_bytes(B, Hq, Hkv, D, max_seq)
    if workspace is None and need:
        workspace = _implicit_workspace(q.device, need)
    rc = _lib.lib().rt_gqa_decode_record_bf16(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), record.data_ptr(), B, Hq, Hkv, D, max_seq,
        kv_lens.data_ptr() if kv_lens is not None else None, 0 if kv_len is None else int(kv_len), kv_begin, kv_end,
        -1.0 if scale is None else float(scale), workspace.data_ptr() if workspace is not None else None,
        workspace.numel() if workspace is not None else 0, _stream_ptr())
    if rc == _lib.RT_ERR_HEAD_COUNT:
        raise HeadCountMismatch(Hq, Hkv)
    _lib.check(rc, "rt_gqa_decode_record_bf16")
    return record


def merge_records(records, out_dtype=None):
    """records f32 [R, rows, D+1] (CUDA) -> (out [rows, D], lse [rows]) via ``rt_attn_merge_records``."""
    import torch
    _guard("records", records, torch.float32)
    if records.dim() != 3:
        raise TypeError(f"records must be [R, rows, D+1], got {tuple(records.shape)}")
    R, rows, D1 = records.shape
    D = D1 - 1
    out_dtype = out_dtype or torch.bfloat16
    out = torch.empty((rows, D), dtype=out_dtype, device=records.device)
    lse = torch.empty((rows,), dtype=torch.float32, device=records.device)
    rc = _lib.lib().rt_attn_merge_records(records.data_ptr(), R, rows, D,
                                          out.data_ptr() if out_dtype == torch.bfloat16 else None,
                                          out.data_ptr() if out_dtype == torch.float32 else None, lse.data_ptr(),
                                          _stream_ptr())
    _lib.check(rc, "rt_attn_merge_records")
    return out, lse


def merge_partials(o_parts, lse_parts, out_dtype=None):
    """o_parts f32 [R,rows,D], lse_parts f32 [R,rows] (CUDA) -> (out [rows,D], lse [rows])."""
    import torch
    _guard("o_parts", o_parts, torch.float32)
    if o_parts.dim() != 3:
        raise TypeError(f"o_parts must be [R, rows, D], got {tuple(o_parts.shape)}")
    R, rows, D = o_parts.shape
    _guard("lse_parts", lse_parts, torch.float32, like=o_parts, shape=(R, rows))
    out_dtype = out_dtype or torch.bfloat16
    out = torch.empty((rows, D), dtype=out_dtype, device=o_parts.device)
    lse = torch.empty((rows,), dtype=torch.float32, device=o_parts.device)
    rc = _lib.lib().rt_attn_merge_partials(o_parts.data_ptr(), lse_parts.data_ptr(), R, rows, D,
                                           out.data_ptr() if out_dtype == torch.bfloat16 else None,
                                           out.data_ptr() if out_dtype == torch.float32 else None, lse.data_ptr(),
                                           _stream_ptr())
    _lib.check(rc, "rt_attn_merge_partials")
    return out, lse


def kv_append(k_cache, v_cache, k_in, v_in, pos=None, positions=None) -> None:
    """Batched kv_append via ``rt_kv_append_bf16``: k_in/v_in [B,Hkv,D] -> caches [B,Hkv,max_seq,D]."""
    import torch
    _guard("k_cache", k_cache, torch.bfloat16)
    if k_cache.dim() != 4:
        raise TypeError(f"k_cache must be [B, Hkv, max_seq, D], got {tuple(k_cache.shape)}")
    B, Hkv, max_seq, D = k_cache.shape
    _guard("v_cache", v_cache, torch.bfloat16, like=k_cache, shape=k_cache.shape)
    _guard("k_in", k_in, torch.bfloat16, like=k_cache, shape=(B, Hkv, D))
    _guard("v_in", v_in, torch.bfloat16, like=k_cache, shape=(B, Hkv, D))
    if positions is not None:
        _guard("positions", positions, torch.int32, like=k_cache, shape=(B,))
    rc = _lib.lib().rt_kv_append_bf16(k_cache.data_ptr(), v_cache.data_ptr(), k_in.data_ptr(), v_in.data_ptr(), B, Hkv,
                                      D, max_seq, 0 if pos is None else int(pos),
                                      positions.data_ptr() if positions is not None else None, _stream_ptr())
    _lib.check(rc, "rt_kv_append_bf16")


def rope_inv_freq(head_dim: int, base: float = 10000.0, device="cuda"):
    """theta^(-2k/D) for k in 0..D/2, the table the reference uploads once (cuda_backend.rs:221-226)."""
    import torch
    k = torch.arange(head_dim // 2, dtype=torch.float32)
    return (1.0 / torch.pow(torch.tensor(float(base), dtype=torch.float32), 2.0 * k / head_dim)).to(device)


def rope_kv_append(q, k_in, v_in, k_cache, v_cache, inv_freq, pos=None, positions=None, style: str = "half_split") -> None:
    """Rotary embedding of q (in place) and of the new K row + append of K, V at each sequence's position, one
    launch (``rt_rope_kv_append_bf16``).  q [B,Hq,D], k_in/v_in [B,Hkv,D], caches [B,Hkv,max_seq,D]."""
    import torch
    B, Hq, Hkv, D, max_seq = _guard_decode_args(q, k_cache, v_cache)
    _guard("k_in", k_in, torch.bfloat16, like=q, shape=(B, Hkv, D))
    _guard("v_in", v_in, torch.bfloat16, like=q, shape=(B, Hkv, D))
    _guard("inv_freq", inv_freq, torch.float32, like=q, shape=(D // 2,))
    if positions is not None:
        _guard("positions", positions, torch.int32, like=q, shape=(B,))
    rc = _lib.lib().rt_rope_kv_append_bf16(q.data_ptr(), k_in.data_ptr(), v_in.data_ptr(), k_cache.data_ptr(),
                                           v_cache.data_ptr(), inv_freq.data_ptr(), B, Hq, Hkv, D, max_seq,
                                           0 if pos is None else int(pos),
                                           positions.data_ptr() if positions is not None else None,
                                           {"half_split": _lib.RT_ROPE_HALF_SPLIT, "adjacent": _lib.RT_ROPE_ADJACENT}[style],
                                           _stream_ptr())
    _lib.check(rc, "rt_rope_kv_append_bf16")
