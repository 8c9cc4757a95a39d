"""Host-side mirror of the ``rustorch-attention`` public API on top of the C ABI.

Same names, argument meaning and error behaviour as the reference
(crates/rustorch-attention/src/lib.rs:27-33):

    AttentionShape, Mask, flash_forward, flash_forward_masked,
    AttentionError{BufferShapeMismatch, OutputShapeMismatch, ZeroDim, Mask(PaddingLengthMismatch)}

``flash_forward*`` take host f32 arrays exactly like the Rust functions take ``&[f32]`` slices
and run on the GPU through ``rt_flash_forward_f32_host``.  ``prefill_bf16`` is the device-resident
entry (torch CUDA tensors in, no host copies) that the benchmark measures.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_float, c_uint8
from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import _lib


# ---------------------------------------------------------------- errors (cpu_forward.rs:93-114, mask.rs:70-78)
class AttentionError(Exception):
    pass


class BufferShapeMismatch(AttentionError):
    def __init__(self, which: str, expected: int, got: int):
        self.which, self.expected, self.got = which, expected, got
        super().__init__(f"{which} buffer has {got} elements, expected {expected}")


class OutputShapeMismatch(AttentionError):
    def __init__(self, expected: int, got: int):
        self.expected, self.got = expected, got
        super().__init__(f"output buffer has {got} elements, expected {expected}")


class ZeroDim(AttentionError):
    def __init__(self):
        super().__init__("dim must be > 0")


class MaskError(AttentionError):
    pass


class PaddingLengthMismatch(MaskError):
    def __init__(self, expected: int, got: int):
        self.expected, self.got = expected, got
        super().__init__(f"mask error: padding mask len {got}, expected {expected}")


# ---------------------------------------------------------------- shape and mask
@dataclass
class AttentionShape:
    """cpu_forward.rs:49-89.  ``br``/``bc`` are kept for signature parity; they only change the
    summation order of the CPU reference and are ignored by the GPU kernels."""
    batch: int
    heads: int
    seq: int
    dim: int
    br: int = 64
    bc: int = 64

    @classmethod
    def new(cls, batch: int, heads: int, seq: int, dim: int) -> "AttentionShape":
        return cls(batch, heads, seq, dim)

    def buffer_len(self) -> int:
        return self.batch * self.heads * self.seq * self.dim


class Mask:
    """mask.rs:26-66: ``Mask.none()``, ``Mask.causal()``, ``Mask.padding(keep)``."""
    NONE, CAUSAL, PADDING = 0, 1, 2

    def __init__(self, kind: int, keep=None):
        self.kind = kind
        self.keep = None if keep is None else np.ascontiguousarray(keep, dtype=np.bool_)

    @classmethod
    def none(cls) -> "Mask":
        return cls(cls.NONE)

    @classmethod
    def causal(cls) -> "Mask":
        return cls(cls.CAUSAL)

    @classmethod
    def padding(cls, keep) -> "Mask":
        return cls(cls.PADDING, keep)

    def is_masked(self, qi: int, kj: int) -> bool:
        if self.kind == Mask.CAUSAL:
            return kj > qi
        if self.kind == Mask.PADDING:
            return kj < len(self.keep) and not bool(self.keep[kj])
        return False

    def validate(self, seq: int) -> None:
        if self.kind == Mask.PADDING and len(self.keep) != seq:
            raise PaddingLengthMismatch(seq, len(self.keep))


def _validate(shape: AttentionShape, q, k, v, out) -> None:  # cpu_forward.rs:142-169
    if shape.dim == 0:
        raise ZeroDim()
    expected = shape.buffer_len()
    for which, buf in (("q", q), ("k", k), ("v", v)):
        if buf.size != expected:
            raise BufferShapeMismatch(which, expected, buf.size)
    if out.size != expected:
        raise OutputShapeMismatch(expected, out.size)


def _f32(a, name):
    if not isinstance(a, np.ndarray) or a.dtype != np.float32 or not a.flags["C_CONTIGUOUS"]:
        raise TypeError(f"{name} must be a C-contiguous float32 numpy array")
    return a.ctypes.data_as(POINTER(c_float))


def flash_forward(shape: AttentionShape, q, k, v, out, precision: str = "f32") -> None:
    """cpu_forward.rs:175-183."""
    flash_forward_masked(shape, q, k, v, Mask.none(), out, precision)


def flash_forward_masked(shape: AttentionShape, q, k, v, mask: Mask, out, precision: str = "f32") -> None:
    """cpu_forward.rs:193-242 on the GPU.  ``precision``: "f32" = f32 CUDA-core kernel (parity with
    the f32 reference at 1e-4), "bf16" = inputs rounded to bf16, tcgen05 kernel (D in {64,128})."""
    _validate(shape, q, k, v, out)
    mask.validate(shape.seq)
    if shape.seq == 0:
        return
    keep_ptr, keep_len = None, 0
    if mask.kind == Mask.PADDING:
        keep_u8 = mask.keep.astype(np.uint8)
        keep_ptr, keep_len = keep_u8.ctypes.data_as(POINTER(c_uint8)), keep_u8.size
    prec = {"f32": _lib.RT_PRECISION_F32, "bf16": _lib.RT_PRECISION_BF16}[precision]
    rc = _lib.lib().rt_flash_forward_f32_host(_f32(q, "q"), q.size, _f32(k, "k"), k.size, _f32(v, "v"), v.size,
                                              _f32(out, "out"), out.size, shape.batch, shape.heads, shape.seq,
                                              shape.dim, mask.kind, keep_ptr, keep_len, prec)
    if rc == _lib.RT_ERR_ZERO_DIM:
        raise ZeroDim()
    if rc == _lib.RT_ERR_MASK_LEN:
        raise PaddingLengthMismatch(shape.seq, keep_len)
    _lib.check(rc, "rt_flash_forward_f32_host")


def flash_backward(shape: AttentionShape, q, k, v, do_, dq, dk, dv, causal: bool = False) -> None:
    """cpu_backward.rs:46-185 on the GPU: host numpy f32 slices in, (dq, dk, dv) overwritten.

    Validation order and errors follow the reference (:57-73): q, k, v, do -> BufferShapeMismatch,
    then dq/dk/dv -> OutputShapeMismatch(expected, largest length); seq == 0 is a no-op (:74-76).
    ``causal=True`` is an extension (the gradient of flash_forward_masked with Mask::Causal).
    """
    expected = shape.buffer_len()
    for which, buf in (("q", q), ("k", k), ("v", v), ("do", do_)):
        if buf.size != expected:
            raise BufferShapeMismatch(which, expected, buf.size)
    if dq.size != expected or dk.size != expected or dv.size != expected:
        raise OutputShapeMismatch(expected, max(dq.size, dk.size, dv.size))
    if shape.seq == 0 or expected == 0:
        return
    rc = _lib.lib().rt_flash_backward_f32_host(_f32(q, "q"), q.size, _f32(k, "k"), k.size, _f32(v, "v"), v.size,
                                               _f32(do_, "do"), do_.size, _f32(dq, "dq"), dq.size, _f32(dk, "dk"),
                                               dk.size, _f32(dv, "dv"), dv.size, shape.batch, shape.heads, shape.seq,
                                               shape.dim, Mask.CAUSAL if causal else Mask.NONE)
    _lib.check(rc, "rt_flash_backward_f32_host")


# ---------------------------------------------------------------- device-resident entry (torch tensors)
def _stream_ptr():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dense_view(t) -> bool:
    """True if t is a permutation of a dense tensor (every element addressed once, no gaps)."""
    if t.numel() == 0:
        return True
    expect = 1
    for size, stride in sorted(zip(t.shape, t.stride()), key=lambda x: x[1]):
        if size == 1:
            continue
        if stride != expect:
            return False
        expect *= size
    return True


def mha_prefill_bf16(q, k, v, n_heads: int, n_kv_heads: Optional[int] = None, causal: bool = False, **kw):
    """Attention on activations in the layout the reference's modules keep them in: q [B,T,Hq*hd],
    k, v [B,S,Hkv*hd] bf16 CUDA tensors (crates/rustorch-nn/src/attention.rs:468-485 transposes them
    to [B,H,T,hd] before the kernel and :499-543 transposes the result back; gqa.rs:151-168 also
    repeats the KV heads).  The transposes and the repeat are folded into the TMA descriptors:
    returns (out [B,T,Hq*hd], lse [B,Hq,T]) without any full-tensor copy.
    """
    n_kv_heads = n_heads if n_kv_heads is None else n_kv_heads
    B, T, E = q.shape
    S = k.shape[1]
    hd = E // n_heads
    if hd * n_heads != E or k.shape[2] != n_kv_heads * hd or v.shape != k.shape:
        raise BufferShapeMismatch("q/k/v", E, k.shape[2])
    qv = q.view(B, T, n_heads, hd).permute(0, 2, 1, 3)
    kv = k.view(B, S, n_kv_heads, hd).permute(0, 2, 1, 3)
    vv = v.view(B, S, n_kv_heads, hd).permute(0, 2, 1, 3)
    out, lse = prefill_bf16(qv, kv, vv, causal=causal, **kw)
    return out.permute(0, 2, 1, 3).reshape(B, T, E), lse


def prefill_bf16(q, k, v, causal: bool = False, kv_lens=None, key_keep=None, scale: Optional[float] = None,
                 out=None, lse=None, return_lse: bool = True, q_offsets=None):
    """Flash-attention forward on bf16 CUDA tensors (D in {64,128}), tcgen05 kernel.

    q [B,Hq,Nq,D]; k, v [B,Hkv,Nkv,D] with Hq a multiple of Hkv and Nkv >= 1 (self-attention: same
    shape as q).  kv_lens: optional int32 CUDA [B] visible keys; q_offsets: optional int32 CUDA [B],
    causal position of query row 0 (a prompt chunk against a cache); key_keep: optional uint8/bool
    CUDA [Nkv] or [B,Nkv].  Returns (out bf16 [B,Hq,Nq,D], lse f32 [B,Hq,Nq] or None).  Enqueues on
    the current stream.  Calls ``rt_attn_prefill_bf16`` for self-attention shapes,
    ``rt_attn_prefill_gqa_bf16`` for other contiguous shapes, and ``rt_attn_prefill_strided_bf16``
    when any of q, k, v, out is a strided view whose last dim is contiguous (e.g. a
    ``[B,T,H,hd]`` activation permuted to ``[B,H,T,hd]``): no transpose copy is made.
    """
    import torch
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not (t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 4):
            raise TypeError(f"{name} must be a 4-D bfloat16 CUDA tensor")
    B, H, N, D = q.shape
    if v.shape != k.shape or k.shape[0] != B or k.shape[3] != D:
        raise BufferShapeMismatch("k/v", k.numel(), v.numel())
    Hkv, Nkv = k.shape[1], k.shape[2]
    if out is None:
        # the output takes q's layout, so a permuted activation view gets a result in the same layout
        out = torch.empty_strided(q.shape, q.stride(), dtype=q.dtype, device=q.device) if _dense_view(q) \
            else torch.empty_like(q, memory_format=torch.contiguous_format)
    strided = not all(t.is_contiguous() for t in (q, k, v, out))
    if strided:
        for name, t in (("q", q), ("k", k), ("v", v), ("out", out)):
            if t.numel() and t.stride(3) != 1:
                raise TypeError(f"{name}: the head dim must be contiguous")
    if lse is None and return_lse:
        lse = torch.empty((B, H, N), dtype=torch.float32, device=q.device)
    keep_ptr, keep_stride = None, 0
    if key_keep is not None:
        key_keep = key_keep.to(torch.uint8).contiguous()
        if key_keep.shape[-1] != Nkv:
            raise PaddingLengthMismatch(Nkv, key_keep.shape[-1])
        keep_stride = Nkv if key_keep.dim() == 2 else 0
        keep_ptr = key_keep.data_ptr()
    for name, t in (("kv_lens", kv_lens), ("q_offsets", q_offsets)):
        if t is not None and not (t.is_cuda and t.dtype == torch.int32 and t.numel() == B):
            raise TypeError(f"{name} must be an int32 CUDA tensor of B elements")
    lens_ptr = kv_lens.data_ptr() if kv_lens is not None else None
    flags = _lib.RT_MASK_CAUSAL if causal else _lib.RT_MASK_NONE
    sc = -1.0 if scale is None else float(scale)
    lse_ptr = lse.data_ptr() if lse is not None else None
    if strided:
        import ctypes
        arrs = [(ctypes.c_int64 * 3)(*t.stride()[:3]) for t in (q, k, v, out)]
        rc = _lib.lib().rt_attn_prefill_strided_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse_ptr,
                                                     B, H, Hkv, N, Nkv, D, arrs[0], arrs[1], arrs[2], arrs[3], flags,
                                                     lens_ptr, q_offsets.data_ptr() if q_offsets is not None else None,
                                                     keep_ptr, keep_stride, sc, _stream_ptr())
        where = "rt_attn_prefill_strided_bf16"
    elif Hkv == H and Nkv == N and q_offsets is None:
        rc = _lib.lib().rt_attn_prefill_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse_ptr, B, H,
                                             N, D, flags, lens_ptr, keep_ptr, keep_stride, sc, _stream_ptr())
        where = "rt_attn_prefill_bf16"
    else:
        rc = _lib.lib().rt_attn_prefill_gqa_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse_ptr, B,
                                                 H, Hkv, N, Nkv, D, flags, lens_ptr,
                                                 q_offsets.data_ptr() if q_offsets is not None else None, keep_ptr,
                                                 keep_stride, sc, _stream_ptr())
        where = "rt_attn_prefill_gqa_bf16"
    if rc == _lib.RT_ERR_ZERO_DIM:
        raise ZeroDim()
    _lib.check(rc, where)
    return out, lse


def prefill_f32(q, k, v, causal: bool = False, kv_lens=None, key_keep=None, scale: Optional[float] = None,
                q_offsets=None):
    """f32 CUDA-core forward on f32 CUDA tensors q [B,Hq,Nq,D], k/v [B,Hkv,Nkv,D] via ``rt_attn_prefill_f32``."""
    import torch
    B, Hq, Nq, D = q.shape
    _, Hkv, Nkv, _ = k.shape
    out = torch.empty_like(q)
    lse = torch.empty((B, Hq, Nq), dtype=torch.float32, device=q.device)
    keep_ptr, keep_stride = None, 0
    if key_keep is not None:
        key_keep = key_keep.to(torch.uint8).contiguous()
        keep_stride = Nkv if key_keep.dim() == 2 else 0
        keep_ptr = key_keep.data_ptr()
    rc = _lib.lib().rt_attn_prefill_f32(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B,
                                        Hq, Hkv, Nq, Nkv, D, _lib.RT_MASK_CAUSAL if causal else _lib.RT_MASK_NONE,
                                        kv_lens.data_ptr() if kv_lens is not None else None,
                                        q_offsets.data_ptr() if q_offsets is not None else None, keep_ptr, keep_stride,
                                        -1.0 if scale is None else float(scale), _stream_ptr())
    if rc == _lib.RT_ERR_ZERO_DIM:
        raise ZeroDim()
    _lib.check(rc, "rt_attn_prefill_f32")
    return out, lse


def backward_f32(q, k, v, out, d_out, lse, causal: bool = False, scale: Optional[float] = None):
    """(dq, dk, dv) on f32 CUDA tensors [B,H,N,D] via ``rt_attn_backward_f32``; ``out`` and ``lse`` are
    the results of ``prefill_f32`` on the same q, k, v, mask and scale."""
    import torch
    B, H, N, D = q.shape
    for name, t in (("q", q), ("k", k), ("v", v), ("out", out), ("d_out", d_out)):
        if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape) == (B, H, N, D)):
            raise TypeError(f"{name} must be a contiguous float32 CUDA tensor of shape {(B, H, N, D)}")
    if not (lse.is_cuda and lse.dtype == torch.float32 and lse.is_contiguous() and tuple(lse.shape) == (B, H, N)):
        raise TypeError("lse must be a contiguous float32 CUDA tensor [B,H,N]")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    need = _lib.lib().rt_attn_backward_workspace_bytes(B, H, N)
    ws = torch.empty((max(need, 4) // 4,), dtype=torch.float32, device=q.device)
    rc = _lib.lib().rt_attn_backward_f32(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), d_out.data_ptr(),
                                         lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, H, N, D,
                                         _lib.RT_MASK_CAUSAL if causal else _lib.RT_MASK_NONE,
                                         -1.0 if scale is None else float(scale), ws.data_ptr(), need, _stream_ptr())
    if rc == _lib.RT_ERR_ZERO_DIM:
        raise ZeroDim()
    _lib.check(rc, "rt_attn_backward_f32")
    return dq, dk, dv


def backward_bf16(q, k, v, out, d_out, lse, causal: bool = False, scale: Optional[float] = None):
    """(dq, dk, dv) f32 from bf16 CUDA tensors [B,H,N,D] (D in {64,128}) via ``rt_attn_backward_bf16``;
    ``out`` and ``lse`` are the results of ``prefill_bf16`` on the same q, k, v, mask and scale."""
    import torch
    B, H, N, D = q.shape
    for name, t in (("q", q), ("k", k), ("v", v), ("out", out), ("d_out", d_out)):
        if not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous() and tuple(t.shape) == (B, H, N, D)):
            raise TypeError(f"{name} must be a contiguous bfloat16 CUDA tensor of shape {(B, H, N, D)}")
    if not (lse.is_cuda and lse.dtype == torch.float32 and lse.is_contiguous() and tuple(lse.shape) == (B, H, N)):
        raise TypeError("lse must be a contiguous float32 CUDA tensor [B,H,N]")
    dq, dk, dv = (torch.empty((B, H, N, D), dtype=torch.float32, device=q.device) for _ in range(3))
    need = _lib.lib().rt_attn_backward_workspace_bytes(B, H, N)
    ws = torch.empty((max(need, 4) // 4,), dtype=torch.float32, device=q.device)
    rc = _lib.lib().rt_attn_backward_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), d_out.data_ptr(),
                                          lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, H, N, D,
                                          _lib.RT_MASK_CAUSAL if causal else _lib.RT_MASK_NONE,
                                          -1.0 if scale is None else float(scale), ws.data_ptr(), need, _stream_ptr())
    if rc == _lib.RT_ERR_ZERO_DIM:
        raise ZeroDim()
    _lib.check(rc, "rt_attn_backward_bf16")
    return dq, dk, dv
