"""rustorch_b200 — B200 (sm_100a) attention kernels behind the reference's attention API.

The product is ``librustorch_attn.so`` (hand-written CUDA, C ABI in ``include/rustorch_attn.h``).
This package is the thin host-side mirror of the reference's Rust entry points for that path:

    rustorch_b200.attention : AttentionShape, Mask, flash_forward, flash_forward_masked, flash_backward,
                              prefill_bf16, mha_prefill_bf16, prefill_f32, backward_f32
    rustorch_b200.gqa       : gqa_forward_f32, LlmKernels.gqa_decode_online_bf16, gqa_decode, merge_partials
"""
from .attention import (AttentionError, AttentionShape, BufferShapeMismatch, Mask, MaskError, OutputShapeMismatch,
                        PaddingLengthMismatch, ZeroDim, backward_bf16, backward_f32, flash_backward, flash_forward,
                        flash_forward_masked, mha_prefill_bf16, prefill_bf16, prefill_f32)
from .gqa import (GQAError, HeadCountMismatch, LlmKernels, WrongInputLen, decode_workspace_bytes, gqa_decode,
                  gqa_decode_online_bf16_static, gqa_decode_record, gqa_forward_f32, kv_append, merge_partials,
                  merge_records, rope_inv_freq, rope_kv_append)

__all__ = [
    "AttentionError", "AttentionShape", "BufferShapeMismatch", "Mask", "MaskError", "OutputShapeMismatch",
    "PaddingLengthMismatch", "ZeroDim", "flash_forward", "flash_forward_masked", "flash_backward", "backward_f32", "backward_bf16",
    "mha_prefill_bf16", "prefill_bf16", "prefill_f32",
    "GQAError", "HeadCountMismatch", "LlmKernels", "WrongInputLen", "decode_workspace_bytes", "gqa_decode",
    "gqa_decode_online_bf16_static", "gqa_decode_record", "gqa_forward_f32", "kv_append", "merge_partials",
    "merge_records", "rope_inv_freq", "rope_kv_append",
]
