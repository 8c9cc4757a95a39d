//! Safe wrappers with the reference's own signatures over `attn_ffi`.  Each function replaces the body of the
//! reference function it is named after and keeps its error behaviour.  Not compiled in this repository.
//!
//!   flash_forward / flash_forward_masked   crates/rustorch-attention/src/cpu_forward.rs:175-242
//!   flash_backward                         crates/rustorch-attention/src/cpu_backward.rs:46-55
//!   gqa_forward_f32                        crates/rustorch-nn/src/gqa.rs:94-105
//!   LlmKernels::gqa_decode_online_bf16     crates/rustorch-cuda/src/llm_kernels.rs:915-958 (naive twin :1000-1042)
//!   LlmKernels::kv_append_bf16             crates/rustorch-cuda/src/llm_kernels.rs:872-911
use std::os::raw::c_int;
use std::sync::Arc;

use crate::attn_ffi::*;

/// 0 = f32 CUDA-core kernel (the reference's own 1e-4 gate), 1 = bf16 tcgen05 kernel (D in {64, 128}).
pub const PRECISION_F32: c_int = 0;
pub const PRECISION_BF16: c_int = 1;

fn first_mismatch(shape: &AttentionShape, q: &[f32], k: &[f32], v: &[f32]) -> AttentionError {
    let expected = shape.buffer_len();
    for (which, buf) in [("q", q), ("k", k), ("v", v)] {
        if buf.len() != expected {
            return AttentionError::BufferShapeMismatch { which, expected, got: buf.len() };
        }
    }
    unreachable!("the library reported a buffer mismatch that the lengths do not show")
}

pub fn flash_forward(shape: &AttentionShape, q: &[f32], k: &[f32], v: &[f32], out: &mut [f32])
    -> Result<(), AttentionError> {
    flash_forward_masked(shape, q, k, v, &Mask::None, out)
}

/// `AttentionShape.br` / `bc` stay in the struct and are ignored: they only reorder the CPU summation.
pub fn flash_forward_masked(shape: &AttentionShape, q: &[f32], k: &[f32], v: &[f32], mask: &Mask<'_>,
                            out: &mut [f32]) -> Result<(), AttentionError> {
    let (kind, keep): (c_int, Vec<u8>) = match mask {
        Mask::None => (0, vec![]),
        Mask::Causal => (1, vec![]),
        Mask::Padding(p) => (2, p.iter().map(|&b| b as u8).collect()),
    };
    let rc = unsafe {
        rt_flash_forward_f32_host(q.as_ptr(), q.len(), k.as_ptr(), k.len(), v.as_ptr(), v.len(), out.as_mut_ptr(),
                                  out.len(), shape.batch as i64, shape.heads as i64, shape.seq as i64,
                                  shape.dim as i64, kind, keep.as_ptr(), keep.len(), attention_precision())
    };
    match rc {
        0 => Ok(()),
        -1 => Err(AttentionError::ZeroDim),
        -2 => Err(first_mismatch(shape, q, k, v)),
        -3 => Err(AttentionError::OutputShapeMismatch { expected: shape.buffer_len(), got: out.len() }),
        -4 => Err(AttentionError::Mask(MaskError::PaddingLengthMismatch { expected: shape.seq, got: keep.len() })),
        e => panic!("rt_flash_forward_f32_host: {e}"), // a CUDA failure: the library has no CPU fallback
    }
}

/// `RUSTORCH_ATTN_PRECISION=bf16` selects the tensor-core kernel (inputs rounded to bf16); the default keeps
/// the reference's f32 numerics.
fn attention_precision() -> c_int {
    match std::env::var("RUSTORCH_ATTN_PRECISION").as_deref() {
        Ok("bf16") => PRECISION_BF16,
        _ => PRECISION_F32,
    }
}

pub fn flash_backward(shape: &AttentionShape, q: &[f32], k: &[f32], v: &[f32], d_out: &[f32], dq: &mut [f32],
                      dk: &mut [f32], dv: &mut [f32]) -> Result<(), AttentionError> {
    let rc = unsafe {
        rt_flash_backward_f32_host(q.as_ptr(), q.len(), k.as_ptr(), k.len(), v.as_ptr(), v.len(), d_out.as_ptr(),
                                   d_out.len(), dq.as_mut_ptr(), dq.len(), dk.as_mut_ptr(), dk.len(),
                                   dv.as_mut_ptr(), dv.len(), shape.batch as i64, shape.heads as i64,
                                   shape.seq as i64, shape.dim as i64, 0)
    };
    let expected = shape.buffer_len();
    match rc {
        0 => Ok(()),
        -2 => {
            for (which, buf) in [("q", q), ("k", k), ("v", v), ("do", d_out)] {
                if buf.len() != expected {
                    return Err(AttentionError::BufferShapeMismatch { which, expected, got: buf.len() });
                }
            }
            unreachable!()
        }
        -3 => Err(AttentionError::OutputShapeMismatch { expected, got: dq.len().max(dk.len()).max(dv.len()) }),
        e => panic!("rt_flash_backward_f32_host: {e}"),
    }
}

pub fn gqa_forward_f32(q: &[f32], k: &[f32], v: &[f32], out: &mut [f32], batch: usize, n_heads: usize,
                       n_kv_heads: usize, seq_q: usize, seq_kv: usize, head_dim: usize) -> Result<(), GQAError> {
    let rc = unsafe {
        rt_gqa_forward_f32_host(q.as_ptr(), q.len(), k.as_ptr(), k.len(), v.as_ptr(), v.len(), out.as_mut_ptr(),
                                out.len(), batch as i64, n_heads as i64, n_kv_heads as i64, seq_q as i64,
                                seq_kv as i64, head_dim as i64)
    };
    match rc {
        0 => Ok(()),
        -5 => Err(GQAError::HeadCountMismatch { n_heads, n_kv_heads }),
        -6 => {
            let qn = batch * n_heads * seq_q * head_dim;
            let kn = batch * n_kv_heads * seq_kv * head_dim;
            for (which, got, expected) in [("q", q.len(), qn), ("k", k.len(), kn), ("v", v.len(), kn), ("out", out.len(), qn)] {
                if got != expected {
                    return Err(GQAError::WrongInputLen { which, expected, got });
                }
            }
            unreachable!()
        }
        e => panic!("rt_gqa_forward_f32_host: {e}"),
    }
}

impl LlmKernels {
    /// Same ten arguments as the reference method; the split-KV scratch is a `CudaSlice<u8>` cached in
    /// `LlmKernels` and grown on demand (`attn_scratch`).
    #[allow(clippy::too_many_arguments)]
    pub unsafe fn gqa_decode_online_bf16(&self, stream: &Arc<CudaStream>, q: u64, k_cache: u64, v_cache: u64,
                                         out: u64, n_heads: i32, n_kv: i32, kv_len: i32, head_dim: i32,
                                         max_seq: i32) -> Result<(), CudaError> {
        let need = rt_gqa_decode_workspace_bytes(1, n_heads as i64, n_kv as i64, head_dim, max_seq as i64);
        let ws = self.attn_scratch(stream, need)?;
        let rc = rt_gqa_decode_online_bf16(q as _, k_cache as _, v_cache as _, out as _, n_heads, n_kv, kv_len,
                                           head_dim, max_seq, ws.ptr as _, need, stream.cu_stream() as _);
        match rc {
            0 => Ok(()),
            -7 => Err(CudaError::Unsupported { msg: "gqa_decode_online_bf16: shape".into() }),
            code => Err(CudaError::Driver { code, location: "gqa_decode_online_bf16::launch" }),
        }
    }

    /// The three-pass twin of the reference gives the same result; it binds to the same kernel.
    #[allow(clippy::too_many_arguments)]
    pub unsafe fn gqa_decode_naive_bf16(&self, stream: &Arc<CudaStream>, q: u64, k_cache: u64, v_cache: u64, out: u64,
                                        n_heads: i32, n_kv: i32, kv_len: i32, head_dim: i32, max_seq: i32)
        -> Result<(), CudaError> {
        self.gqa_decode_online_bf16(stream, q, k_cache, v_cache, out, n_heads, n_kv, kv_len, head_dim, max_seq)
    }

    /// For a caller that may not allocate once its pools are set up: the library's built-in 8 MiB scratch.
    /// Make the first call before any stream capture; calls that overlap on one GPU race on that array.
    #[allow(clippy::too_many_arguments)]
    pub unsafe fn gqa_decode_online_bf16_no_alloc(&self, stream: &Arc<CudaStream>, q: u64, k_cache: u64, v_cache: u64,
                                                  out: u64, n_heads: i32, n_kv: i32, kv_len: i32, head_dim: i32,
                                                  max_seq: i32) -> Result<(), CudaError> {
        match rt_gqa_decode_online_bf16_static(q as _, k_cache as _, v_cache as _, out as _, n_heads, n_kv, kv_len,
                                               head_dim, max_seq, stream.cu_stream() as _) {
            0 => Ok(()),
            -13 => Err(CudaError::Unsupported { msg: "gqa_decode_online_bf16: needs more than the built-in scratch".into() }),
            code => Err(CudaError::Driver { code, location: "gqa_decode_online_bf16_static::launch" }),
        }
    }

    #[allow(clippy::too_many_arguments)]
    pub unsafe fn kv_append_bf16(&self, stream: &Arc<CudaStream>, k_cache: u64, v_cache: u64, k_in: u64, v_in: u64,
                                 pos: i32, n_kv: i32, head_dim: i32, max_seq: i32) -> Result<(), CudaError> {
        match rt_kv_append_bf16(k_cache as _, v_cache as _, k_in as _, v_in as _, 1, n_kv, head_dim, max_seq as i64,
                                pos as i64, std::ptr::null(), stream.cu_stream() as _) {
            0 => Ok(()),
            code => Err(CudaError::Driver { code, location: "kv_append_bf16::launch" }),
        }
    }
}
