//! FFI declarations of `librustorch_attn` (the sm_100a attention library), one per symbol of
//! `include/rustorch_attn.h`.  Goes to `crates/rustorch-cuda/src/attn_ffi.rs` of the reference; the precedent
//! there is the hand-declared `extern "C"` block for cuSPARSELt (`crates/rustorch-cuda/src/cusparse_lt.rs:190`).
//! Not compiled in this repository (no Rust toolchain on the build machines); `tests/test_abi.py` checks the
//! names and argument counts below against the C header and the ctypes prototypes.
#![allow(clippy::too_many_arguments)]
use std::os::raw::{c_char, c_int, c_void};
extern "C" {
    pub fn rt_attn_version() -> c_int;
    pub fn rt_attn_error_string(status: c_int) -> *const c_char;
    pub fn rt_attn_device_status(status: *mut c_int) -> c_int;
    pub fn rt_attn_prefill_bf16(q: *const c_void, k: *const c_void, v: *const c_void, out: *mut c_void,
        lse: *mut f32, batch: i64, heads: i64, seq: i64, dim: c_int, mask_flags: c_int,
        kv_lens: *const i32, key_keep: *const u8, keep_batch_stride: i64, scale: f32,
        stream: *mut c_void) -> c_int;
    pub fn rt_attn_prefill_gqa_bf16(q: *const c_void, k: *const c_void, v: *const c_void, out: *mut c_void,
        lse: *mut f32, batch: i64, heads_q: i64, heads_kv: i64, seq_q: i64, seq_kv: i64, dim: c_int,
        mask_flags: c_int, kv_lens: *const i32, q_offsets: *const i32, key_keep: *const u8,
        keep_batch_stride: i64, scale: f32, stream: *mut c_void) -> c_int;
    pub fn rt_attn_prefill_strided_bf16(q: *const c_void, k: *const c_void, v: *const c_void, out: *mut c_void,
        lse: *mut f32, batch: i64, heads_q: i64, heads_kv: i64, seq_q: i64, seq_kv: i64, dim: c_int,
        q_strides: *const i64, k_strides: *const i64, v_strides: *const i64, out_strides: *const i64,
        mask_flags: c_int, kv_lens: *const i32, q_offsets: *const i32, key_keep: *const u8,
        keep_batch_stride: i64, scale: f32, stream: *mut c_void) -> c_int;
    pub fn rt_attn_backward_workspace_bytes(batch: i64, heads: i64, seq: i64) -> usize;
    pub fn rt_attn_backward_f32(q: *const f32, k: *const f32, v: *const f32, out: *const f32, d_out: *const f32,
        lse: *const f32, dq: *mut f32, dk: *mut f32, dv: *mut f32, batch: i64, heads: i64, seq: i64,
        dim: c_int, mask_flags: c_int, scale: f32, workspace: *mut c_void, workspace_bytes: usize,
        stream: *mut c_void) -> c_int;
    pub fn rt_attn_backward_bf16(q: *const c_void, k: *const c_void, v: *const c_void, out: *const c_void,
        d_out: *const c_void, lse: *const f32, dq: *mut f32, dk: *mut f32, dv: *mut f32, batch: i64, heads: i64,
        seq: i64, dim: c_int, mask_flags: c_int, scale: f32, workspace: *mut c_void, workspace_bytes: usize,
        stream: *mut c_void) -> c_int;
    pub fn rt_splitkv_push_record(record: *const f32, peer_slots: *const *mut c_void,
        peer_flags: *const *mut c_void, world: c_int, rows: i64, dim: c_int, epoch: u32,
        stream: *mut c_void) -> c_int;
    pub fn rt_gqa_decode_record_push_bf16(q: *const c_void, k_cache: *const c_void, v_cache: *const c_void,
        record: *mut f32, peer_slots: *const *mut c_void, peer_flags: *const *mut c_void, world: c_int, epoch: u32,
        done_counter: *mut c_int, batch: i64, n_heads: i64, n_kv_heads: i64, head_dim: c_int, max_seq: i64,
        kv_lens: *const i32, kv_len_uniform: i64, kv_begin: i64, kv_end: i64, scale: f32, workspace: *mut c_void,
        workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn rt_attn_merge_records_after(records: *const f32, flags: *const u32, epoch: u32, wait_clocks: i64,
        n_parts: i64, rows: i64, dim: c_int, out_bf16: *mut c_void, out_f32: *mut f32, lse: *mut f32,
        stream: *mut c_void) -> c_int;
    pub fn rt_flash_backward_f32_host(q: *const f32, q_len: usize, k: *const f32, k_len: usize, v: *const f32,
        v_len: usize, d_out: *const f32, d_out_len: usize, dq: *mut f32, dq_len: usize, dk: *mut f32,
        dk_len: usize, dv: *mut f32, dv_len: usize, batch: i64, heads: i64, seq: i64, dim: i64,
        mask_kind: c_int) -> c_int;
    pub fn rt_attn_prefill_f32(q: *const f32, k: *const f32, v: *const f32, out: *mut f32, lse: *mut f32,
        batch: i64, heads_q: i64, heads_kv: i64, seq_q: i64, seq_kv: i64, dim: c_int, mask_flags: c_int,
        kv_lens: *const i32, q_offsets: *const i32, key_keep: *const u8, keep_batch_stride: i64, scale: f32,
        stream: *mut c_void) -> c_int;
    pub fn rt_gqa_decode_online_bf16_static(q: *const c_void, k_cache: *const c_void, v_cache: *const c_void,
        out: *mut c_void, n_heads: c_int, n_kv: c_int, kv_len: c_int, head_dim: c_int, max_seq: c_int,
        stream: *mut c_void) -> c_int;
    pub fn rt_flash_forward_f32_host(q: *const f32, q_len: usize, k: *const f32, k_len: usize,
        v: *const f32, v_len: usize, out: *mut f32, out_len: usize, batch: i64, heads: i64, seq: i64,
        dim: i64, mask_kind: c_int, keep: *const u8, keep_len: usize, precision: c_int) -> c_int;
    pub fn rt_attn_prefill_bf16_host(q: *const c_void, k: *const c_void, v: *const c_void,
        out: *mut c_void, lse: *mut f32, batch: i64, heads: i64, seq: i64, dim: c_int,
        mask_flags: c_int, kv_lens: *const i32, scale: f32) -> c_int;
    pub fn rt_gqa_decode_workspace_bytes(batch: i64, n_heads: i64, n_kv_heads: i64, head_dim: c_int,
        max_seq: i64) -> usize;
    pub fn rt_gqa_decode_bf16(q: *const c_void, k_cache: *const c_void, v_cache: *const c_void,
        out_bf16: *mut c_void, out_f32: *mut f32, lse: *mut f32, batch: i64, n_heads: i64,
        n_kv_heads: i64, head_dim: c_int, max_seq: i64, kv_lens: *const i32, kv_len_uniform: i64,
        kv_begin: i64, kv_end: i64, scale: f32, workspace: *mut c_void, workspace_bytes: usize,
        stream: *mut c_void) -> c_int;
    pub fn rt_gqa_decode_online_bf16(q: *const c_void, k_cache: *const c_void, v_cache: *const c_void,
        out: *mut c_void, n_heads: c_int, n_kv: c_int, kv_len: c_int, head_dim: c_int, max_seq: c_int,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn rt_gqa_decode_record_bf16(q: *const c_void, k_cache: *const c_void, v_cache: *const c_void,
        record: *mut f32, batch: i64, n_heads: i64, n_kv_heads: i64, head_dim: c_int, max_seq: i64,
        kv_lens: *const i32, kv_len_uniform: i64, kv_begin: i64, kv_end: i64, scale: f32,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn rt_attn_merge_records(records: *const f32, n_parts: i64, rows: i64, dim: c_int,
        out_bf16: *mut c_void, out_f32: *mut f32, lse: *mut f32, stream: *mut c_void) -> c_int;
    pub fn rt_attn_merge_partials(o_parts: *const f32, lse_parts: *const f32, n_parts: i64, rows: i64,
        dim: c_int, out_bf16: *mut c_void, out_f32: *mut f32, lse: *mut f32, stream: *mut c_void) -> c_int;
    pub fn rt_gqa_forward_f32_host(q: *const f32, q_len: usize, k: *const f32, k_len: usize,
        v: *const f32, v_len: usize, out: *mut f32, out_len: usize, batch: i64, n_heads: i64,
        n_kv_heads: i64, seq_q: i64, seq_kv: i64, head_dim: i64) -> c_int;
    pub fn rt_rope_kv_append_bf16(q: *mut c_void, k_in: *const c_void, v_in: *const c_void, k_cache: *mut c_void,
        v_cache: *mut c_void, inv_freq: *const f32, batch: i64, n_heads: c_int, n_kv: c_int, head_dim: c_int,
        max_seq: i64, pos: i64, positions: *const i32, rope_style: c_int, stream: *mut c_void) -> c_int;
    pub fn rt_kv_append_bf16(k_cache: *mut c_void, v_cache: *mut c_void, k_in: *const c_void,
        v_in: *const c_void, batch: i64, n_kv: c_int, head_dim: c_int, max_seq: i64, pos: i64,
        positions: *const i32, stream: *mut c_void) -> c_int;
    pub fn rt_gqa_decode_exchange_bf16(q: *const c_void, k_cache: *const c_void, v_cache: *const c_void,
        out_bf16: *mut c_void, out_f32: *mut f32, lse: *mut f32, peer_slots: *const *mut c_void,
        peer_flags: *const *mut c_void, local_slots: *const f32, local_flags: *const u32, world: c_int, rank: c_int,
        epoch: u32, wait_clocks: i64, do_wait: c_int, batch: i64, n_heads: i64, n_kv_heads: i64, head_dim: c_int,
        max_seq: i64, kv_lens: *const i32, kv_len_uniform: i64, kv_begin: i64, kv_end: i64, scale: f32,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn rt_attn_merge_records_after_rows(records: *const f32, row_flags: *const u32, epoch: u32, wait_clocks: i64,
        n_parts: i64, rows: i64, dim: c_int, out_bf16: *mut c_void, out_f32: *mut f32, lse: *mut f32,
        stream: *mut c_void) -> c_int;
    pub fn rt_gqa_decode_exchange_ll_bf16(q: *const c_void, k_cache: *const c_void, v_cache: *const c_void,
        out_bf16: *mut c_void, out_f32: *mut f32, lse: *mut f32, peer_words: *const *mut c_void,
        local_words: *const c_void, scratch_record: *mut f32, world: c_int, rank: c_int, epoch: u32, wait_clocks: i64,
        do_wait: c_int, batch: i64, n_heads: i64, n_kv_heads: i64, head_dim: c_int, max_seq: i64,
        kv_lens: *const i32, kv_len_uniform: i64, kv_begin: i64, kv_end: i64, scale: f32, workspace: *mut c_void,
        workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn rt_attn_merge_ll_rows(local_words: *const c_void, epoch: u32, wait_clocks: i64, world: c_int, rows: i64,
        dim: c_int, out_bf16: *mut c_void, out_f32: *mut f32, lse: *mut f32, stream: *mut c_void) -> c_int;
    pub fn rt_convert_f32_to_bf16(src: *const f32, dst: *mut c_void, n: i64, stream: *mut c_void) -> c_int;
    pub fn rt_convert_bf16_to_f32(src: *const c_void, dst: *mut f32, n: i64, stream: *mut c_void) -> c_int;
    pub fn rt_debug_tc_selftest(a: *const c_void, b: *const c_void, v: *const c_void, s_out: *mut f32,
        o_out: *mut f32, dim: c_int, stream: *mut c_void) -> c_int;
}
