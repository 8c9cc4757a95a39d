/*
 * rustorch_attn.h — C ABI of the B200 (sm_100a) attention library.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, and returns an
 * `int` status: 0 = success, > 0 = a `cudaError_t` value (maps to the reference's
 * `CudaError::Driver{code, location}`, crates/rustorch-cuda/src/error.rs:8-62),
 * < 0 = a validation error (RT_ERR_* below) raised BEFORE any device work is queued.
 *
 * Conventions
 *   - "device" pointers are CUDA device addresses (the reference passes them as `u64`
 *     obtained from `CudaSlice::device_ptr`, crates/rustorch-llm/src/cuda_backend.rs:969-972).
 *   - bf16 buffers are raw 16-bit words (`__nv_bfloat16`), produced with round-to-nearest-even
 *     (crates/rustorch-amp/src/dtypes.rs:10-24).
 *   - `stream` is a `cudaStream_t` passed as `void*`; NULL = the legacy default stream.
 *     Device entry points only enqueue work and return; the caller synchronises, like
 *     `LlamaModelCuda::decode_step` does (crates/rustorch-llm/src/cuda_backend.rs:1088-1091).
 *     `*_host` entry points take host memory, copy both ways and block until done.  They stage
 *     through device buffers that the library keeps per device and only ever grows, so repeated
 *     calls of one size allocate once; one host entry runs at a time per process.
 *   - Tensors are dense row-major: prefill `[B,H,N,D]` (crates/rustorch-attention/src/cpu_forward.rs:22-27),
 *     KV cache `[B,Hkv,max_seq,D]` (crates/rustorch-nn/src/kv_cache.rs:49-60; the CUDA model's
 *     `[Hkv,max_seq,D]` of crates/rustorch-cuda/src/llm_kernels.rs:349-352 is the B = 1 case),
 *     decode q/out `[B,Hq,D]`.
 *   - LSE is the natural-log log-sum-exp of the scaled scores of a row (`m + ln l` of
 *     `OnlineSoftmaxState`, crates/rustorch-attention/src/online_softmax.rs:44-56);
 *     a row with no visible key has LSE = -inf.
 *   - There is no CPU fallback: without a CUDA device every compute entry point fails.
 */
#ifndef RUSTORCH_ATTN_H
#define RUSTORCH_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------ */
#define RT_OK 0
/* AttentionError::ZeroDim (cpu_forward.rs:108) */
#define RT_ERR_ZERO_DIM (-1)
/* AttentionError::BufferShapeMismatch{which,expected,got} (cpu_forward.rs:94-102) */
#define RT_ERR_BUFFER_SHAPE (-2)
/* AttentionError::OutputShapeMismatch (cpu_forward.rs:103-108) */
#define RT_ERR_OUTPUT_SHAPE (-3)
/* AttentionError::Mask(MaskError::PaddingLengthMismatch) (mask.rs:70-78) */
#define RT_ERR_MASK_LEN (-4)
/* GQAError::HeadCountMismatch (gqa.rs:37-44) */
#define RT_ERR_HEAD_COUNT (-5)
/* GQAError::WrongInputLen (gqa.rs:45-54) */
#define RT_ERR_WRONG_INPUT_LEN (-6)
/* CudaError::Unsupported{msg} (error.rs): shape outside what the kernels implement */
#define RT_ERR_UNSUPPORTED (-7)
#define RT_ERR_NULL_POINTER (-8)
/* kv_len > max_seq, negative sizes */
#define RT_ERR_BAD_LENGTH (-9)
/* caller workspace too small or missing */
#define RT_ERR_WORKSPACE (-10)
/* a device pointer is not 16-byte aligned */
#define RT_ERR_ALIGNMENT (-11)
/* a bounded device-side wait ran out; see rt_attn_device_status() */
#define RT_ERR_DEVICE_TIMEOUT (-12)
/* the problem needs more scratch than the library's built-in static buffer holds */
#define RT_ERR_STATIC_SCRATCH (-13)

/* ---- mask flags for the prefill entry points ---------------------------------------- */
#define RT_MASK_NONE 0
/* Mask::Causal: key j > query i is masked (mask.rs:43) */
#define RT_MASK_CAUSAL 1

/* Mask kinds of the reference enum, for the host entry that mirrors it (mask.rs:26-34) */
#define RT_MASKKIND_NONE 0
#define RT_MASKKIND_CAUSAL 1
#define RT_MASKKIND_PADDING 2

/* precision selector of the f32 host entry points */
#define RT_PRECISION_F32 0  /* f32 CUDA-core kernel, parity with the f32 reference at 1e-4 */
#define RT_PRECISION_BF16 1 /* inputs rounded to bf16 (RNE), tcgen05 tensor-core kernel */

/* Library version: major*10000 + minor*100 + patch. */
int rt_attn_version(void);

/* Static description of a status code (never NULL). */
const char* rt_attn_error_string(int status);

/*
 * Reads (and clears) the device-side status word of the current device: 0 = clean,
 * otherwise a code identifying which bounded wait inside a kernel gave up (101-113: a barrier of
 * the prefill kernel, 301: a TMA stage of the decode kernel, 401: a peer's record in
 * rt_attn_merge_records_after).  Synchronises the device.  Returns RT_OK, a cudaError_t, or RT_ERR_DEVICE_TIMEOUT when *status != 0.
 */
int rt_attn_device_status(int* status);

/* ===================================================================================== *
 * Prefill — replaces rustorch_attention::flash_forward / flash_forward_masked
 * (crates/rustorch-attention/src/cpu_forward.rs:175-242) on device memory.
 * ===================================================================================== */

/*
 * Tiled flash-attention forward on bf16 device tensors, tcgen05/TMEM tensor-core kernel.
 *   q, k, v, out : bf16 [B,H,N,D], 16-byte aligned.  D must be 64 or 128.
 *   lse          : NULL or f32 [B,H,N].
 *   mask_flags   : RT_MASK_NONE or RT_MASK_CAUSAL.
 *   kv_lens      : NULL or device int32 [B]; keys j >= kv_lens[b] are masked for batch b
 *                  (the padding mask of a right-padded batch; combines with causal).
 *   key_keep     : NULL or device u8 keep flags (0 = masked), the reference's
 *                  Mask::Padding (mask.rs:31-33); batch b reads key_keep + b*keep_batch_stride,
 *                  stride 0 shares one vector of length N across the batch as the reference does.
 *   scale        : softmax scale; <= 0 selects the reference's 1/sqrt(D) (cpu_forward.rs:208).
 * Semantics follow the reference with two documented choices: a row whose visible keys
 * begin after a fully masked stretch gets the finite (naive_forward_masked) answer, and a
 * row with no visible key is NaN with LSE = -inf (cpu_forward.rs:411-420).  Padded QUERY
 * rows are computed like any other row (mask.rs:44 masks keys only).
 * N = 0 is a no-op (cpu_forward.rs:203-206).
 */
int rt_attn_prefill_bf16(const void* q, const void* k, const void* v, void* out, float* lse,
                         int64_t batch, int64_t heads, int64_t seq, int dim, int mask_flags,
                         const int32_t* kv_lens, const uint8_t* key_keep, int64_t keep_batch_stride,
                         float scale, void* stream);

/*
 * The same kernel for the shapes around self-attention that the reference's callers produce:
 * grouped KV heads without materialising the repeated heads (the reference copies them,
 * crates/rustorch-nn/src/gqa.rs:154-168), and a block of seq_q queries against seq_kv >= seq_q keys —
 * a prompt chunk attending to an existing KV cache, which the reference's CUDA model cannot do
 * (its prefill is a loop of single-token decode steps, crates/rustorch-llm/src/cuda_backend.rs:26-27)
 * and its Metal backend does with gqa_decode_batched_f32 (crates/rustorch-metal/src/kernels.rs:14422-14516).
 *   q, out : bf16 [B,Hq,seq_q,D];  k, v : bf16 [B,Hkv,seq_kv,D] (a cache passes seq_kv = max_seq);
 *   lse    : NULL or f32 [B,Hq,seq_q].  Query head h reads KV head h / (Hq/Hkv) (gqa.rs:233).
 *   kv_lens   : NULL or device int32 [B], visible keys per batch (<= seq_kv).
 *   q_offsets : NULL or device int32 [B]; with RT_MASK_CAUSAL query row i of batch b sits at key
 *               position i + q_offsets[b] and sees keys 0 .. i + q_offsets[b] (the Metal kernel's
 *               pos_base).  NULL = 0, i.e. Mask::Causal of self-attention (mask.rs:43).
 *   key_keep, keep_batch_stride, scale : as in rt_attn_prefill_bf16 (flags indexed by key, length seq_kv).
 */
int rt_attn_prefill_gqa_bf16(const void* q, const void* k, const void* v, void* out, float* lse,
                             int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seq_q,
                             int64_t seq_kv, int dim, int mask_flags, const int32_t* kv_lens,
                             const int32_t* q_offsets, const uint8_t* key_keep,
                             int64_t keep_batch_stride, float scale, void* stream);

/*
 * rt_attn_prefill_gqa_bf16 on strided views.  The reference's attention modules keep activations
 * as [B, T, H*hd] and pay a full-tensor transpose to [B, H, T, hd] for each of Q, K and V before
 * the kernel and one back after it (crates/rustorch-nn/src/attention.rs:468-485 and 499-543,
 * gqa.rs:151-168).  Here the layout is described to the TMA unit instead: each tensor is given by
 * the element strides {batch, head, row} of its [B, H, N, D] view, the head dim being contiguous.
 * A [B, T, H*hd] activation is the view with strides {T*H*hd, hd, H*hd}; a contiguous
 * [B, H, N, D] tensor has {H*N*D, N*D, D}.
 *   q_strides, k_strides, v_strides, out_strides : HOST pointers to 3 int64 each; every stride
 *       a positive multiple of 8 elements (16 bytes), row stride >= D.
 *   lse stays a contiguous f32 [B,Hq,seq_q]; all other arguments as in rt_attn_prefill_gqa_bf16.
 */
int rt_attn_prefill_strided_bf16(const void* q, const void* k, const void* v, void* out, float* lse,
                                 int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seq_q,
                                 int64_t seq_kv, int dim, const int64_t* q_strides,
                                 const int64_t* k_strides, const int64_t* v_strides,
                                 const int64_t* out_strides, int mask_flags, const int32_t* kv_lens,
                                 const int32_t* q_offsets, const uint8_t* key_keep,
                                 int64_t keep_batch_stride, float scale, void* stream);

/*
 * The same operator on f32 device tensors with f32 arithmetic on CUDA cores (any D in
 * [1,256]); grouped KV heads and seq_q != seq_kv are allowed so that it also serves
 * gqa_forward_f32's prefill and cross-attention branches (gqa.rs:151-210).
 *   q, out : f32 [B,Hq,Nq,D];  k, v : f32 [B,Hkv,Nkv,D];  lse : NULL or f32 [B,Hq,Nq].
 *   kv_lens, q_offsets, key_keep : as in rt_attn_prefill_gqa_bf16.
 */
int rt_attn_prefill_f32(const float* q, const float* k, const float* v, float* out, float* lse,
                        int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seq_q,
                        int64_t seq_kv, int dim, int mask_flags, const int32_t* kv_lens,
                        const int32_t* q_offsets, const uint8_t* key_keep, int64_t keep_batch_stride,
                        float scale, void* stream);

/*
 * Flash-attention backward on f32 device tensors, CUDA cores: (dQ, dK, dV) of
 * O = softmax(scale * Q K^T [+ causal mask]) V for an upstream gradient dO.  Replaces
 * flash_backward (crates/rustorch-attention/src/cpu_backward.rs:46-185), which rebuilds the whole
 * N x N probability matrix per (batch, head); this entry consumes what the forward pass saved
 * instead (the module header of cpu_backward.rs, :29-34, names that as the GPU recomputation path):
 *   q, k, v, out, d_out, dq, dk, dv : f32 [B,H,N,D], D in [1,256];
 *   lse : f32 [B,H,N], the LSE output of rt_attn_prefill_f32 on the same q, k, mask and scale;
 *   mask_flags : RT_MASK_NONE (the reference's case) or RT_MASK_CAUSAL;
 *   workspace  : device scratch of rt_attn_backward_workspace_bytes() bytes (holds dO . O per row).
 * The outputs are fully overwritten (the reference zeroes them first, :78-87).  N = 0 is a no-op
 * (:74-76).  Deterministic: no atomics, fixed summation order.
 */
size_t rt_attn_backward_workspace_bytes(int64_t batch, int64_t heads, int64_t seq);
int rt_attn_backward_f32(const float* q, const float* k, const float* v, const float* out,
                         const float* d_out, const float* lse, float* dq, float* dk, float* dv,
                         int64_t batch, int64_t heads, int64_t seq, int dim, int mask_flags,
                         float scale, void* workspace, size_t workspace_bytes, void* stream);

/*
 * The backward of rt_attn_prefill_bf16 on the tensor cores (mma.sync, bf16 operands, f32
 * accumulation; D in {64,128}): the same math as rt_attn_backward_f32 with P and dS rounded to
 * bf16 for the accumulating products, as the forward rounds P.
 *   q, k, v, out, d_out : bf16 [B,H,N,D];  lse : f32 [B,H,N] from the forward on the same inputs;
 *   dq, dk, dv : f32 [B,H,N,D], fully overwritten;  workspace as for rt_attn_backward_f32.
 */
int rt_attn_backward_bf16(const void* q, const void* k, const void* v, const void* out,
                          const void* d_out, const float* lse, float* dq, float* dk, float* dv,
                          int64_t batch, int64_t heads, int64_t seq, int dim, int mask_flags,
                          float scale, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Host-slice mirror of
 *   flash_backward(shape:&AttentionShape, q, k, v, do_:&[f32], dq, dk, dv:&mut [f32])
 * (cpu_backward.rs:46-55).  Lengths are validated in the reference's order: q, k, v, do give
 * RT_ERR_BUFFER_SHAPE (:57-65), dq, dk, dv give RT_ERR_OUTPUT_SHAPE (:66-73).  Runs the f32 forward
 * for O and LSE, then rt_attn_backward_f32; copies back, blocks.  mask_kind: RT_MASKKIND_NONE
 * (the reference) or RT_MASKKIND_CAUSAL.
 */
int rt_flash_backward_f32_host(const float* q, size_t q_len, const float* k, size_t k_len,
                               const float* v, size_t v_len, const float* d_out, size_t d_out_len,
                               float* dq, size_t dq_len, float* dk, size_t dk_len, float* dv,
                               size_t dv_len, int64_t batch, int64_t heads, int64_t seq,
                               int64_t dim, int mask_kind);

/*
 * Host-slice mirror of
 *   flash_forward_masked(shape:&AttentionShape, q:&[f32], k:&[f32], v:&[f32], mask:&Mask, out:&mut [f32])
 * (cpu_forward.rs:193-200; flash_forward at :175-183 is mask_kind = RT_MASKKIND_NONE).
 * `*_len` are the slice lengths in elements and are validated exactly like validate()
 * (cpu_forward.rs:142-169) and Mask::validate (mask.rs:51-65).  `br`/`bc` of AttentionShape
 * only change summation order in the reference and are not part of this ABI.
 * Copies to the device, runs the selected kernel, copies back, blocks.
 */
int rt_flash_forward_f32_host(const float* q, size_t q_len, const float* k, size_t k_len,
                              const float* v, size_t v_len, float* out, size_t out_len,
                              int64_t batch, int64_t heads, int64_t seq, int64_t dim, int mask_kind,
                              const uint8_t* keep, size_t keep_len, int precision);

/*
 * Host entry for bf16 tensors: the end-to-end call a host-resident caller makes.
 * q,k,v,out are host bf16 [B,H,N,D] (pinned memory recommended), lse NULL or host f32 [B,H,N],
 * kv_lens NULL or host int32 [B].  Copies in, runs rt_attn_prefill_bf16, copies out, blocks.
 */
int rt_attn_prefill_bf16_host(const void* q, const void* k, const void* v, void* out, float* lse,
                              int64_t batch, int64_t heads, int64_t seq, int dim, int mask_flags,
                              const int32_t* kv_lens, float scale);

/* ===================================================================================== *
 * Decode — replaces LlmKernels::gqa_decode_online_bf16 / gqa_decode_naive_bf16
 * (crates/rustorch-cuda/src/llm_kernels.rs:376-536, wrappers :915-958, :1000-1042) and the
 * seq_q == 1 branch of rustorch_nn::gqa::gqa_forward_f32 (crates/rustorch-nn/src/gqa.rs:190-270).
 * ===================================================================================== */

/*
 * Bytes of device scratch the split-KV decode needs for this problem size (partial
 * (O, m, l) records of every KV chunk).  Returns 0 when no scratch is needed.
 */
size_t rt_gqa_decode_workspace_bytes(int64_t batch, int64_t n_heads, int64_t n_kv_heads, int head_dim,
                                     int64_t max_seq);

/*
 * Batched single-token GQA decode over a bf16 KV cache with per-sequence lengths.
 *   q [B,Hq,D] bf16;  k_cache, v_cache [B,Hkv,max_seq,D] bf16;  16-byte aligned.
 *   out_bf16 : NULL or bf16 [B,Hq,D];  out_f32 : NULL or f32 [B,Hq,D] (at least one of them);
 *   lse      : NULL or f32 [B,Hq].
 *   kv_lens  : device int32 [B], or NULL to use `kv_len_uniform` for every sequence.
 *   kv_begin / kv_end : sequence b attends to positions [kv_begin, min(kv_end, len_b));
 *              kv_end < 0 = unbounded.  A non-trivial range yields the partial result of a
 *              KV shard; merge shards with rt_attn_merge_partials.
 *   Query head h reads KV head h / (Hq/Hkv) (gqa.rs:233; llm_kernels.rs:410 is the same map).
 *   head_dim must be 64, 128 or 256 and Hq/Hkv one of 1,2,4,8.
 *   An empty range gives out = 0 and lse = -inf (the reference kernels return zeros too:
 *   gqa.rs:262-269 with seq_kv = 0, llm_kernels.rs:456).
 *   workspace : device scratch of at least rt_gqa_decode_workspace_bytes(...) bytes.
 */
int rt_gqa_decode_bf16(const void* q, const void* k_cache, const void* v_cache, void* out_bf16,
                       float* out_f32, float* lse, int64_t batch, int64_t n_heads, int64_t n_kv_heads,
                       int head_dim, int64_t max_seq, const int32_t* kv_lens, int64_t kv_len_uniform,
                       int64_t kv_begin, int64_t kv_end, float scale, void* workspace,
                       size_t workspace_bytes, void* stream);

/*
 * rt_gqa_decode_bf16 for a KV shard, writing the partial as one packed record per output row:
 *   record f32 [B*Hq, D+1] = normalised O (D floats) followed by LSE — the unit that the ranks of a
 * split-KV decode exchange (one all-gather of B*Hq*(D+1) floats per rank) and that
 * rt_attn_merge_records consumes.  Same arguments and rules as rt_gqa_decode_bf16 otherwise.
 */
int rt_gqa_decode_record_bf16(const void* q, const void* k_cache, const void* v_cache, float* record,
                              int64_t batch, int64_t n_heads, int64_t n_kv_heads, int head_dim, int64_t max_seq,
                              const int32_t* kv_lens, int64_t kv_len_uniform, int64_t kv_begin, int64_t kv_end,
                              float scale, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Drop-in for
 *   LlmKernels::gqa_decode_online_bf16(stream, q, k_cache, v_cache, out, n_heads, n_kv, kv_len, head_dim, max_seq)
 * (llm_kernels.rs:915-927): one sequence, caches [n_kv,max_seq,head_dim], scale = 1/sqrt(head_dim)
 * (llm_kernels.rs:933), plus the caller-owned scratch this library needs instead of
 * allocating.  gqa_decode_naive_bf16 (llm_kernels.rs:1000-1012) has the same signature and
 * the same result; bind both names to this symbol.
 */
int rt_gqa_decode_online_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                              int n_heads, int n_kv, int kv_len, int head_dim, int max_seq,
                              void* workspace, size_t workspace_bytes, void* stream);

/*
 * Size of the scratch array built into the library for rt_gqa_decode_online_bf16_static.
 * 8 MiB holds 508 chunk partials of one sequence with Hq = 32, D = 128 (16,512 bytes each), i.e.
 * about 65,000 cached tokens at the smallest chunk size and up to 520,192 at the largest.
 */
#define RT_DECODE_STATIC_SCRATCH_BYTES (8u << 20)

/*
 * rt_gqa_decode_online_bf16 for callers that cannot hand over scratch memory.  No counterpart in
 * the reference (its kernel needs no scratch); the argument list is exactly the reference's
 * LlmKernels::gqa_decode_online_bf16, which is the point: a binding with that fixed signature has
 * nowhere to pass a workspace, and a serving loop that gave all device memory to its own pools
 * must not trigger cudaMalloc.  The scratch is a static array in device memory that every GPU
 * loading the library holds until exit (RT_DECODE_STATIC_SCRATCH_BYTES).
 *   - Allocates nothing: no cudaMalloc / cudaFree, no allocating library call.
 *   - The first call on each device resolves the array's device address (it may create the CUDA
 *     context); make that first call before starting any stream capture.
 *   - A problem whose partials exceed the array (rt_gqa_decode_workspace_bytes(1, n_heads, n_kv,
 *     head_dim, max_seq) > RT_DECODE_STATIC_SCRATCH_BYTES) returns RT_ERR_STATIC_SCRATCH.
 *   - All calls share the one array.  Nothing in it needs clearing between calls, but two calls
 *     that overlap on the GPU (different streams, or different host threads) race on it:
 *     serialise them, or use rt_gqa_decode_online_bf16 with separate workspaces.
 * Results are identical to rt_gqa_decode_online_bf16.
 */
int rt_gqa_decode_online_bf16_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                     int n_heads, int n_kv, int kv_len, int head_dim, int max_seq,
                                     void* stream);

/*
 * Merge R partial results of the same rows (split-KV across GPUs or across calls):
 *   LSE = logsumexp_r LSE_r,   O = sum_r exp(LSE_r - LSE) * O_r
 * — combine_tiles (online_softmax.rs:105-131) with a value vector attached; a partial with
 * LSE = -inf is the identity element.
 *   o_parts f32 [R,rows,D], lse_parts f32 [R,rows]  (device)
 *   out_bf16 NULL or bf16 [rows,D]; out_f32 NULL or f32 [rows,D]; lse NULL or f32 [rows].
 */
int rt_attn_merge_partials(const float* o_parts, const float* lse_parts, int64_t n_parts, int64_t rows,
                           int dim, void* out_bf16, float* out_f32, float* lse, void* stream);

/*
 * rt_attn_merge_partials over packed records: records f32 [R, rows, D+1] as written by
 * rt_gqa_decode_record_bf16 (and gathered from R ranks).  n_parts <= 8192, D <= 256.
 */
int rt_attn_merge_records(const float* records, int64_t n_parts, int64_t rows, int dim, void* out_bf16,
                          float* out_f32, float* lse, void* stream);

/*
 * Split-KV exchange over peer memory (NVLink), the fused form of "all-gather the records, then
 * merge": each rank owns a buffer of `world` record slots and `world` 32-bit flags that its peers
 * can write (symmetric memory / IPC mappings; the reference's NCCL layer is a stub,
 * crates/rustorch-cuda/src/nccl.rs, so there is no reference counterpart).
 *   rt_splitkv_push_record : copies this rank's packed record ([rows, D+1] f32, as written by
 *       rt_gqa_decode_record_bf16) into peer_slots[r] on every rank r with plain peer stores and then
 *       sets *peer_flags[r] = epoch with a system-scope release.  peer_slots / peer_flags are HOST
 *       arrays of `world` device pointers (the entry for this rank may alias `record`, which skips
 *       the copy).  Never waits.  rows * (D+1) must be a multiple of 4.
 *   rt_attn_merge_records_after : rt_attn_merge_records on the local slots once flags[r] >= epoch
 *       for every r < n_parts.  The wait is bounded by wait_clocks SM clocks (<= 0: 2^31, about a
 *       second); on expiry the kernel writes nothing and rt_attn_device_status reports 401.
 * Epochs must increase by one per exchange; with two slot sets used alternately a rank can never
 * overwrite a record that a slower peer is still merging.
 */
int rt_splitkv_push_record(const float* record, void* const* peer_slots, void* const* peer_flags,
                           int world, int64_t rows, int dim, uint32_t epoch, void* stream);
int rt_attn_merge_records_after(const float* records, const uint32_t* flags, uint32_t epoch,
                                int64_t wait_clocks, int64_t n_parts, int64_t rows, int dim,
                                void* out_bf16, float* out_f32, float* lse, void* stream);

/*
 * rt_gqa_decode_record_bf16 and rt_splitkv_push_record in one call: the kernel that merges the
 * chunk partials of this rank's KV shard into its record also stores every row into the slot each
 * peer keeps for this rank, and the CTA that finishes last sets the peers' flags to `epoch`, so the
 * record crosses NVLink while the remaining rows are still being merged and no separate copy
 * kernel runs.  `record` is this rank's own slot; peer_slots / peer_flags as in
 * rt_splitkv_push_record; done_counter is a device int32 that is zero between calls (the kernel
 * resets it).  A launch whose record comes straight from the decode kernel (a single chunk, or
 * chunks merged in-kernel) falls back to the copy kernel; the effect is the same.
 */
int rt_gqa_decode_record_push_bf16(const void* q, const void* k_cache, const void* v_cache,
                                   float* record, void* const* peer_slots, void* const* peer_flags,
                                   int world, uint32_t epoch, int* done_counter, int64_t batch,
                                   int64_t n_heads, int64_t n_kv_heads, int head_dim, int64_t max_seq,
                                   const int32_t* kv_lens, int64_t kv_len_uniform, int64_t kv_begin,
                                   int64_t kv_end, float scale, void* workspace,
                                   size_t workspace_bytes, void* stream);

/*
 * The whole tail of a split-KV decode in one kernel, row by row (no reference counterpart: the
 * reference has no multi-device attention).  After the decode kernel has written the chunk partials of
 * this rank's KV shard, ONE kernel with one CTA per output row merges the row's partials, stores the
 * row (O | LSE) into the slot every rank keeps for this rank (plain stores, over NVLink for the peers;
 * nothing is loaded from a peer), raises that rank's flag for (this rank, row), waits (bounded by
 * wait_clocks SM clocks, <= 0: 2^31; expiry: nothing is written, device status 401) for the same row
 * from every rank, and merges the `world` rows from local memory into out / lse.  Compared with
 * rt_gqa_decode_record_bf16 + rt_splitkv_push_record + rt_attn_merge_records_after there is no record-
 * wide flag, no counter shared between CTAs and no kernel boundary between merge, delivery and merge.
 *   peer_slots[r] : on rank r, the [rows, D+1] f32 slot r keeps for THIS rank (r == rank: local memory)
 *   peer_flags[r] : on rank r, the [rows] u32 flags r keeps for THIS rank
 *   local_slots   : this rank's slots for all ranks, [world][rows][D+1] f32 (peer_slots[rank] points into it)
 *   local_flags   : this rank's flags for all ranks, [world][rows] u32 (zero before the first epoch)
 *   do_wait = 0   : stop after the delivery; rt_attn_merge_records_after_rows then finishes the step
 *                   (needed where several ranks are emulated on ONE GPU: a kernel must never wait for
 *                   a flag that a later launch on the same GPU raises).
 * Epochs increase by one per exchange and two slot / flag sets are used alternately, as above.
 */
int rt_gqa_decode_exchange_bf16(const void* q, const void* k_cache, const void* v_cache, void* out_bf16,
                                float* out_f32, float* lse, void* const* peer_slots,
                                void* const* peer_flags, const float* local_slots,
                                const uint32_t* local_flags, int world, int rank, uint32_t epoch,
                                int64_t wait_clocks, int do_wait, int64_t batch, int64_t n_heads,
                                int64_t n_kv_heads, int head_dim, int64_t max_seq, const int32_t* kv_lens,
                                int64_t kv_len_uniform, int64_t kv_begin, int64_t kv_end, float scale,
                                void* workspace, size_t workspace_bytes, void* stream);
/* rt_attn_merge_records_after with one flag per (rank, row): row_flags u32 [n_parts][rows]. */
int rt_attn_merge_records_after_rows(const float* records, const uint32_t* row_flags, uint32_t epoch,
                                     int64_t wait_clocks, int64_t n_parts, int64_t rows, int dim,
                                     void* out_bf16, float* out_f32, float* lse, void* stream);

/*
 * rt_gqa_decode_exchange_bf16 with the flag inside the data (no reference counterpart).  Every element of a
 * row travels as one 8-byte word {f32 bits, epoch}; an aligned 8-byte store is one access, so a reader that
 * finds the epoch in a word has the value that came with it.  There is no system-scope fence between data and
 * flag and no flag store: one NVLink round trip less per step.  The reader spins (bounded by wait_clocks, as
 * above; expiry: device status 401) on the words themselves.
 *   peer_words[r]  : on rank r, the [rows][D+1] u64 words r keeps for THIS rank (8-byte aligned; r == rank: local)
 *   local_words    : this rank's words for all ranks, [world][rows][D+1] u64, zero before the first epoch
 *   scratch_record : [rows, D+1] f32 of local memory (the decode writes the record here when the shard is one chunk)
 *   epoch          : >= 1, increasing by one per exchange; two word sets are used alternately by the caller
 *   do_wait = 0    : stop after the delivery; rt_attn_merge_ll_rows finishes the step (several ranks on ONE GPU)
 * head_dim 64 or 128 (one thread per word of a row: D + 1 <= 256; 256 returns RT_ERR_UNSUPPORTED before any launch).
 */
int rt_gqa_decode_exchange_ll_bf16(const void* q, const void* k_cache, const void* v_cache, void* out_bf16,
                                   float* out_f32, float* lse, void* const* peer_words,
                                   const void* local_words, float* scratch_record, int world, int rank,
                                   uint32_t epoch, int64_t wait_clocks, int do_wait, int64_t batch,
                                   int64_t n_heads, int64_t n_kv_heads, int head_dim, int64_t max_seq,
                                   const int32_t* kv_lens, int64_t kv_len_uniform, int64_t kv_begin,
                                   int64_t kv_end, float scale, void* workspace, size_t workspace_bytes,
                                   void* stream);
/* The second half of rt_gqa_decode_exchange_ll_bf16(do_wait = 0): bounded wait for every rank's words, then the merge. */
int rt_attn_merge_ll_rows(const void* local_words, uint32_t epoch, int64_t wait_clocks, int world,
                          int64_t rows, int dim, void* out_bf16, float* out_f32, float* lse, void* stream);

/*
 * Host-slice mirror of
 *   gqa_forward_f32(q,k,v,out, batch,n_heads,n_kv_heads,seq_q,seq_kv,head_dim) -> Result<(),GQAError>
 * (gqa.rs:94-105), f32 arithmetic.  seq_q == seq_kv runs the unmasked prefill without
 * materialising the repeated KV heads (the reference copies them, gqa.rs:154-168);
 * other shapes run the same f32 kernel with seq_q != seq_kv.  Blocks.
 */
int rt_gqa_forward_f32_host(const float* q, size_t q_len, const float* k, size_t k_len, const float* v,
                            size_t v_len, float* out, size_t out_len, int64_t batch, int64_t n_heads,
                            int64_t n_kv_heads, int64_t seq_q, int64_t seq_kv, int64_t head_dim);

/*
 * Drop-in for LlmKernels::kv_append_bf16(stream, k_cache, v_cache, k_in, v_in, pos, n_kv, head_dim, max_seq)
 * (llm_kernels.rs:345-373, wrapper :872-911), batched: k_in, v_in are bf16 [B,Hkv,D] and are
 * written at position pos (or positions[b] when `positions` is a device int32 [B]) of the
 * [B,Hkv,max_seq,D] caches.
 */
int rt_kv_append_bf16(void* k_cache, void* v_cache, const void* k_in, const void* v_in, int64_t batch,
                      int n_kv, int head_dim, int64_t max_seq, int64_t pos, const int32_t* positions,
                      void* stream);

/* Pairing of dimensions for the rotary embedding */
#define RT_ROPE_HALF_SPLIT 0 /* (k, k + D/2): crates/rustorch-nn/src/rope.rs:162-205, the CPU model and HF weights */
#define RT_ROPE_ADJACENT 1   /* (2k, 2k+1): rope.rs:96-150 and the CUDA kernel at llm_kernels.rs:109-143 */

/*
 * One launch for what LlamaModelCuda::decode_step does with three per layer and token
 * (rope_half_split_bf16 on Q, the same on K, kv_append_bf16: crates/rustorch-llm/src/cuda_backend.rs:917-966):
 * rotates q in place, rotates the new K row and writes it and the V row into the caches at the
 * sequence's position.  The caches are then ready for rt_gqa_decode_bf16 with kv_len = pos + 1.
 *   q [B,Hq,D] bf16 (in place); k_in, v_in [B,Hkv,D] bf16; caches [B,Hkv,max_seq,D] bf16;
 *   inv_freq device f32 [D/2] = theta^(-2k/D) as the reference uploads it (cuda_backend.rs:221-226);
 *   positions device int32 [B], or NULL to use `pos` for every sequence;  D must be even.
 * angle = pos * inv_freq[k] in f32 (RoPE::new, rope.rs:73-83); results are rounded to bf16 (RNE).
 */
int rt_rope_kv_append_bf16(void* q, const void* k_in, const void* v_in, void* k_cache, void* v_cache,
                           const float* inv_freq, int64_t batch, int n_heads, int n_kv, int head_dim,
                           int64_t max_seq, int64_t pos, const int32_t* positions, int rope_style, void* stream);

/* f32 <-> bf16 (RNE) conversion of n elements on the device; helpers of the host entries. */
int rt_convert_f32_to_bf16(const float* src, void* dst, int64_t n, void* stream);
int rt_convert_bf16_to_f32(const void* src, float* dst, int64_t n, void* stream);

/* ===================================================================================== *
 * Diagnostics (no counterpart in the reference).
 * ===================================================================================== */

/*
 * Runs the two tensor-core MMA shapes of the prefill kernel on one 128-row tile and returns
 * the raw f32 accumulators, so that the TMA / shared-memory / instruction descriptor
 * encodings can be checked against a plain matrix product:
 *   s_out [128,128] = A * B^T                 (A, B: bf16 [128,dim], the Q and K roles)
 *   o_out [128,dim] = bf16(s_out / 16) * V    (V: bf16 [128,dim])
 * dim must be 64 or 128; all pointers are device pointers.
 */
int rt_debug_tc_selftest(const void* a, const void* b, const void* v, float* s_out, float* o_out, int dim,
                         void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RUSTORCH_ATTN_H */
