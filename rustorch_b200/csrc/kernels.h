// Internal launch interface between the C ABI (api.cu) and the kernel translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace rt {

// ---- api.cu: device address of the status word of the current device (NULL on failure)
int* device_status_ptr();
// Multiprocessors of the current device, queried once per device; 148 (B200) when no device answers,
// so that the size queries that need no GPU (workspace bytes) stay deterministic.
int sm_count();

// ---- decode.cu
struct MergePush;
struct DecodeTail;
int decode_chunk_tokens(int64_t batch, int n_kv, int64_t max_seq);
int decode_num_chunks(int64_t batch, int n_kv, int64_t max_seq);
// Whether merge_partials_kernel can combine n_parts partials of this head dim (its weights live in
// shared memory).
bool merge_fits(int64_t n_parts, int dim);
cudaError_t launch_gqa_decode(const void* q, const void* k, const void* v, void* out_bf16, float* out_f32,
                              float* lse, int64_t batch, int n_heads, int n_kv, int head_dim,
                              int64_t max_seq, const int32_t* kv_lens, int64_t kv_len_uniform,
                              int64_t kv_begin, int64_t kv_end, float scale, void* workspace,
                              int64_t of_stride, int64_t lse_stride, cudaStream_t stream,
                              const struct MergePush* push = nullptr, bool* pushed = nullptr,
                              struct DecodeTail* tail = nullptr);
// With a DecodeTail the decode launches no chunk merge of its own: the caller gets the chunk partials
// ([n_chunks][rows][dim] O and [n_chunks][rows] LSE in the workspace) and combines them itself.  With a
// single chunk there are no partials; the outputs passed to launch_gqa_decode hold the result then.
struct DecodeTail {
    int n_chunks;
    const float* part_o;
    const float* part_lse;
};
// o_parts rows are in_row_stride floats apart, lse_parts entries in_lse_stride floats apart
// Optional bounded wait in front of a merge: flags[r] >= epoch means part r has arrived.
struct MergeWait {
    const uint32_t* flags;
    int n_flags;
    uint32_t epoch;
    long long max_clocks;
    int* status;
    int per_row;  // 0: flags[r]; 1: one flag per (part, row), flags[r * rows + row]
};
constexpr int kMaxPeers = 16;
// Optional delivery of a merge's output record ([rows, dim + 1] f32: O | LSE) to the peers of a split-KV
// decode: every row is also stored into dst[r] (r < world, entries equal to the local record are skipped);
// the CTA that finishes last (done_counter, zero between launches) then sets *flag[r] = epoch.
struct MergePush {
    float* dst[kMaxPeers];
    uint32_t* flag[kMaxPeers];
    int world;
    uint32_t epoch;
    int* done_counter;
};
cudaError_t launch_merge_partials(const float* o_parts, const float* lse_parts, int64_t n_parts, int64_t rows,
                                  int dim, int64_t in_row_stride, int64_t in_lse_stride, void* out_bf16,
                                  float* out_f32, float* lse, cudaStream_t stream, const MergeWait* wait = nullptr,
                                  const MergePush* push = nullptr, int64_t of_stride = 0, int64_t lse_stride = 0);
cudaError_t launch_row_exchange(const float* o_parts, const float* lse_parts, int64_t n_parts, int64_t rows, int dim,
                                int64_t in_row_stride, int64_t in_lse_stride, void* out_bf16, float* out_f32, float* lse,
                                void* const* peer_slots, void* const* peer_flags, const float* local_slots,
                                const uint32_t* local_flags, int world, uint32_t epoch, long long wait_clocks,
                                int do_wait, cudaStream_t stream);
// The row exchange with the flag inside every 8-byte word (no fence, no flag store): see decode.cu.
cudaError_t launch_row_exchange_ll(const float* o_parts, const float* lse_parts, int64_t n_parts, int64_t rows, int dim,
                                   int64_t in_row_stride, int64_t in_lse_stride, void* out_bf16, float* out_f32,
                                   float* lse, void* const* peer_words, const void* local_words, int world,
                                   uint32_t epoch, long long wait_clocks, int do_wait, cudaStream_t stream);
cudaError_t launch_ll_merge(const void* local_words, int world, int64_t rows, int dim, uint32_t epoch,
                            long long wait_clocks, void* out_bf16, float* out_f32, float* lse, cudaStream_t stream);
cudaError_t launch_push_records(const float* record, void* const* peer_slots, void* const* peer_flags, int world,
                                int64_t record_floats, uint32_t epoch, cudaStream_t stream);
cudaError_t launch_kv_append(void* k_cache, void* v_cache, const void* k_in, const void* v_in, int64_t batch,
                             int n_kv, int head_dim, int64_t max_seq, int64_t pos, const int32_t* positions,
                             cudaStream_t stream);

cudaError_t launch_rope_kv_append(void* q, const void* k_in, const void* v_in, void* k_cache, void* v_cache,
                                  const float* inv_freq, const int32_t* positions, int64_t pos_uniform,
                                  int64_t batch, int n_heads, int n_kv, int head_dim, int64_t max_seq, int style,
                                  cudaStream_t stream);

// ---- decode_tc.cu: TMA + mma.sync decode for head dim 64/128; cudaErrorNotSupported = shape not covered
cudaError_t launch_gqa_decode_tc(const void* q, const void* k, const void* v, void* out_bf16, float* out_f32,
                                 float* lse, int64_t batch, int n_heads, int n_kv, int head_dim, int64_t max_seq,
                                 const int32_t* kv_lens, int64_t kv_len_uniform, int64_t kv_begin, int64_t kv_end,
                                 float scale, float* part_o, float* part_lse, int* counters, int chunk, int n_chunks,
                                 int64_t of_stride, int64_t lse_stride, bool* merged, const MergePush* push,
                                 cudaStream_t stream);

// ---- prefill_simt.cu
cudaError_t launch_prefill_f32(const float* q, const float* k, const float* v, float* out, float* lse,
                               int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seq_q,
                               int64_t seq_kv, int dim, int causal, const int32_t* kv_lens,
                               const int32_t* q_offsets, const uint8_t* key_keep, int64_t keep_batch_stride,
                               float scale, cudaStream_t stream);
cudaError_t launch_f32_to_bf16(const float* src, void* dst, int64_t n, cudaStream_t stream);
cudaError_t launch_bf16_to_f32(const void* src, float* dst, int64_t n, cudaStream_t stream);

// Raises a kernel's dynamic shared-memory limit once per device instead of on every launch (the value
// per kernel never changes; a race between two first launches sets the same value twice).
template <auto Kern>
inline cudaError_t set_max_dynamic_smem_once(int bytes) {
    static bool done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
    return e;
}

// ---- backward_simt.cu
cudaError_t launch_backward_f32(const float* q, const float* k, const float* v, const float* out, const float* d_out,
                                const float* lse, float* dq, float* dk, float* dv, float* delta_ws, int64_t batch,
                                int64_t heads, int64_t seq, int dim, int causal, float scale, cudaStream_t stream);

// ---- backward_tc.cu (mma.sync bf16)
cudaError_t launch_backward_bf16(const void* q, const void* k, const void* v, const void* out, const void* d_out,
                                 const float* lse, float* dq, float* dk, float* dv, float* delta_ws, int64_t batch,
                                 int64_t heads, int64_t seq, int dim, int causal, float scale, cudaStream_t stream);

// ---- backward_tcgen05.cu (tcgen05 / TMEM / TMA); cudaErrorNotSupported = shape not covered
cudaError_t launch_backward_tcgen05(const void* q, const void* k, const void* v, const void* d_out, const float* lse,
                                    const float* delta, float* dq, float* dk, float* dv, int64_t batch, int64_t heads,
                                    int64_t seq, int dim, int causal, float scale, cudaStream_t stream);

// ---- prefill_tc.cu (tcgen05 / TMEM / TMA)
// Element strides of a [B, H, N, D] view whose inner dim is contiguous.
struct TensorStrides {
    int64_t batch, head, row;
    static TensorStrides contiguous(int64_t heads, int64_t seq, int dim) {
        return TensorStrides{heads * seq * dim, seq * dim, (int64_t)dim};
    }
};
cudaError_t launch_prefill_tc(const void* q, const void* k, const void* v, void* out, float* lse,
                              int64_t batch, int64_t heads, int64_t heads_kv, int64_t seq, int64_t seq_kv, int dim,
                              const TensorStrides& sq, const TensorStrides& sk, const TensorStrides& sv,
                              const TensorStrides& so, int causal, const int32_t* kv_lens,
                              const int32_t* q_offsets, const uint8_t* key_keep, int64_t keep_batch_stride,
                              float scale, cudaStream_t stream);

}  // namespace rt
