// Host launchers for the reference's own CUDA C kernels.  TEST INFRASTRUCTURE ONLY.
//
// The reference keeps its decode-side CUDA kernels as string constants that it hands to NVRTC at
// run time (crates/rustorch-cuda/src/llm_kernels.rs).  build_ref.py extracts three of those strings,
// untouched, into a scratch directory at build time and compiles them together with this file into
// oracle/_ref/libref_llm_kernels.so; no reference source is kept in this repository.  The launch
// geometry below is the reference wrappers':
//   gqa_decode_online_bf16  llm_kernels.rs:915-958  grid (n_heads), block (head_dim), smem 4*head_dim,
//                                                    scale = 1/sqrt(head_dim) computed by the wrapper
//   kv_append_bf16          llm_kernels.rs:872-911  grid (n_kv, ceil(head_dim/block)), block min(64, head_dim)
//   rope_half_split_bf16    llm_kernels.rs:726-757  grid (n_heads, ceil(half/block)), block min(64, half)
// and the compile flags are the reference's NVRTC options (fast math, llm_kernels.rs:605-613).
// Only the tests and the benchmark's baseline rows load the resulting library; the shipped library
// never does.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "ref_gqa_decode_online_bf16.inc"
#include "ref_kv_append_bf16.inc"
#include "ref_rope_half_split_bf16.inc"

extern "C" int ref_gqa_decode_online_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                                          int n_heads, int n_kv, int kv_len, int head_dim, int max_seq, void* stream) {
    // The kernel's tree reduction assumes blockDim.x == head_dim and a power of two; one block holds at
    // most 1024 threads.  Anything else is refused here rather than launched.
    if (n_heads <= 0 || n_kv <= 0 || head_dim <= 0 || head_dim > 1024 || (head_dim & (head_dim - 1)) ||
        kv_len < 0 || kv_len > max_seq)
        return -1;
    const float scale = 1.0f / sqrtf((float)head_dim);
    gqa_decode_online_bf16<<<n_heads, head_dim, head_dim * 4, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out,
        n_heads, n_kv, kv_len, head_dim, max_seq, scale);
    return (int)cudaGetLastError();
}

extern "C" int ref_kv_append_bf16(void* k_cache, void* v_cache, const void* k_in, const void* v_in, int pos, int n_kv,
                                  int head_dim, int max_seq, void* stream) {
    if (n_kv <= 0 || head_dim <= 0 || pos < 0 || pos >= max_seq) return -1;
    const unsigned block = head_dim < 64 ? head_dim : 64;
    dim3 grid(n_kv, (head_dim + block - 1) / block);
    kv_append_bf16<<<grid, block, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
                                                            (const __nv_bfloat16*)k_in, (const __nv_bfloat16*)v_in,
                                                            pos, n_kv, head_dim, max_seq);
    return (int)cudaGetLastError();
}

extern "C" int ref_rope_half_split_bf16(void* x, const float* inv_freq, int pos, int n_heads, int head_dim,
                                        void* stream) {
    if (n_heads <= 0 || head_dim < 2 || (head_dim & 1) || pos < 0) return -1;
    const int half = head_dim / 2;
    const unsigned block = half < 64 ? half : 64;
    dim3 grid(n_heads, (half + block - 1) / block);
    rope_half_split_bf16<<<grid, block, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, inv_freq, pos, n_heads,
                                                                  head_dim);
    return (int)cudaGetLastError();
}
