// Single-sequence GQA decode that never allocates: the split-KV scratch lives inside the library.
//
// Who needs this.  The decode kernel writes one partial result per chunk of 128 to 1024 tokens and merges
// them, so it needs scratch memory.  The library's other decode entries take that scratch from
// the caller.  Two kinds of caller cannot supply it:
//   * a caller bound to the reference's ten-argument
//     LlmKernels::gqa_decode_online_bf16(stream, q, k_cache, v_cache, out, n_heads, n_kv, kv_len,
//     head_dim, max_seq): that signature has no scratch argument, and the call sits inside a
//     per-token, per-layer loop where nothing owns an allocator handle;
//   * a serving runtime that carved all device memory into its weight and KV-cache pools at
//     start-up and forbids cudaMalloc afterwards (cudaMalloc also synchronises the whole device,
//     which a decode loop cannot afford).
// For them this file keeps a fixed-size scratch array in device global memory.  Every GPU that
// loads the library carries the array (RT_DECODE_STATIC_SCRATCH_BYTES) until the process exits.
#include <mutex>

#include "../../include/rustorch_attn.h"
#include "kernels.h"

namespace {

// In host code this name is only a handle for the runtime, not a device address: the address
// each device uses is looked up once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_decode_static_scratch[RT_DECODE_STATIC_SCRATCH_BYTES];

std::mutex g_setup_mutex;
void* g_scratch_addr[64] = {nullptr};

// One-time set-up for the current device: resolve the device address of the scratch array.
// Runs on the first call made on each device; it may initialise the CUDA context and load the
// module, so that first call should happen before any stream capture begins.
int static_scratch_for_current_device(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return RT_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return RT_ERR_NULL_POINTER;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return RT_OK;
}

}  // namespace

extern "C" int rt_gqa_decode_online_bf16_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                                int n_heads, int n_kv, int kv_len, int head_dim, int max_seq,
                                                void* stream) {
    // Size first: a problem whose chunk partials do not fit the built-in array is refused
    // before anything touches the device.
    if (n_heads > 0 && n_kv > 0 && head_dim > 0 && max_seq > 0) {
        const size_t need = rt_gqa_decode_workspace_bytes(1, n_heads, n_kv, head_dim, max_seq);
        if (need > (size_t)RT_DECODE_STATIC_SCRATCH_BYTES) return RT_ERR_STATIC_SCRATCH;
    }
    void* scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != RT_OK) return rc;
    // Nothing in the array has to start at zero: every chunk slot the merge kernel reads is
    // written by this call's decode kernel first (a chunk with no visible token writes
    // LSE = -inf, which the merge skips), so whatever an earlier call left behind is never read.
    return rt_gqa_decode_online_bf16(q, k_cache, v_cache, out, n_heads, n_kv, kv_len, head_dim, max_seq, scratch,
                                     (size_t)RT_DECODE_STATIC_SCRATCH_BYTES, stream);
}
