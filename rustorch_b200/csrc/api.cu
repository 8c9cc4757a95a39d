// extern "C" boundary of the attention library: argument validation (mirroring the reference's
// validate() / Mask::validate / gqa_forward_f32 checks) and dispatch to the sm_100a kernels.
// Nothing here computes attention on the host: without a CUDA device every compute entry fails.
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <mutex>

#include "../../include/rustorch_attn.h"
#include "common.cuh"
#include "kernels.h"

namespace rt {
__device__ int g_device_status = 0;

int* device_status_ptr() {
    static std::atomic<int*> cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    int* p = cache[dev].load(std::memory_order_acquire);
    if (!p) {  // two first callers may both look the address up; they store the same value
        void* q = nullptr;
        if (cudaGetSymbolAddress(&q, g_device_status) != cudaSuccess) return nullptr;
        p = static_cast<int*>(q);
        cache[dev].store(p, std::memory_order_release);
    }
    return p;
}

int sm_count() {
    static std::atomic<int> cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cache[dev].load(std::memory_order_relaxed);
    if (n <= 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
        cache[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}
}  // namespace rt

namespace {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline float default_scale(float scale, int dim) { return scale > 0.f ? scale : 1.0f / std::sqrt((float)dim); }

// Device staging buffers of the blocking host entry points.  They are kept per device and only
// ever grow, so a caller that streams same-sized problems through a *_host entry pays for
// cudaMalloc once, not per call.  One host entry runs at a time per process (the pool is locked
// for the duration of the call); the device-pointer entries never touch it.
struct HostStaging {
    static constexpr int kSlots = 10;
    void* ptr[64][kSlots] = {};
    size_t cap[64][kSlots] = {};
    std::mutex mu;
    cudaError_t get(int slot, size_t bytes, void** out) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
        if (bytes == 0) bytes = 1;
        if (cap[dev][slot] < bytes) {
            if (ptr[dev][slot]) {
                e = cudaFree(ptr[dev][slot]);
                ptr[dev][slot] = nullptr;
                cap[dev][slot] = 0;
                if (e != cudaSuccess) return e;
            }
            e = cudaMalloc(&ptr[dev][slot], bytes);
            if (e != cudaSuccess) return e;
            cap[dev][slot] = bytes;
        }
        *out = ptr[dev][slot];
        return cudaSuccess;
    }
};
HostStaging g_staging;

// One staging buffer of the pool (slot = which of the call's tensors).
struct DevBuf {
    void* p = nullptr;
    int slot;
    explicit DevBuf(int s) : slot(s) {}
    cudaError_t alloc(size_t bytes) { return g_staging.get(slot, bytes, &p); }
    template <class T>
    T* as() const { return static_cast<T*>(p); }
};

#define RT_CUDA(expr)                         \
    do {                                      \
        cudaError_t _e = (expr);              \
        if (_e != cudaSuccess) return (int)_e; \
    } while (0)

}  // namespace

extern "C" {

int rt_attn_version(void) { return 100; }

const char* rt_attn_error_string(int status) {
    switch (status) {
        case RT_OK: return "ok";
        case RT_ERR_ZERO_DIM: return "dim must be > 0";
        case RT_ERR_BUFFER_SHAPE: return "q/k/v buffer length does not match the shape";
        case RT_ERR_OUTPUT_SHAPE: return "output buffer length does not match the shape";
        case RT_ERR_MASK_LEN: return "padding mask length does not match seq";
        case RT_ERR_HEAD_COUNT: return "n_heads not divisible by n_kv_heads";
        case RT_ERR_WRONG_INPUT_LEN: return "gqa buffer length does not match the shape";
        case RT_ERR_UNSUPPORTED: return "shape not supported by the sm_100a kernels";
        case RT_ERR_NULL_POINTER: return "required pointer is NULL";
        case RT_ERR_BAD_LENGTH: return "negative size or kv_len > max_seq";
        case RT_ERR_WORKSPACE: return "workspace missing or too small";
        case RT_ERR_ALIGNMENT: return "device pointer not 16-byte aligned";
        case RT_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait expired";
        case RT_ERR_STATIC_SCRATCH: return "problem needs more scratch than the built-in static buffer holds";
        default: return status > 0 ? cudaGetErrorString((cudaError_t)status) : "unknown status";
    }
}

int rt_attn_device_status(int* status) {
    if (!status) return RT_ERR_NULL_POINTER;
    RT_CUDA(cudaDeviceSynchronize());
    int v = 0;
    RT_CUDA(cudaMemcpyFromSymbol(&v, rt::g_device_status, sizeof(int)));
    if (v != 0) {
        const int zero = 0;
        RT_CUDA(cudaMemcpyToSymbol(rt::g_device_status, &zero, sizeof(int)));
    }
    *status = v;
    return v ? RT_ERR_DEVICE_TIMEOUT : RT_OK;
}

// ------------------------------------------------------------------------------ prefill

// Shared body of the bf16 prefill entries; strides are in elements.
static int prefill_bf16_common(const void* q, const void* k, const void* v, void* out, float* lse, int64_t batch,
                               int64_t heads_q, int64_t heads_kv, int64_t seq_q, int64_t seq_kv, int dim,
                               const rt::TensorStrides& sq, const rt::TensorStrides& sk, const rt::TensorStrides& sv,
                               const rt::TensorStrides& so, int mask_flags, const int32_t* kv_lens,
                               const int32_t* q_offsets, const uint8_t* key_keep, int64_t keep_batch_stride,
                               float scale, void* stream) {
    if (dim == 0) return RT_ERR_ZERO_DIM;
    if (batch < 0 || heads_q < 0 || heads_kv < 0 || seq_q < 0 || seq_kv < 0 || dim < 0 || keep_batch_stride < 0)
        return RT_ERR_BAD_LENGTH;
    if (batch == 0 || heads_q == 0 || seq_q == 0) return RT_OK;  // cpu_forward.rs:203-206
    if (heads_kv == 0 || heads_q % heads_kv != 0) return RT_ERR_HEAD_COUNT;  // gqa.rs:106-111
    if (!q || !out || (seq_kv > 0 && (!k || !v))) return RT_ERR_NULL_POINTER;
    if (dim != 64 && dim != 128) return RT_ERR_UNSUPPORTED;
    if (seq_q > (1 << 30) || seq_kv > (1 << 30) || batch * heads_q > (1 << 30)) return RT_ERR_UNSUPPORTED;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return RT_ERR_ALIGNMENT;
    if (mask_flags & ~RT_MASK_CAUSAL) return RT_ERR_UNSUPPORTED;
    for (const rt::TensorStrides* s : {&sq, &sk, &sv, &so}) {
        // TMA strides: positive multiples of 16 bytes below 2^40; a row must hold the head dim
        if (s->batch <= 0 || s->head <= 0 || s->row < dim) return RT_ERR_BAD_LENGTH;
        if ((s->batch | s->head | s->row) & 7) return RT_ERR_ALIGNMENT;
        if (s->batch >= (1ll << 39) || s->head >= (1ll << 39) || s->row >= (1ll << 39)) return RT_ERR_UNSUPPORTED;
    }
    RT_CUDA(rt::launch_prefill_tc(q, k, v, out, lse, batch, heads_q, heads_kv, seq_q, seq_kv, dim, sq, sk, sv, so,
                                  mask_flags & RT_MASK_CAUSAL, kv_lens, q_offsets, key_keep, keep_batch_stride,
                                  default_scale(scale, dim), as_stream(stream)));
    return RT_OK;
}

int rt_attn_prefill_gqa_bf16(const void* q, const void* k, const void* v, void* out, float* lse, int64_t batch,
                             int64_t heads_q, int64_t heads_kv, int64_t seq_q, int64_t seq_kv, int dim, int mask_flags,
                             const int32_t* kv_lens, const int32_t* q_offsets, const uint8_t* key_keep,
                             int64_t keep_batch_stride, float scale, void* stream) {
    const int d = dim > 0 ? dim : 1;
    const rt::TensorStrides sq = rt::TensorStrides::contiguous(heads_q > 0 ? heads_q : 1, seq_q > 0 ? seq_q : 1, d);
    const rt::TensorStrides sk = rt::TensorStrides::contiguous(heads_kv > 0 ? heads_kv : 1, seq_kv > 0 ? seq_kv : 1, d);
    return prefill_bf16_common(q, k, v, out, lse, batch, heads_q, heads_kv, seq_q, seq_kv, dim, sq, sk, sk, sq,
                               mask_flags, kv_lens, q_offsets, key_keep, keep_batch_stride, scale, stream);
}

int rt_attn_prefill_strided_bf16(const void* q, const void* k, const void* v, void* out, float* lse, int64_t batch,
                                 int64_t heads_q, int64_t heads_kv, int64_t seq_q, int64_t seq_kv, int dim,
                                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                 const int64_t* out_strides, int mask_flags, const int32_t* kv_lens,
                                 const int32_t* q_offsets, const uint8_t* key_keep, int64_t keep_batch_stride,
                                 float scale, void* stream) {
    if (!q_strides || !k_strides || !v_strides || !out_strides) return RT_ERR_NULL_POINTER;
    const rt::TensorStrides sq{q_strides[0], q_strides[1], q_strides[2]};
    const rt::TensorStrides sk{k_strides[0], k_strides[1], k_strides[2]};
    const rt::TensorStrides sv{v_strides[0], v_strides[1], v_strides[2]};
    const rt::TensorStrides so{out_strides[0], out_strides[1], out_strides[2]};
    return prefill_bf16_common(q, k, v, out, lse, batch, heads_q, heads_kv, seq_q, seq_kv, dim, sq, sk, sv, so,
                               mask_flags, kv_lens, q_offsets, key_keep, keep_batch_stride, scale, stream);
}

int rt_attn_prefill_bf16(const void* q, const void* k, const void* v, void* out, float* lse, int64_t batch,
                         int64_t heads, int64_t seq, int dim, int mask_flags, const int32_t* kv_lens,
                         const uint8_t* key_keep, int64_t keep_batch_stride, float scale, void* stream) {
    if (batch > 0 && heads > 0 && seq > 0 && dim > 0 && (!k || !v)) return RT_ERR_NULL_POINTER;
    return rt_attn_prefill_gqa_bf16(q, k, v, out, lse, batch, heads, heads > 0 ? heads : 1, seq, seq, dim, mask_flags,
                                    kv_lens, nullptr, key_keep, keep_batch_stride, scale, stream);
}

int rt_attn_prefill_f32(const float* q, const float* k, const float* v, float* out, float* lse, int64_t batch,
                        int64_t heads_q, int64_t heads_kv, int64_t seq_q, int64_t seq_kv, int dim, int mask_flags,
                        const int32_t* kv_lens, const int32_t* q_offsets, const uint8_t* key_keep,
                        int64_t keep_batch_stride, float scale, void* stream) {
    if (dim == 0) return RT_ERR_ZERO_DIM;
    if (batch < 0 || heads_q < 0 || heads_kv < 0 || seq_q < 0 || seq_kv < 0 || dim < 0) return RT_ERR_BAD_LENGTH;
    if (heads_kv == 0 || heads_q % heads_kv != 0) return heads_q == 0 ? RT_OK : RT_ERR_HEAD_COUNT;
    if (batch == 0 || heads_q == 0 || seq_q == 0) return RT_OK;
    if (!q || !out || (seq_kv > 0 && (!k || !v))) return RT_ERR_NULL_POINTER;
    if (dim > 256) return RT_ERR_UNSUPPORTED;
    if (mask_flags & ~RT_MASK_CAUSAL) return RT_ERR_UNSUPPORTED;
    RT_CUDA(rt::launch_prefill_f32(q, k, v, out, lse, batch, heads_q, heads_kv, seq_q, seq_kv, dim,
                                   mask_flags & RT_MASK_CAUSAL, kv_lens, q_offsets, key_keep, keep_batch_stride,
                                   default_scale(scale, dim), as_stream(stream)));
    return RT_OK;
}

// How a host call is cut into (batch element, head range) chunks for the three-stream pipeline.  The
// upload is the long pole (three tensors in, one out) and the last chunk's kernel and download cannot hide
// behind an upload, so the list starts with a few large chunks (few copies, each near the PCIe rate) and
// ends by halving: ..., n/2, n/4, ... down to ~8 MB of upload (0.15 ms; below that the per-chunk launches cost more).  Each download stays shorter than the next
// chunk's upload, and the exposed tail shrinks from a quarter of the call to a few tens of microseconds.
struct HostChunk {
    int64_t b0, nb, h0, h1;  // batch elements [b0, b0 + nb), heads [h0, h1)
};
constexpr int kMaxHostChunks = 32;
static int plan_host_chunks(int64_t batch, int64_t heads, size_t unit_upload_bytes, HostChunk* out) {
    constexpr int kTail = 8;  // entries kept for the halving tail
    // A small call (under 32 MB of upload, ~0.6 ms) runs as one chunk: its kernels would not fill the GPU
    // chunk by chunk, and four sets of copies and launches cost more than the overlap returns.
    if ((size_t)batch * (size_t)heads * unit_upload_bytes < (size_t(32) << 20)) {
        out[0] = HostChunk{0, batch, 0, heads};
        return 1;
    }
    int64_t per_batch = (4 + batch - 1) / batch;
    if (per_batch > heads) per_batch = heads;
    int64_t batch_step = 1;  // batch elements per chunk
    if (batch * per_batch > kMaxHostChunks - kTail) {
        per_batch = 1;
        batch_step = (batch + (kMaxHostChunks - kTail) - 1) / (kMaxHostChunks - kTail);
    }
    int n = 0;
    for (int64_t b0 = 0; b0 < batch; b0 += batch_step) {
        const int64_t nb = (b0 + batch_step <= batch) ? batch_step : batch - b0;
        for (int64_t part = 0; part < per_batch; ++part)
            out[n++] = HostChunk{b0, nb, heads * part / per_batch, heads * (part + 1) / per_batch};
    }
    HostChunk last = out[n - 1];
    if (last.nb == 1) {
        --n;
        while (last.h1 - last.h0 > 1 && n < kMaxHostChunks - 1 &&
               (size_t)(last.h1 - last.h0) * unit_upload_bytes > (size_t(8) << 20)) {
            const int64_t take = (last.h1 - last.h0 + 1) / 2;
            out[n++] = HostChunk{last.b0, 1, last.h0, last.h0 + take};
            last.h0 += take;
        }
        out[n++] = last;
    }
    return n;
}


// Streams and events of the pipelined host entry, created once per device.
namespace {
struct HostPipeline {
    static constexpr int kMaxChunks = kMaxHostChunks;
    cudaStream_t in[64] = {}, comp[64] = {}, out[64] = {};
    cudaEvent_t ev_in[64][kMaxChunks] = {}, ev_comp[64][kMaxChunks] = {};
    bool ready[64] = {};
    cudaError_t init(int dev) {
        if (ready[dev]) return cudaSuccess;
        cudaError_t e;
        if ((e = cudaStreamCreateWithFlags(&in[dev], cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&comp[dev], cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&out[dev], cudaStreamNonBlocking)) != cudaSuccess) return e;
        for (int i = 0; i < kMaxChunks; ++i) {
            if ((e = cudaEventCreateWithFlags(&ev_in[dev][i], cudaEventDisableTiming)) != cudaSuccess) return e;
            if ((e = cudaEventCreateWithFlags(&ev_comp[dev][i], cudaEventDisableTiming)) != cudaSuccess) return e;
        }
        ready[dev] = true;
        return cudaSuccess;
    }
};
HostPipeline g_pipe;
}  // namespace

// flash_forward / flash_forward_masked on host f32 slices (cpu_forward.rs:175-242).  The (batch, head
// range) chunks run through three streams: upload of chunk c+1, conversion + kernel of chunk c and
// download of chunk c-1 overlap (fully with pinned host memory; with pageable memory the driver
// stages the copies, and the kernels still overlap them).
int rt_flash_forward_f32_host(const float* q, size_t q_len, const float* k, size_t k_len, const float* v,
                              size_t v_len, float* out, size_t out_len, int64_t batch, int64_t heads, int64_t seq,
                              int64_t dim, int mask_kind, const uint8_t* keep, size_t keep_len, int precision) {
    // validate(): cpu_forward.rs:142-169
    if (dim == 0) return RT_ERR_ZERO_DIM;
    if (batch < 0 || heads < 0 || seq < 0 || dim < 0) return RT_ERR_BAD_LENGTH;
    const size_t expected = (size_t)batch * (size_t)heads * (size_t)seq * (size_t)dim;
    if (q_len != expected || k_len != expected || v_len != expected) return RT_ERR_BUFFER_SHAPE;
    if (out_len != expected) return RT_ERR_OUTPUT_SHAPE;
    // Mask::validate: mask.rs:51-65
    if (mask_kind < RT_MASKKIND_NONE || mask_kind > RT_MASKKIND_PADDING) return RT_ERR_UNSUPPORTED;
    if (mask_kind == RT_MASKKIND_PADDING && keep_len != (size_t)seq) return RT_ERR_MASK_LEN;
    if (seq == 0 || expected == 0) return RT_OK;
    if (!q || !k || !v || !out) return RT_ERR_NULL_POINTER;
    if (mask_kind == RT_MASKKIND_PADDING && !keep) return RT_ERR_NULL_POINTER;
    if (precision != RT_PRECISION_F32 && precision != RT_PRECISION_BF16) return RT_ERR_UNSUPPORTED;
    if (precision == RT_PRECISION_BF16 && dim != 64 && dim != 128) return RT_ERR_UNSUPPORTED;
    if (precision == RT_PRECISION_F32 && dim > 256) return RT_ERR_UNSUPPORTED;

    const size_t bytes = expected * sizeof(float);
    std::lock_guard<std::mutex> lock(g_staging.mu);
    int dev = 0;
    RT_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return RT_ERR_UNSUPPORTED;
    RT_CUDA(g_pipe.init(dev));
    cudaStream_t s_in = g_pipe.in[dev], s_comp = g_pipe.comp[dev], s_out = g_pipe.out[dev];
    DevBuf dq(0), dk(1), dv(2), dout(3), dkeep(4), bq(5), bk(6), bv(7), bo(8);
    RT_CUDA(dq.alloc(bytes));
    RT_CUDA(dk.alloc(bytes));
    RT_CUDA(dv.alloc(bytes));
    RT_CUDA(dout.alloc(bytes));
    const bool bf16 = precision == RT_PRECISION_BF16;
    if (bf16) {
        RT_CUDA(bq.alloc(expected * 2));
        RT_CUDA(bk.alloc(expected * 2));
        RT_CUDA(bv.alloc(expected * 2));
        RT_CUDA(bo.alloc(expected * 2));
    }
    const uint8_t* keep_dev = nullptr;
    if (mask_kind == RT_MASKKIND_PADDING) {
        RT_CUDA(dkeep.alloc(keep_len));
        RT_CUDA(cudaMemcpyAsync(dkeep.p, keep, keep_len, cudaMemcpyHostToDevice, s_in));
        keep_dev = dkeep.as<uint8_t>();
    }
    const int flags = (mask_kind == RT_MASKKIND_CAUSAL) ? RT_MASK_CAUSAL : RT_MASK_NONE;
    const size_t slab = (size_t)seq * (size_t)dim;  // elements of one (b,h)
    HostChunk plan[kMaxHostChunks];
    const int n_chunks = plan_host_chunks(batch, heads, 3 * slab * sizeof(float), plan);
    for (int c = 0; c < n_chunks; ++c) {
        {
            const int64_t b0 = plan[c].b0, nb = plan[c].nb, h0 = plan[c].h0, h1 = plan[c].h1;
            // a chunk of several batch elements holds all their heads (h0 = 0, h1 = heads)
            const size_t off = ((size_t)b0 * heads + h0) * slab, cnt = (size_t)nb * (size_t)(h1 - h0) * slab;
            RT_CUDA(cudaMemcpyAsync(dq.as<float>() + off, q + off, cnt * 4, cudaMemcpyHostToDevice, s_in));
            RT_CUDA(cudaMemcpyAsync(dk.as<float>() + off, k + off, cnt * 4, cudaMemcpyHostToDevice, s_in));
            RT_CUDA(cudaMemcpyAsync(dv.as<float>() + off, v + off, cnt * 4, cudaMemcpyHostToDevice, s_in));
            RT_CUDA(cudaEventRecord(g_pipe.ev_in[dev][c], s_in));
            RT_CUDA(cudaStreamWaitEvent(s_comp, g_pipe.ev_in[dev][c], 0));
            int rc;
            if (bf16) {
                RT_CUDA(rt::launch_f32_to_bf16(dq.as<float>() + off, bq.as<char>() + off * 2, (int64_t)cnt, s_comp));
                RT_CUDA(rt::launch_f32_to_bf16(dk.as<float>() + off, bk.as<char>() + off * 2, (int64_t)cnt, s_comp));
                RT_CUDA(rt::launch_f32_to_bf16(dv.as<float>() + off, bv.as<char>() + off * 2, (int64_t)cnt, s_comp));
                rc = rt_attn_prefill_bf16(bq.as<char>() + off * 2, bk.as<char>() + off * 2, bv.as<char>() + off * 2,
                                          bo.as<char>() + off * 2, nullptr, nb, h1 - h0, seq, (int)dim, flags, nullptr,
                                          keep_dev, 0, -1.f, s_comp);
                if (rc == RT_OK)
                    RT_CUDA(rt::launch_bf16_to_f32(bo.as<char>() + off * 2, dout.as<float>() + off, (int64_t)cnt, s_comp));
            } else {
                rc = rt_attn_prefill_f32(dq.as<float>() + off, dk.as<float>() + off, dv.as<float>() + off,
                                         dout.as<float>() + off, nullptr, nb, h1 - h0, h1 - h0, seq, seq, (int)dim, flags,
                                         nullptr, nullptr, keep_dev, 0, -1.f, s_comp);
            }
            if (rc != RT_OK) {
                cudaDeviceSynchronize();
                return rc;
            }
            RT_CUDA(cudaEventRecord(g_pipe.ev_comp[dev][c], s_comp));
            RT_CUDA(cudaStreamWaitEvent(s_out, g_pipe.ev_comp[dev][c], 0));
            RT_CUDA(cudaMemcpyAsync(out + off, dout.as<float>() + off, cnt * 4, cudaMemcpyDeviceToHost, s_out));
        }
    }
    RT_CUDA(cudaStreamSynchronize(s_out));
    RT_CUDA(cudaStreamSynchronize(s_comp));
    RT_CUDA(cudaStreamSynchronize(s_in));
    return RT_OK;
}

// The (b, head-range) chunks run through three streams (copy in, kernel, copy out), so the upload
// of chunk c+1, the kernel of chunk c and the download of chunk c-1 overlap; with pinned host
// memory the call is bounded by the slower PCIe direction instead of the sum of both.
int rt_attn_prefill_bf16_host(const void* q, const void* k, const void* v, void* out, float* lse, int64_t batch,
                              int64_t heads, int64_t seq, int dim, int mask_flags, const int32_t* kv_lens,
                              float scale) {
    if (dim == 0) return RT_ERR_ZERO_DIM;
    if (batch < 0 || heads < 0 || seq < 0 || dim < 0) return RT_ERR_BAD_LENGTH;
    const size_t n = (size_t)batch * heads * seq * dim;
    if (n == 0) return RT_OK;
    if (!q || !k || !v || !out) return RT_ERR_NULL_POINTER;
    if (dim != 64 && dim != 128) return RT_ERR_UNSUPPORTED;
    if (mask_flags & ~RT_MASK_CAUSAL) return RT_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_staging.mu);
    int dev = 0;
    RT_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return RT_ERR_UNSUPPORTED;
    RT_CUDA(g_pipe.init(dev));
    DevBuf dq(0), dk(1), dv(2), dout(3), dlse(4), dlens(5);
    RT_CUDA(dq.alloc(n * 2));
    RT_CUDA(dk.alloc(n * 2));
    RT_CUDA(dv.alloc(n * 2));
    RT_CUDA(dout.alloc(n * 2));
    const size_t rows = (size_t)batch * heads * seq;
    if (lse) RT_CUDA(dlse.alloc(rows * 4));
    cudaStream_t s_in = g_pipe.in[dev], s_comp = g_pipe.comp[dev], s_out = g_pipe.out[dev];
    if (kv_lens) {
        RT_CUDA(dlens.alloc((size_t)batch * 4));
        RT_CUDA(cudaMemcpyAsync(dlens.p, kv_lens, (size_t)batch * 4, cudaMemcpyHostToDevice, s_in));
    }
    const size_t slab = (size_t)seq * dim;  // elements of one (b,h)
    HostChunk plan[kMaxHostChunks];
    // per-batch kv_lens are passed by offset, so a chunk must stay inside one batch element
    const int n_chunks = batch <= kMaxHostChunks - 8 ? plan_host_chunks(batch, heads, 3 * slab * 2, plan) : 0;
    if (n_chunks == 0 || plan[0].nb != 1) {  // very large batch: run unpipelined
        RT_CUDA(cudaMemcpyAsync(dq.p, q, n * 2, cudaMemcpyHostToDevice, s_in));
        RT_CUDA(cudaMemcpyAsync(dk.p, k, n * 2, cudaMemcpyHostToDevice, s_in));
        RT_CUDA(cudaMemcpyAsync(dv.p, v, n * 2, cudaMemcpyHostToDevice, s_in));
        int rc = rt_attn_prefill_bf16(dq.p, dk.p, dv.p, dout.p, lse ? dlse.as<float>() : nullptr, batch, heads, seq,
                                      dim, mask_flags, kv_lens ? dlens.as<int32_t>() : nullptr, nullptr, 0, scale, s_in);
        if (rc != RT_OK) return rc;
        RT_CUDA(cudaMemcpyAsync(out, dout.p, n * 2, cudaMemcpyDeviceToHost, s_in));
        if (lse) RT_CUDA(cudaMemcpyAsync(lse, dlse.p, rows * 4, cudaMemcpyDeviceToHost, s_in));
        RT_CUDA(cudaStreamSynchronize(s_in));
        return RT_OK;
    }
    for (int c = 0; c < n_chunks; ++c) {
        {
            const int64_t b = plan[c].b0, h0 = plan[c].h0, h1 = plan[c].h1;
            const size_t off = ((size_t)b * heads + h0) * slab, cnt = (size_t)(h1 - h0) * slab;
            const size_t roff = ((size_t)b * heads + h0) * seq, rcnt = (size_t)(h1 - h0) * seq;
            const char* hq = (const char*)q + off * 2;
            const char* hk = (const char*)k + off * 2;
            const char* hv = (const char*)v + off * 2;
            RT_CUDA(cudaMemcpyAsync(dq.as<char>() + off * 2, hq, cnt * 2, cudaMemcpyHostToDevice, s_in));
            RT_CUDA(cudaMemcpyAsync(dk.as<char>() + off * 2, hk, cnt * 2, cudaMemcpyHostToDevice, s_in));
            RT_CUDA(cudaMemcpyAsync(dv.as<char>() + off * 2, hv, cnt * 2, cudaMemcpyHostToDevice, s_in));
            RT_CUDA(cudaEventRecord(g_pipe.ev_in[dev][c], s_in));
            RT_CUDA(cudaStreamWaitEvent(s_comp, g_pipe.ev_in[dev][c], 0));
            int rc = rt_attn_prefill_bf16(dq.as<char>() + off * 2, dk.as<char>() + off * 2, dv.as<char>() + off * 2,
                                          dout.as<char>() + off * 2, lse ? dlse.as<float>() + roff : nullptr, 1, h1 - h0,
                                          seq, dim, mask_flags, kv_lens ? dlens.as<int32_t>() + b : nullptr, nullptr, 0,
                                          scale, s_comp);
            if (rc != RT_OK) {
                cudaDeviceSynchronize();
                return rc;
            }
            RT_CUDA(cudaEventRecord(g_pipe.ev_comp[dev][c], s_comp));
            RT_CUDA(cudaStreamWaitEvent(s_out, g_pipe.ev_comp[dev][c], 0));
            RT_CUDA(cudaMemcpyAsync((char*)out + off * 2, dout.as<char>() + off * 2, cnt * 2, cudaMemcpyDeviceToHost,
                                    s_out));
            if (lse) RT_CUDA(cudaMemcpyAsync(lse + roff, dlse.as<float>() + roff, rcnt * 4, cudaMemcpyDeviceToHost, s_out));
        }
    }
    RT_CUDA(cudaStreamSynchronize(s_out));
    RT_CUDA(cudaStreamSynchronize(s_comp));
    return RT_OK;
}

// ------------------------------------------------------------------------------ backward

size_t rt_attn_backward_workspace_bytes(int64_t batch, int64_t heads, int64_t seq) {
    if (batch <= 0 || heads <= 0 || seq <= 0) return 0;
    return (size_t)batch * (size_t)heads * (size_t)seq * sizeof(float);
}

int rt_attn_backward_f32(const float* q, const float* k, const float* v, const float* out, const float* d_out,
                         const float* lse, float* dq, float* dk, float* dv, int64_t batch, int64_t heads, int64_t seq,
                         int dim, int mask_flags, float scale, void* workspace, size_t workspace_bytes, void* stream) {
    if (dim == 0) return RT_ERR_ZERO_DIM;
    if (batch < 0 || heads < 0 || seq < 0 || dim < 0) return RT_ERR_BAD_LENGTH;
    if (batch == 0 || heads == 0 || seq == 0) return RT_OK;  // cpu_backward.rs:74-76
    if (!q || !k || !v || !out || !d_out || !lse || !dq || !dk || !dv) return RT_ERR_NULL_POINTER;
    if (dim > 256 || batch * heads > 65535) return RT_ERR_UNSUPPORTED;
    if (mask_flags & ~RT_MASK_CAUSAL) return RT_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < rt_attn_backward_workspace_bytes(batch, heads, seq)) return RT_ERR_WORKSPACE;
    RT_CUDA(rt::launch_backward_f32(q, k, v, out, d_out, lse, dq, dk, dv, static_cast<float*>(workspace), batch, heads,
                                    seq, dim, mask_flags & RT_MASK_CAUSAL, default_scale(scale, dim),
                                    as_stream(stream)));
    return RT_OK;
}

int rt_attn_backward_bf16(const void* q, const void* k, const void* v, const void* out, const void* d_out,
                          const float* lse, float* dq, float* dk, float* dv, int64_t batch, int64_t heads, int64_t seq,
                          int dim, int mask_flags, float scale, void* workspace, size_t workspace_bytes, void* stream) {
    if (dim == 0) return RT_ERR_ZERO_DIM;
    if (batch < 0 || heads < 0 || seq < 0 || dim < 0) return RT_ERR_BAD_LENGTH;
    if (batch == 0 || heads == 0 || seq == 0) return RT_OK;
    if (!q || !k || !v || !out || !d_out || !lse || !dq || !dk || !dv) return RT_ERR_NULL_POINTER;
    if ((dim != 64 && dim != 128) || batch * heads > 65535) return RT_ERR_UNSUPPORTED;
    if (mask_flags & ~RT_MASK_CAUSAL) return RT_ERR_UNSUPPORTED;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(d_out) || !aligned16(out)) return RT_ERR_ALIGNMENT;
    if (!workspace || workspace_bytes < rt_attn_backward_workspace_bytes(batch, heads, seq)) return RT_ERR_WORKSPACE;
    RT_CUDA(rt::launch_backward_bf16(q, k, v, out, d_out, lse, dq, dk, dv, static_cast<float*>(workspace), batch, heads,
                                     seq, dim, mask_flags & RT_MASK_CAUSAL, default_scale(scale, dim),
                                     as_stream(stream)));
    return RT_OK;
}

int rt_flash_backward_f32_host(const float* q, size_t q_len, const float* k, size_t k_len, const float* v,
                               size_t v_len, const float* d_out, size_t d_out_len, float* dq, size_t dq_len, float* dk,
                               size_t dk_len, float* dv, size_t dv_len, int64_t batch, int64_t heads, int64_t seq,
                               int64_t dim, int mask_kind) {
    // flash_backward has no dim check of its own: with dim = 0 every length is 0 and the call is a no-op
    if (batch < 0 || heads < 0 || seq < 0 || dim < 0) return RT_ERR_BAD_LENGTH;
    const size_t expected = (size_t)batch * (size_t)heads * (size_t)seq * (size_t)dim;
    // cpu_backward.rs:57-73: inputs first (q, k, v, do), then the three outputs
    if (q_len != expected || k_len != expected || v_len != expected || d_out_len != expected)
        return RT_ERR_BUFFER_SHAPE;
    if (dq_len != expected || dk_len != expected || dv_len != expected) return RT_ERR_OUTPUT_SHAPE;
    if (mask_kind != RT_MASKKIND_NONE && mask_kind != RT_MASKKIND_CAUSAL) return RT_ERR_UNSUPPORTED;
    if (seq == 0 || expected == 0) return RT_OK;  // :74-76
    if (!q || !k || !v || !d_out || !dq || !dk || !dv) return RT_ERR_NULL_POINTER;
    if (dim > 256 || batch * heads > 65535) return RT_ERR_UNSUPPORTED;

    const size_t bytes = expected * sizeof(float);
    const size_t stat_bytes = rt_attn_backward_workspace_bytes(batch, heads, seq);
    std::lock_guard<std::mutex> lock(g_staging.mu);
    DevBuf bq(0), bk(1), bv(2), bo(3), bdo(4), blse(5), bdelta(6), bdq(7), bdk(8), bdv(9);
    RT_CUDA(bq.alloc(bytes));
    RT_CUDA(bk.alloc(bytes));
    RT_CUDA(bv.alloc(bytes));
    RT_CUDA(bo.alloc(bytes));
    RT_CUDA(bdo.alloc(bytes));
    RT_CUDA(blse.alloc(stat_bytes));
    RT_CUDA(bdelta.alloc(stat_bytes));
    RT_CUDA(bdq.alloc(bytes));
    RT_CUDA(bdk.alloc(bytes));
    RT_CUDA(bdv.alloc(bytes));
    RT_CUDA(cudaMemcpy(bq.p, q, bytes, cudaMemcpyHostToDevice));
    RT_CUDA(cudaMemcpy(bk.p, k, bytes, cudaMemcpyHostToDevice));
    RT_CUDA(cudaMemcpy(bv.p, v, bytes, cudaMemcpyHostToDevice));
    RT_CUDA(cudaMemcpy(bdo.p, d_out, bytes, cudaMemcpyHostToDevice));
    const int flags = (mask_kind == RT_MASKKIND_CAUSAL) ? RT_MASK_CAUSAL : RT_MASK_NONE;
    // the reference recomputes the probabilities from Q and K (:96-127); here the forward pass supplies
    // O and the row statistics that the tiled backward consumes
    int rc = rt_attn_prefill_f32(bq.as<float>(), bk.as<float>(), bv.as<float>(), bo.as<float>(), blse.as<float>(),
                                 batch, heads, heads, seq, seq, (int)dim, flags, nullptr, nullptr, nullptr, 0, -1.f,
                                 nullptr);
    if (rc != RT_OK) return rc;
    rc = rt_attn_backward_f32(bq.as<float>(), bk.as<float>(), bv.as<float>(), bo.as<float>(), bdo.as<float>(),
                              blse.as<float>(), bdq.as<float>(), bdk.as<float>(), bdv.as<float>(), batch, heads, seq,
                              (int)dim, flags, -1.f, bdelta.p, stat_bytes, nullptr);
    if (rc != RT_OK) return rc;
    RT_CUDA(cudaMemcpy(dq, bdq.p, bytes, cudaMemcpyDeviceToHost));
    RT_CUDA(cudaMemcpy(dk, bdk.p, bytes, cudaMemcpyDeviceToHost));
    RT_CUDA(cudaMemcpy(dv, bdv.p, bytes, cudaMemcpyDeviceToHost));
    return RT_OK;
}

// ------------------------------------------------------------------------------ decode

size_t rt_gqa_decode_workspace_bytes(int64_t batch, int64_t n_heads, int64_t n_kv_heads, int head_dim,
                                     int64_t max_seq) {
    if (batch <= 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || max_seq <= 0) return 0;
    const size_t chunks = (size_t)rt::decode_num_chunks(batch, (int)n_kv_heads, max_seq);
    if (chunks <= 1) return 0;
    // chunk partials (O | LSE) followed by one completion counter per (sequence, KV head)
    return chunks * (size_t)batch * (size_t)n_heads * ((size_t)head_dim + 1) * sizeof(float) +
           (((size_t)batch * (size_t)n_kv_heads * sizeof(int) + 15) & ~(size_t)15);
}

// Shared validation + launch of the decode entries; of_stride / lse_stride are the row pitches (in
// floats) of out_f32 / lse (0 = dense).
static int decode_common(const void* q, const void* k_cache, const void* v_cache, void* out_bf16, float* out_f32,
                         float* lse, int64_t of_stride, int64_t lse_stride, int64_t batch, int64_t n_heads,
                         int64_t n_kv_heads, int head_dim, int64_t max_seq, const int32_t* kv_lens,
                         int64_t kv_len_uniform, int64_t kv_begin, int64_t kv_end, float scale, void* workspace,
                         size_t workspace_bytes, void* stream, const rt::MergePush* push = nullptr,
                         bool* pushed = nullptr, rt::DecodeTail* tail = nullptr) {
    if (pushed) *pushed = false;
    if (n_kv_heads <= 0 || n_heads <= 0 || n_heads % n_kv_heads != 0) return RT_ERR_HEAD_COUNT;  // gqa.rs:106-111
    if (head_dim == 0) return RT_ERR_ZERO_DIM;
    if (batch < 0 || max_seq <= 0 || kv_begin < 0 || head_dim < 0) return RT_ERR_BAD_LENGTH;
    if (!kv_lens && (kv_len_uniform < 0 || kv_len_uniform > max_seq)) return RT_ERR_BAD_LENGTH;
    if (batch == 0) return RT_OK;
    if (!q || !k_cache || !v_cache || (!out_bf16 && !out_f32)) return RT_ERR_NULL_POINTER;
    const int64_t group = n_heads / n_kv_heads;
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return RT_ERR_UNSUPPORTED;
    if (group != 1 && group != 2 && group != 4 && group != 8) return RT_ERR_UNSUPPORTED;
    if (batch > 65535 || n_kv_heads > 65535) return RT_ERR_UNSUPPORTED;
    if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache)) return RT_ERR_ALIGNMENT;
    const size_t need = rt_gqa_decode_workspace_bytes(batch, n_heads, n_kv_heads, head_dim, max_seq);
    if (need > 0 && (!workspace || workspace_bytes < need)) return RT_ERR_WORKSPACE;
    // Everything that could fail after the decode kernel is enqueued is checked here instead: the chunk merge
    // keeps one weight per chunk in shared memory, and a record delivered to peers travels in 16-byte pieces.
    if (!rt::merge_fits((int64_t)rt::decode_num_chunks(batch, (int)n_kv_heads, max_seq), head_dim))
        return RT_ERR_UNSUPPORTED;
    if (push && ((batch * n_heads * ((int64_t)head_dim + 1)) & 3)) return RT_ERR_ALIGNMENT;
    RT_CUDA(rt::launch_gqa_decode(q, k_cache, v_cache, out_bf16, out_f32, lse, batch, (int)n_heads, (int)n_kv_heads,
                                  head_dim, max_seq, kv_lens, kv_len_uniform, kv_begin, kv_end,
                                  default_scale(scale, head_dim), need ? workspace : nullptr, of_stride, lse_stride,
                                  as_stream(stream), push, pushed, tail));
    return RT_OK;
}

int rt_gqa_decode_bf16(const void* q, const void* k_cache, const void* v_cache, void* out_bf16, float* out_f32,
                       float* lse, int64_t batch, int64_t n_heads, int64_t n_kv_heads, int head_dim, int64_t max_seq,
                       const int32_t* kv_lens, int64_t kv_len_uniform, int64_t kv_begin, int64_t kv_end, float scale,
                       void* workspace, size_t workspace_bytes, void* stream) {
    return decode_common(q, k_cache, v_cache, out_bf16, out_f32, lse, 0, 0, batch, n_heads, n_kv_heads, head_dim,
                         max_seq, kv_lens, kv_len_uniform, kv_begin, kv_end, scale, workspace, workspace_bytes, stream);
}

int rt_gqa_decode_record_bf16(const void* q, const void* k_cache, const void* v_cache, float* record, int64_t batch,
                              int64_t n_heads, int64_t n_kv_heads, int head_dim, int64_t max_seq,
                              const int32_t* kv_lens, int64_t kv_len_uniform, int64_t kv_begin, int64_t kv_end,
                              float scale, void* workspace, size_t workspace_bytes, void* stream) {
    if (batch > 0 && !record) return RT_ERR_NULL_POINTER;
    return decode_common(q, k_cache, v_cache, nullptr, record, record ? record + head_dim : nullptr, head_dim + 1,
                         head_dim + 1, batch, n_heads, n_kv_heads, head_dim, max_seq, kv_lens, kv_len_uniform, kv_begin,
                         kv_end, scale, workspace, workspace_bytes, stream);
}

int rt_gqa_decode_record_push_bf16(const void* q, const void* k_cache, const void* v_cache, float* record,
                                   void* const* peer_slots, void* const* peer_flags, int world, uint32_t epoch,
                                   int* done_counter, int64_t batch, int64_t n_heads, int64_t n_kv_heads, int head_dim,
                                   int64_t max_seq, const int32_t* kv_lens, int64_t kv_len_uniform, int64_t kv_begin,
                                   int64_t kv_end, float scale, void* workspace, size_t workspace_bytes, void* stream) {
    if (world <= 0) return RT_ERR_BAD_LENGTH;
    if (world > rt::kMaxPeers) return RT_ERR_UNSUPPORTED;
    if ((batch > 0 && !record) || !peer_slots || !peer_flags || !done_counter) return RT_ERR_NULL_POINTER;
    rt::MergePush push{};
    for (int r = 0; r < world; ++r) {
        if (!peer_slots[r] || !peer_flags[r]) return RT_ERR_NULL_POINTER;
        if (!aligned16(peer_slots[r])) return RT_ERR_ALIGNMENT;
        push.dst[r] = static_cast<float*>(peer_slots[r]);
        push.flag[r] = static_cast<uint32_t*>(peer_flags[r]);
    }
    push.world = world;
    push.epoch = epoch;
    push.done_counter = done_counter;
    bool pushed = false;
    const int rc = decode_common(q, k_cache, v_cache, nullptr, record, record ? record + head_dim : nullptr,
                                 head_dim + 1, head_dim + 1, batch, n_heads, n_kv_heads, head_dim, max_seq, kv_lens,
                                 kv_len_uniform, kv_begin, kv_end, scale, workspace, workspace_bytes, stream, &push,
                                 &pushed);
    if (rc != RT_OK || pushed || batch == 0) return rc;
    // the record came straight out of the decode kernel (one chunk, or chunks merged in-kernel): copy it over
    return rt_splitkv_push_record(record, peer_slots, peer_flags, world, batch * n_heads, head_dim, epoch, stream);
}

int rt_gqa_decode_online_bf16(const void* q, const void* k_cache, const void* v_cache, void* out, int n_heads,
                              int n_kv, int kv_len, int head_dim, int max_seq, void* workspace,
                              size_t workspace_bytes, void* stream) {
    return rt_gqa_decode_bf16(q, k_cache, v_cache, out, nullptr, nullptr, 1, n_heads, n_kv, head_dim, max_seq, nullptr,
                              kv_len, 0, -1, -1.f, workspace, workspace_bytes, stream);
}

int rt_attn_merge_partials(const float* o_parts, const float* lse_parts, int64_t n_parts, int64_t rows, int dim,
                           void* out_bf16, float* out_f32, float* lse, void* stream) {
    if (dim == 0) return RT_ERR_ZERO_DIM;
    if (n_parts < 0 || rows < 0 || dim < 0 || n_parts > 0x7fffffff) return RT_ERR_BAD_LENGTH;
    if (dim > 256 || n_parts > 8192) return RT_ERR_UNSUPPORTED;
    if (rows == 0) return RT_OK;
    if ((n_parts > 0 && (!o_parts || !lse_parts)) || (!out_bf16 && !out_f32)) return RT_ERR_NULL_POINTER;
    RT_CUDA(rt::launch_merge_partials(o_parts, lse_parts, n_parts, rows, dim, dim, 1, out_bf16, out_f32, lse,
                                      as_stream(stream)));
    return RT_OK;
}

int rt_attn_merge_records(const float* records, int64_t n_parts, int64_t rows, int dim, void* out_bf16,
                          float* out_f32, float* lse, void* stream) {
    if (dim == 0) return RT_ERR_ZERO_DIM;
    if (n_parts < 0 || rows < 0 || dim < 0 || n_parts > 0x7fffffff) return RT_ERR_BAD_LENGTH;
    if (dim > 256 || n_parts > 8192) return RT_ERR_UNSUPPORTED;
    if (rows == 0) return RT_OK;
    if ((n_parts > 0 && !records) || (!out_bf16 && !out_f32)) return RT_ERR_NULL_POINTER;
    RT_CUDA(rt::launch_merge_partials(records, records + dim, n_parts, rows, dim, dim + 1, dim + 1, out_bf16, out_f32,
                                      lse, as_stream(stream)));
    return RT_OK;
}

int rt_splitkv_push_record(const float* record, void* const* peer_slots, void* const* peer_flags, int world,
                           int64_t rows, int dim, uint32_t epoch, void* stream) {
    if (dim == 0) return RT_ERR_ZERO_DIM;
    if (world <= 0 || rows < 0 || dim < 0) return RT_ERR_BAD_LENGTH;
    if (world > rt::kMaxPeers || dim > 256) return RT_ERR_UNSUPPORTED;
    if (rows == 0) return RT_OK;
    if (!record || !peer_slots || !peer_flags) return RT_ERR_NULL_POINTER;
    const int64_t n = rows * (dim + 1);
    if (n & 3) return RT_ERR_ALIGNMENT;  // the record is copied in 16-byte pieces
    for (int r = 0; r < world; ++r) {
        if (!peer_slots[r] || !peer_flags[r]) return RT_ERR_NULL_POINTER;
        if (!aligned16(peer_slots[r])) return RT_ERR_ALIGNMENT;
    }
    if (!aligned16(record)) return RT_ERR_ALIGNMENT;
    RT_CUDA(rt::launch_push_records(record, peer_slots, peer_flags, world, n, epoch, as_stream(stream)));
    return RT_OK;
}

int rt_attn_merge_records_after(const float* records, const uint32_t* flags, uint32_t epoch, int64_t wait_clocks,
                                int64_t n_parts, int64_t rows, int dim, void* out_bf16, float* out_f32, float* lse,
                                void* stream) {
    if (dim == 0) return RT_ERR_ZERO_DIM;
    if (n_parts <= 0 || rows < 0 || dim < 0) return RT_ERR_BAD_LENGTH;
    if (dim > 256 || n_parts > rt::kMaxPeers) return RT_ERR_UNSUPPORTED;
    if (rows == 0) return RT_OK;
    if (!records || !flags || (!out_bf16 && !out_f32)) return RT_ERR_NULL_POINTER;
    rt::MergeWait w{flags, (int)n_parts, epoch, wait_clocks > 0 ? (long long)wait_clocks : (1ll << 31),
                    rt::device_status_ptr(), 0};
    if (!w.status) return (int)cudaErrorInvalidSymbol;
    RT_CUDA(rt::launch_merge_partials(records, records + dim, n_parts, rows, dim, dim + 1, dim + 1, out_bf16, out_f32,
                                      lse, as_stream(stream), &w));
    return RT_OK;
}

int rt_gqa_decode_exchange_bf16(const void* q, const void* k_cache, const void* v_cache, void* out_bf16, float* out_f32,
                                float* lse, void* const* peer_slots, void* const* peer_flags, const float* local_slots,
                                const uint32_t* local_flags, int world, int rank, uint32_t epoch, int64_t wait_clocks,
                                int do_wait, int64_t batch, int64_t n_heads, int64_t n_kv_heads, int head_dim,
                                int64_t max_seq, const int32_t* kv_lens, int64_t kv_len_uniform, int64_t kv_begin,
                                int64_t kv_end, float scale, void* workspace, size_t workspace_bytes, void* stream) {
    if (world <= 0 || rank < 0 || rank >= world) return RT_ERR_BAD_LENGTH;
    if (world > rt::kMaxPeers) return RT_ERR_UNSUPPORTED;
    if (!peer_slots || !peer_flags || !local_slots || !local_flags) return RT_ERR_NULL_POINTER;
    for (int r = 0; r < world; ++r)
        if (!peer_slots[r] || !peer_flags[r]) return RT_ERR_NULL_POINTER;
    if (do_wait && !out_bf16 && !out_f32) return RT_ERR_NULL_POINTER;
    // The decode writes chunk partials (or, with a single chunk, the record itself into this rank's own
    // local slot); the row-exchange kernel merges, delivers, waits and merges again.
    float* self_slot = static_cast<float*>(peer_slots[rank]);
    rt::DecodeTail tail{0, nullptr, nullptr};
    const int rc = decode_common(q, k_cache, v_cache, nullptr, self_slot, self_slot + head_dim, head_dim + 1,
                                 head_dim + 1, batch, n_heads, n_kv_heads, head_dim, max_seq, kv_lens, kv_len_uniform,
                                 kv_begin, kv_end, scale, workspace, workspace_bytes, stream, nullptr, nullptr, &tail);
    if (rc != RT_OK || batch == 0) return rc;
    const int64_t rows = batch * n_heads;
    const bool direct = tail.n_chunks <= 1;
    RT_CUDA(rt::launch_row_exchange(direct ? self_slot : tail.part_o, direct ? self_slot + head_dim : tail.part_lse,
                                    direct ? 1 : tail.n_chunks, rows, head_dim, direct ? head_dim + 1 : head_dim,
                                    direct ? head_dim + 1 : 1, out_bf16, out_f32, lse, peer_slots, peer_flags,
                                    local_slots, local_flags, world, epoch, (long long)wait_clocks, do_wait,
                                    as_stream(stream)));
    return RT_OK;
}

int rt_gqa_decode_exchange_ll_bf16(const void* q, const void* k_cache, const void* v_cache, void* out_bf16,
                                   float* out_f32, float* lse, void* const* peer_words, const void* local_words,
                                   float* scratch_record, int world, int rank, uint32_t epoch, int64_t wait_clocks,
                                   int do_wait, int64_t batch, int64_t n_heads, int64_t n_kv_heads, int head_dim,
                                   int64_t max_seq, const int32_t* kv_lens, int64_t kv_len_uniform, int64_t kv_begin,
                                   int64_t kv_end, float scale, void* workspace, size_t workspace_bytes, void* stream) {
    if (world <= 0 || rank < 0 || rank >= world) return RT_ERR_BAD_LENGTH;
    if (world > rt::kMaxPeers) return RT_ERR_UNSUPPORTED;
    if (epoch == 0) return RT_ERR_BAD_LENGTH;  // zeroed words carry epoch 0
    if (head_dim > 255) return RT_ERR_UNSUPPORTED;  // one thread per word of a row (D + 1 <= 256); checked before any launch
    if (!peer_words || !local_words || !scratch_record) return RT_ERR_NULL_POINTER;
    for (int r = 0; r < world; ++r) {
        if (!peer_words[r]) return RT_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(peer_words[r]) & 7) return RT_ERR_ALIGNMENT;
    }
    if (reinterpret_cast<uintptr_t>(local_words) & 7) return RT_ERR_ALIGNMENT;
    if (do_wait && !out_bf16 && !out_f32) return RT_ERR_NULL_POINTER;
    // The decode writes chunk partials, or with a single chunk the f32 record itself into scratch_record;
    // the row-exchange kernel merges, delivers the words, waits for every rank's words and merges again.
    rt::DecodeTail tail{0, nullptr, nullptr};
    const int rc = decode_common(q, k_cache, v_cache, nullptr, scratch_record, scratch_record + head_dim, head_dim + 1,
                                 head_dim + 1, batch, n_heads, n_kv_heads, head_dim, max_seq, kv_lens, kv_len_uniform,
                                 kv_begin, kv_end, scale, workspace, workspace_bytes, stream, nullptr, nullptr, &tail);
    if (rc != RT_OK || batch == 0) return rc;
    const int64_t rows = batch * n_heads;
    const bool direct = tail.n_chunks <= 1;
    RT_CUDA(rt::launch_row_exchange_ll(direct ? scratch_record : tail.part_o,
                                       direct ? scratch_record + head_dim : tail.part_lse, direct ? 1 : tail.n_chunks,
                                       rows, head_dim, direct ? head_dim + 1 : head_dim, direct ? head_dim + 1 : 1,
                                       out_bf16, out_f32, lse, peer_words, local_words, world, epoch,
                                       (long long)wait_clocks, do_wait, as_stream(stream)));
    return RT_OK;
}

int rt_attn_merge_ll_rows(const void* local_words, uint32_t epoch, int64_t wait_clocks, int world, int64_t rows,
                          int dim, void* out_bf16, float* out_f32, float* lse, void* stream) {
    if (dim == 0) return RT_ERR_ZERO_DIM;
    if (world <= 0 || rows < 0 || dim < 0 || epoch == 0) return RT_ERR_BAD_LENGTH;
    if (dim > 255 || world > rt::kMaxPeers) return RT_ERR_UNSUPPORTED;
    if (rows == 0) return RT_OK;
    if (!local_words || (!out_bf16 && !out_f32)) return RT_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(local_words) & 7) return RT_ERR_ALIGNMENT;
    RT_CUDA(rt::launch_ll_merge(local_words, world, rows, dim, epoch, (long long)wait_clocks, out_bf16, out_f32, lse,
                                as_stream(stream)));
    return RT_OK;
}

int rt_attn_merge_records_after_rows(const float* records, const uint32_t* row_flags, uint32_t epoch,
                                     int64_t wait_clocks, int64_t n_parts, int64_t rows, int dim, void* out_bf16,
                                     float* out_f32, float* lse, void* stream) {
    if (dim == 0) return RT_ERR_ZERO_DIM;
    if (n_parts <= 0 || rows < 0 || dim < 0) return RT_ERR_BAD_LENGTH;
    if (dim > 256 || n_parts > rt::kMaxPeers) return RT_ERR_UNSUPPORTED;
    if (rows == 0) return RT_OK;
    if (!records || !row_flags || (!out_bf16 && !out_f32)) return RT_ERR_NULL_POINTER;
    rt::MergeWait w{row_flags, (int)n_parts, epoch, wait_clocks > 0 ? (long long)wait_clocks : (1ll << 31),
                    rt::device_status_ptr(), 1};
    if (!w.status) return (int)cudaErrorInvalidSymbol;
    RT_CUDA(rt::launch_merge_partials(records, records + dim, n_parts, rows, dim, dim + 1, dim + 1, out_bf16, out_f32,
                                      lse, as_stream(stream), &w));
    return RT_OK;
}

int rt_gqa_forward_f32_host(const float* q, size_t q_len, const float* k, size_t k_len, const float* v, size_t v_len,
                            float* out, size_t out_len, int64_t batch, int64_t n_heads, int64_t n_kv_heads,
                            int64_t seq_q, int64_t seq_kv, int64_t head_dim) {
    // gqa.rs:106-141
    if (n_kv_heads <= 0 || n_heads < 0 || n_heads % n_kv_heads != 0) return RT_ERR_HEAD_COUNT;
    if (batch < 0 || seq_q < 0 || seq_kv < 0 || head_dim < 0) return RT_ERR_BAD_LENGTH;
    const size_t qn = (size_t)batch * n_heads * seq_q * head_dim;
    const size_t kn = (size_t)batch * n_kv_heads * seq_kv * head_dim;
    if (q_len != qn || k_len != kn || v_len != kn || out_len != qn) return RT_ERR_WRONG_INPUT_LEN;
    if (qn == 0) return RT_OK;
    if (head_dim > 256) return RT_ERR_UNSUPPORTED;
    if (!q || !out || (kn > 0 && (!k || !v))) return RT_ERR_NULL_POINTER;
    std::lock_guard<std::mutex> lock(g_staging.mu);
    DevBuf dq(0), dk(1), dv(2), dout(3);
    RT_CUDA(dq.alloc(qn * 4));
    RT_CUDA(dk.alloc(kn * 4));
    RT_CUDA(dv.alloc(kn * 4));
    RT_CUDA(dout.alloc(qn * 4));
    RT_CUDA(cudaMemcpy(dq.p, q, qn * 4, cudaMemcpyHostToDevice));
    if (kn) {
        RT_CUDA(cudaMemcpy(dk.p, k, kn * 4, cudaMemcpyHostToDevice));
        RT_CUDA(cudaMemcpy(dv.p, v, kn * 4, cudaMemcpyHostToDevice));
    }
    if (seq_kv == 0) {
        // The reference's row kernel returns zeros when there is nothing to attend to (gqa.rs:262-269).
        RT_CUDA(cudaMemset(dout.p, 0, qn * 4));
    } else {
        int rc = rt_attn_prefill_f32(dq.as<float>(), dk.as<float>(), dv.as<float>(), dout.as<float>(), nullptr, batch,
                                     n_heads, n_kv_heads, seq_q, seq_kv, (int)head_dim, RT_MASK_NONE, nullptr,
                                     nullptr, nullptr, 0, -1.f, nullptr);
        if (rc != RT_OK) return rc;
    }
    RT_CUDA(cudaMemcpy(out, dout.p, qn * 4, cudaMemcpyDeviceToHost));
    return RT_OK;
}

int rt_kv_append_bf16(void* k_cache, void* v_cache, const void* k_in, const void* v_in, int64_t batch, int n_kv,
                      int head_dim, int64_t max_seq, int64_t pos, const int32_t* positions, void* stream) {
    if (batch < 0 || n_kv < 0 || head_dim < 0 || max_seq < 0) return RT_ERR_BAD_LENGTH;
    if (!positions && (pos < 0 || pos >= max_seq)) return RT_ERR_BAD_LENGTH;  // kv_cache.rs:88-93 overflow
    if (batch == 0 || n_kv == 0 || head_dim == 0) return RT_OK;
    if (!k_cache || !v_cache || !k_in || !v_in) return RT_ERR_NULL_POINTER;
    if (batch > 65535) return RT_ERR_UNSUPPORTED;
    RT_CUDA(rt::launch_kv_append(k_cache, v_cache, k_in, v_in, batch, n_kv, head_dim, max_seq, pos, positions,
                                 as_stream(stream)));
    return RT_OK;
}

int rt_rope_kv_append_bf16(void* q, const void* k_in, const void* v_in, void* k_cache, void* v_cache,
                           const float* inv_freq, int64_t batch, int n_heads, int n_kv, int head_dim, int64_t max_seq,
                           int64_t pos, const int32_t* positions, int rope_style, void* stream) {
    if (batch < 0 || n_heads < 0 || n_kv < 0 || head_dim < 0 || max_seq < 0) return RT_ERR_BAD_LENGTH;
    if (head_dim == 0) return RT_ERR_ZERO_DIM;
    if (head_dim % 2 != 0 || (rope_style != RT_ROPE_HALF_SPLIT && rope_style != RT_ROPE_ADJACENT))
        return RT_ERR_UNSUPPORTED;  // RoPE::new asserts an even head_dim (rope.rs:64-68)
    if (!positions && (pos < 0 || pos >= max_seq)) return RT_ERR_BAD_LENGTH;  // RoPEError::PositionOverflow
    if (batch == 0 || n_heads + n_kv == 0) return RT_OK;
    if (batch > 65535) return RT_ERR_UNSUPPORTED;
    if (!inv_freq || (n_heads > 0 && !q) || (n_kv > 0 && (!k_in || !v_in || !k_cache || !v_cache)))
        return RT_ERR_NULL_POINTER;
    RT_CUDA(rt::launch_rope_kv_append(q, k_in, v_in, k_cache, v_cache, inv_freq, positions, pos, batch, n_heads, n_kv,
                                      head_dim, max_seq, rope_style, as_stream(stream)));
    return RT_OK;
}

int rt_convert_f32_to_bf16(const float* src, void* dst, int64_t n, void* stream) {
    if (n < 0) return RT_ERR_BAD_LENGTH;
    if (n == 0) return RT_OK;
    if (!src || !dst) return RT_ERR_NULL_POINTER;
    RT_CUDA(rt::launch_f32_to_bf16(src, dst, n, as_stream(stream)));
    return RT_OK;
}

int rt_convert_bf16_to_f32(const void* src, float* dst, int64_t n, void* stream) {
    if (n < 0) return RT_ERR_BAD_LENGTH;
    if (n == 0) return RT_OK;
    if (!src || !dst) return RT_ERR_NULL_POINTER;
    RT_CUDA(rt::launch_bf16_to_f32(src, dst, n, as_stream(stream)));
    return RT_OK;
}

}  // extern "C"
