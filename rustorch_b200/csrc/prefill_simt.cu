// f32 flash-attention forward on CUDA cores, plus the f32 <-> bf16 conversion kernels.
//
// This is the exact-arithmetic companion of the tensor-core kernel: f32 inputs, f32
// accumulation, accurate expf, any head dim up to 256, seq_q != seq_kv and grouped KV heads.
// It backs the host mirrors of flash_forward_masked (crates/rustorch-attention/src/cpu_forward.rs:193-242)
// and gqa_forward_f32 (crates/rustorch-nn/src/gqa.rs:94-210) at the reference's own 1e-4
// tolerance.  One warp owns one query row and walks the keys in tiles of 32 staged in shared
// memory; the online-softmax recurrence is the reference's (cpu_forward.rs:355-386) with the
// leading-masked-tile case resolved to the finite answer.
#include "common.cuh"
#include "kernels.h"

namespace rt {

constexpr int kSimtRows = 8;   // query rows (warps) per CTA
constexpr int kSimtKeys = 32;  // keys per tile (one per lane)

struct SimtParams {
    const float *q, *k, *v;
    float *out, *lse;
    int64_t heads_q, heads_kv, seq_q, seq_kv;
    int dim, causal;
    const int32_t* kv_lens;
    const int32_t* q_offsets;
    const uint8_t* key_keep;
    int64_t keep_batch_stride;
    float scale;
};

__global__ void __launch_bounds__(kSimtRows * 32) prefill_f32_kernel(const SimtParams p) {
    extern __shared__ float smem[];
    const int D = p.dim;
    float* Ks = smem;                              // [32][D+1]
    float* Vs = Ks + kSimtKeys * (D + 1);          // [32][D]
    float* Qs = Vs + kSimtKeys * D;                // [rows][D]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t b = blockIdx.z, hq = blockIdx.y;
    const int64_t hkv = hq / (p.heads_q / p.heads_kv);
    const int64_t row0 = (int64_t)blockIdx.x * kSimtRows;
    const int64_t qi = row0 + warp;
    const bool row_valid = qi < p.seq_q;

    const float* qptr = p.q + ((b * p.heads_q + hq) * p.seq_q) * D;
    const float* kptr = p.k + ((b * p.heads_kv + hkv) * p.seq_kv) * D;
    const float* vptr = p.v + ((b * p.heads_kv + hkv) * p.seq_kv) * D;
    const uint8_t* keep = p.key_keep ? p.key_keep + b * p.keep_batch_stride : nullptr;

    for (int i = threadIdx.x; i < kSimtRows * D; i += blockDim.x) {
        const int64_t r = row0 + i / D;
        Qs[i] = (r < p.seq_q) ? qptr[r * D + i % D] : 0.f;
    }

    int64_t k_hi = p.seq_kv;
    if (p.kv_lens && p.kv_lens[b] < k_hi) k_hi = p.kv_lens[b] < 0 ? 0 : p.kv_lens[b];
    const int64_t q_off = p.q_offsets ? p.q_offsets[b] : 0;  // query row i sits at key position i + q_off
    int64_t k_loop = k_hi;
    if (p.causal) {
        int64_t last = row0 + kSimtRows;  // keys <= position of the last query row of the CTA
        if (last > p.seq_q) last = p.seq_q;
        last += q_off;
        if (last < 0) last = 0;
        if (last < k_loop) k_loop = last;
    }

    float m = -INFINITY, l = 0.f;
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = 0.f;

    for (int64_t kj = 0; kj < k_loop; kj += kSimtKeys) {
        __syncthreads();
        for (int i = threadIdx.x; i < kSimtKeys * D; i += blockDim.x) {
            const int r = i / D, d = i % D;
            const bool in = kj + r < k_hi;
            Ks[r * (D + 1) + d] = in ? kptr[(kj + r) * D + d] : 0.f;
            Vs[r * D + d] = in ? vptr[(kj + r) * D + d] : 0.f;
        }
        __syncthreads();
        if (!row_valid) continue;

        const int64_t key = kj + lane;
        float s = 0.f;
        const float* qrow = Qs + warp * D;
        const float* krow = Ks + lane * (D + 1);
        for (int d = 0; d < D; ++d) s = fmaf(qrow[d], krow[d], s);
        s *= p.scale;
        bool masked = key >= k_hi;
        if (p.causal && key > qi + q_off) masked = true;
        if (keep && key < p.seq_kv && !keep[key]) masked = true;
        if (masked) s = -INFINITY;

        float m_tile = s;
#pragma unroll
        for (int off = 16; off; off >>= 1) m_tile = fmaxf(m_tile, __shfl_xor_sync(kFullMask, m_tile, off));
        const float m_new = fmaxf(m, m_tile);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_use);
        const float pe = masked ? 0.f : expf(s - m_use);
        float psum = pe;
#pragma unroll
        for (int off = 16; off; off >>= 1) psum += __shfl_xor_sync(kFullMask, psum, off);
        l = l * alpha + psum;
        m = m_new;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] *= alpha;
        for (int jj = 0; jj < kSimtKeys; ++jj) {
            const float pj = __shfl_sync(kFullMask, pe, jj);
            const float* vrow = Vs + jj * D;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int d = lane + 32 * i;
                if (d < D) o[i] = fmaf(pj, vrow[d], o[i]);
            }
        }
    }

    if (!row_valid) return;
    float* dst = p.out + ((b * p.heads_q + hq) * p.seq_q + qi) * D;
    const bool ok = (l > 0.f) && isfinite(l);  // cpu_forward.rs:411
    const float inv = ok ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = lane + 32 * i;
        if (d < D) dst[d] = ok ? o[i] * inv : NAN;
    }
    if (p.lse && lane == 0)
        p.lse[(b * p.heads_q + hq) * p.seq_q + qi] = (l > 0.f) ? m + logf(l) : (l == 0.f ? -INFINITY : NAN);
}

cudaError_t launch_prefill_f32(const float* q, const float* k, const float* v, float* out, float* lse,
                               int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seq_q,
                               int64_t seq_kv, int dim, int causal, const int32_t* kv_lens,
                               const int32_t* q_offsets, const uint8_t* key_keep, int64_t keep_batch_stride,
                               float scale, cudaStream_t stream) {
    if (batch == 0 || heads_q == 0 || seq_q == 0) return cudaSuccess;
    SimtParams p{q, k, v, out, lse, heads_q, heads_kv, seq_q, seq_kv, dim, causal, kv_lens, q_offsets, key_keep,
                 keep_batch_stride, scale};
    const size_t smem = sizeof(float) * ((size_t)kSimtKeys * (dim + 1) + (size_t)kSimtKeys * dim +
                                         (size_t)kSimtRows * dim);
    cudaError_t e = cudaFuncSetAttribute(prefill_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return e;
    const int64_t row_blocks = (seq_q + kSimtRows - 1) / kSimtRows;
    if (row_blocks > 0x7fffffff || heads_q > 65535 || batch > 65535) return cudaErrorInvalidValue;
    dim3 grid((unsigned)row_blocks, (unsigned)heads_q, (unsigned)batch);
    prefill_f32_kernel<<<grid, kSimtRows * 32, smem, stream>>>(p);
    return cudaGetLastError();
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = __float2bfloat16_rn(src[i]);
}

__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = __bfloat162float(src[i]);
}

static unsigned grid_for(int64_t n) {
    int64_t g = (n + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    return (unsigned)(g > cap ? cap : (g < 1 ? 1 : g));
}

cudaError_t launch_f32_to_bf16(const float* src, void* dst, int64_t n, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    f32_to_bf16_kernel<<<grid_for(n), 256, 0, stream>>>(src, (__nv_bfloat16*)dst, n);
    return cudaGetLastError();
}

cudaError_t launch_bf16_to_f32(const void* src, float* dst, int64_t n, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    bf16_to_f32_kernel<<<grid_for(n), 256, 0, stream>>>((const __nv_bfloat16*)src, dst, n);
    return cudaGetLastError();
}

}  // namespace rt
