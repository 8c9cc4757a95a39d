// f32 flash-attention forward on CUDA cores, plus the f32 <-> bf16 conversion kernels.
//
// This is the exact-arithmetic companion of the tensor-core kernel: f32 inputs, f32
// accumulation, accurate expf, any head dim up to 256, seq_q != seq_kv and grouped KV heads.
// It backs the host mirrors of flash_forward_masked (crates/rustorch-attention/src/cpu_forward.rs:193-242)
// and gqa_forward_f32 (crates/rustorch-nn/src/gqa.rs:94-210) at the reference's own 1e-4
// tolerance.  One warp owns one query row and walks the keys in tiles of 32 staged in shared
// memory; the online-softmax recurrence is the reference's (cpu_forward.rs:355-386) with the
// leading-masked-tile case resolved to the finite answer.
#include <cstdlib>

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

// ---------------------------------------------------------------------------------------------
// Register-tiled variant: one CTA of 256 threads (16 x 16) owns 64 query rows and walks the keys in
// tiles of 64.  Q and K sit transposed in shared memory ([d][row], [d][key]) so that the score
// product reads one 16-byte vector of each per 16 multiply-adds (thread (ty, tx) holds the 4 x 4
// block rows 4 ty.., keys 4 tx..); the probabilities go through shared memory ([row][key]) and the
// P V product reads 4 keys x (4 rows of P + NG vectors of V) per 64 NG multiply-adds.  Same recurrence,
// masks and NaN rules as the kernel above; NG = ceil(D / 64) groups of 64 output columns.
constexpr int kTileRows = 64, kTileKeys = 64, kTilePad = 68;  // 68: rows stay 16-byte aligned, 4-bank skew

template <int NG>
__global__ void __launch_bounds__(256) prefill_f32_tiled_kernel(const SimtParams p) {
    extern __shared__ __align__(16) float smem[];
    const int D = p.dim;
    constexpr int DP = NG * 64;
    float* Qt = smem;                         // [D][68]   Q transposed, scaled
    float* Kt = Qt + (size_t)D * kTilePad;    // [D][68]   K transposed
    float* Vs = Kt + (size_t)D * kTilePad;    // [64][DP]  V, columns >= D zero
    float* Ps = Vs + (size_t)kTileKeys * DP;  // [64][68]  probabilities [row][key]

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int64_t b = blockIdx.z, hq = blockIdx.y;
    const int64_t hkv = hq / (p.heads_q / p.heads_kv);
    const int64_t row0 = (int64_t)(gridDim.x - 1 - blockIdx.x) * kTileRows;  // heaviest causal blocks first

    const float* qptr = p.q + ((b * p.heads_q + hq) * p.seq_q) * D;
    const float* kptr = p.k + ((b * p.heads_kv + hkv) * p.seq_kv) * D;
    const float* vptr = p.v + ((b * p.heads_kv + hkv) * p.seq_kv) * D;
    const uint8_t* keep = p.key_keep ? p.key_keep + b * p.keep_batch_stride : nullptr;

    for (int i = tid; i < kTileRows * D; i += 256) {
        const int r = i / D, d = i % D;
        Qt[d * kTilePad + r] = (row0 + r < p.seq_q) ? qptr[(row0 + r) * D + d] * p.scale : 0.f;
    }

    int64_t k_hi = p.seq_kv;
    if (p.kv_lens && p.kv_lens[b] < k_hi) k_hi = p.kv_lens[b] < 0 ? 0 : p.kv_lens[b];
    const int64_t q_off = p.q_offsets ? p.q_offsets[b] : 0;  // query row i sits at key position i + q_off
    int64_t k_loop = k_hi;
    if (p.causal) {
        int64_t last = row0 + kTileRows;  // keys <= position of the last query row of the CTA
        if (last > p.seq_q) last = p.seq_q;
        last += q_off;
        if (last < 0) last = 0;
        if (last < k_loop) k_loop = last;
    }

    float m[4], l[4], o[4][NG][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int g = 0; g < NG; ++g)
#pragma unroll
            for (int c = 0; c < 4; ++c) o[i][g][c] = 0.f;
    }

    for (int64_t kj = 0; kj < k_loop; kj += kTileKeys) {
        __syncthreads();  // the previous tile's K, V and P are no longer read
        for (int i = tid; i < kTileKeys * D; i += 256) {
            const int r = i / D, d = i % D;
            const bool in = kj + r < k_hi;
            Kt[d * kTilePad + r] = in ? kptr[(kj + r) * D + d] : 0.f;
            Vs[r * DP + d] = in ? vptr[(kj + r) * D + d] : 0.f;
        }
        if (D < DP) {
            const int extra = DP - D;
            for (int i = tid; i < kTileKeys * extra; i += 256) Vs[(i / extra) * DP + D + i % extra] = 0.f;
        }
        __syncthreads();

        // ---- S = (scale Q) K^T, 4 x 4 per thread
        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll 4
        for (int d = 0; d < D; ++d) {
            const float4 q4 = *reinterpret_cast<const float4*>(Qt + d * kTilePad + ty * 4);
            const float4 k4 = *reinterpret_cast<const float4*>(Kt + d * kTilePad + tx * 4);
            const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, ka[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) s[i][j] = fmaf(qa[i], ka[j], s[i][j]);
        }

        // ---- masks, online softmax (the 16 threads of a row group agree through shuffles)
        bool masked[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t key = kj + tx * 4 + j;
            const bool off = key >= k_hi || (keep && key < p.seq_kv && !keep[key]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                masked[i][j] = off || (p.causal && key > row0 + ty * 4 + i + q_off);
                if (masked[i][j]) s[i][j] = -INFINITY;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float m_tile = fmaxf(fmaxf(s[i][0], s[i][1]), fmaxf(s[i][2], s[i][3]));
#pragma unroll
            for (int off = 8; off; off >>= 1) m_tile = fmaxf(m_tile, __shfl_xor_sync(kFullMask, m_tile, off));
            const float m_new = fmaxf(m[i], m_tile);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = (m[i] == -INFINITY) ? 0.f : expf(m[i] - m_use);
            float psum = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                s[i][j] = masked[i][j] ? 0.f : expf(s[i][j] - m_use);
                psum += s[i][j];
            }
#pragma unroll
            for (int off = 8; off; off >>= 1) psum += __shfl_xor_sync(kFullMask, psum, off);
            l[i] = l[i] * alpha + psum;
            m[i] = m_new;
#pragma unroll
            for (int g = 0; g < NG; ++g)
#pragma unroll
                for (int c = 0; c < 4; ++c) o[i][g][c] *= alpha;
            *reinterpret_cast<float4*>(Ps + (ty * 4 + i) * kTilePad + tx * 4) = make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
        }
        __syncthreads();

        // ---- O += P V: rows 4 ty.., columns 64 g + 4 tx..
#pragma unroll 2
        for (int kk = 0; kk < kTileKeys; kk += 4) {
            float pa[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 t = *reinterpret_cast<const float4*>(Ps + (ty * 4 + i) * kTilePad + kk);
                pa[i][0] = t.x; pa[i][1] = t.y; pa[i][2] = t.z; pa[i][3] = t.w;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    const float4 v4 = *reinterpret_cast<const float4*>(Vs + (kk + u) * DP + g * 64 + tx * 4);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        o[i][g][0] = fmaf(pa[i][u], v4.x, o[i][g][0]);
                        o[i][g][1] = fmaf(pa[i][u], v4.y, o[i][g][1]);
                        o[i][g][2] = fmaf(pa[i][u], v4.z, o[i][g][2]);
                        o[i][g][3] = fmaf(pa[i][u], v4.w, o[i][g][3]);
                    }
                }
        }
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t qi = row0 + ty * 4 + i;
        if (qi >= p.seq_q) continue;
        float* dst = p.out + ((b * p.heads_q + hq) * p.seq_q + qi) * D;
        const bool ok = (l[i] > 0.f) && isfinite(l[i]);  // cpu_forward.rs:411
        const float inv = ok ? 1.f / l[i] : 0.f;
#pragma unroll
        for (int g = 0; g < NG; ++g)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int d = g * 64 + tx * 4 + c;
                if (d < D) dst[d] = ok ? o[i][g][c] * inv : NAN;
            }
        if (p.lse && tx == 0)
            p.lse[(b * p.heads_q + hq) * p.seq_q + qi] =
                (l[i] > 0.f) ? m[i] + logf(l[i]) : (l[i] == 0.f ? -INFINITY : NAN);
    }
}

template <int NG>
static cudaError_t launch_tiled(const SimtParams& p, int64_t batch, cudaStream_t stream) {
    const size_t smem = sizeof(float) * (2 * (size_t)p.dim * kTilePad + (size_t)kTileKeys * NG * 64 +
                                         (size_t)kTileRows * kTilePad);
    cudaError_t e = cudaFuncSetAttribute(prefill_f32_tiled_kernel<NG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return e;
    const int64_t row_blocks = (p.seq_q + kTileRows - 1) / kTileRows;
    if (row_blocks > 0x7fffffff || p.heads_q > 65535 || batch > 65535) return cudaErrorInvalidValue;
    dim3 grid((unsigned)row_blocks, (unsigned)p.heads_q, (unsigned)batch);
    prefill_f32_tiled_kernel<NG><<<grid, 256, smem, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_prefill_f32(const float* q, const float* k, const float* v, float* out, float* lse,
                               int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seq_q,
                               int64_t seq_kv, int dim, int causal, const int32_t* kv_lens,
                               const int32_t* q_offsets, const uint8_t* key_keep, int64_t keep_batch_stride,
                               float scale, cudaStream_t stream) {
    if (batch == 0 || heads_q == 0 || seq_q == 0) return cudaSuccess;
    SimtParams p{q, k, v, out, lse, heads_q, heads_kv, seq_q, seq_kv, dim, causal, kv_lens, q_offsets, key_keep,
                 keep_batch_stride, scale};
    // The register-tiled kernel is the path for 16 query rows and more; a decode-shaped call (a few rows against
    // a long cache) would waste most of its 64-row tile and keeps the warp-per-row kernel, which
    // RT_ATTN_PREFILL_F32_IMPL=rows selects for every shape (comparisons).  The tiled kernel applies the scale
    // to Q once, the other one to every score.
    static const bool rows_impl = [] {
        const char* e = getenv("RT_ATTN_PREFILL_F32_IMPL");
        return e && e[0] == 'r';
    }();
    if (!rows_impl && dim <= 256 && seq_q >= 16) {
        if (dim <= 64) return launch_tiled<1>(p, batch, stream);
        if (dim <= 128) return launch_tiled<2>(p, batch, stream);
        return launch_tiled<4>(p, batch, stream);
    }
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
