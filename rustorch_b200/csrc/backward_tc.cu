// bf16 flash-attention backward on the tensor cores (mma.sync.m16n8k16, f32 accumulate).
//
// Same math as rustorch_attention::flash_backward (crates/rustorch-attention/src/cpu_backward.rs:16-27,
// 96-189) with the saved row statistics in place of the N x N probability matrix:
//   P = exp(scale * Q K^T - LSE),  dP = dO V^T,  dS = P o (dP - delta),  delta_i = dO_i . O_i,
//   dV = P^T dO,  dQ = scale * dS K,  dK = scale * dS^T Q.
// Two deterministic passes share one kernel template.  A CTA owns 64 rows of one side (4 warps x 16
// rows) and walks the 64-row tiles of the other side:
//   query side: X1 = Q, X2 = dO (own rows);  per key tile  T1 = Q K^T, T2 = dO V^T -> dS;  dQ += dS K
//   key side:   X1 = K, X2 = V  (own rows);  per query tile T1 = K Q^T, T2 = V dO^T -> P^T, dS^T;
//               dV += P^T dO,  dK += dS^T Q
// so every product has the shape "own rows (A, from shared memory via ldmatrix) x other tile (B)":
// B comes from the other tile untransposed for the score-like products and through ldmatrix.trans
// for the accumulating ones, and the score accumulators are re-packed in registers as the A operand
// of the accumulating product.  P and dS are rounded to bf16 for those products, as the forward
// rounds P.  No atomics; a causal launch skips the tiles beyond the diagonal.
// The other side's tiles travel global -> 128-byte-swizzled shared memory with cp.async into two
// stages, so the loads of tile t+1 overlap the MMAs of tile t.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "mma_sync.cuh"

namespace rt {

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

constexpr int kRows = 64;  // rows per tile (own side and other side)

// Byte offset of the 16-byte chunk (row, chunk16) of a [64 x D] bf16 tile: 64-column sub-tiles of
// 128-byte rows, chunk index XORed with the row (conflict-free ldmatrix in both orientations).
__device__ __forceinline__ uint32_t tile_off(int row, int chunk16) {
    return (uint32_t)((chunk16 >> 3) * (kRows * 128) + row * 128 + (((chunk16 & 7) ^ (row & 7)) << 4));
}

// Cooperative load of rows [r0, r0+64) of a [N x D] bf16 matrix into a swizzled tile; rows >= N are zero.
template <int D>
__device__ __forceinline__ void load_tile(uint8_t* tile, const __nv_bfloat16* src, int64_t r0, int64_t n_rows) {
    constexpr int CH = D / 8;  // 16-byte chunks per row
    for (int i = threadIdx.x; i < kRows * CH; i += blockDim.x) {
        const int r = i / CH, c = i % CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r0 + r < n_rows) v = *reinterpret_cast<const uint4*>(src + (r0 + r) * D + c * 8);
        *reinterpret_cast<uint4*>(tile + tile_off(r, c)) = v;
    }
}

// The same through cp.async (no registers held, completion by commit/wait groups); rows >= N are
// zero-filled by a zero source size (the source address is clamped to a valid row).
template <int D>
__device__ __forceinline__ void load_tile_async(uint8_t* tile, const __nv_bfloat16* src, int64_t r0, int64_t n_rows) {
    constexpr int CH = D / 8;
    const uint32_t base = smem_u32(tile);
    for (int i = threadIdx.x; i < kRows * CH; i += blockDim.x) {
        const int r = i / CH, c = i % CH;
        const bool in = r0 + r < n_rows;
        const __nv_bfloat16* g = src + (in ? r0 + r : 0) * D + c * 8;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(base + tile_off(r, c)), "l"(g),
                     "r"(in ? 16 : 0)
                     : "memory");
    }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

}  // namespace

struct BwdTcParams {
    const __nv_bfloat16 *q, *k, *v, *d_out;
    const float *lse, *delta;
    float *dq, *dk, *dv;
    int64_t seq;
    int causal;
    float scale, scale_log2;
};

// delta_i = dO_i . O_i from the bf16 forward output.  Each thread takes 16 bytes (8 elements) of both
// tensors, so D / 8 neighbouring lanes cover a row, a warp covers 32 / (D / 8) rows per pass and runs two
// passes with all four loads in flight: the kernel is a pure HBM stream (4 D bytes per row).
template <int D>
__global__ void __launch_bounds__(256) bwd_delta_bf16_kernel(const __nv_bfloat16* __restrict__ out,
                                                             const __nv_bfloat16* __restrict__ d_out,
                                                             float* __restrict__ delta, int64_t rows) {
    constexpr int LPR = D / 8;        // lanes per row
    constexpr int RPW = 32 / LPR;     // rows per warp and pass
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane / LPR, col = (lane % LPR) * 8;
    const int64_t row0 = ((int64_t)blockIdx.x * 8 + warp) * (2 * RPW) + sub;
    float acc[2];
    uint4 a[2], b[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int64_t row = row0 + u * RPW;
        if (row < rows) {
            a[u] = __ldg(reinterpret_cast<const uint4*>(out + row * D + col));
            b[u] = __ldg(reinterpret_cast<const uint4*>(d_out + row * D + col));
        } else {
            a[u] = b[u] = make_uint4(0u, 0u, 0u, 0u);
        }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a[u]);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b[u]);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
            s = fmaf(x.x, y.x, fmaf(x.y, y.y, s));
        }
#pragma unroll
        for (int off = LPR / 2; off; off >>= 1) s += __shfl_xor_sync(kFullMask, s, off);
        acc[u] = s;
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int64_t row = row0 + u * RPW;
        if (col == 0 && row < rows) delta[row] = acc[u];
    }
}

template <int D, bool kKeySide>
__global__ void __launch_bounds__(128) bwd_tc_kernel(const BwdTcParams p) {
    constexpr int TILE = kRows * D * 2;
    constexpr int NT_D = D / 8;   // n-tiles across the head dim
    extern __shared__ __align__(1024) uint8_t smem_bwd[];
    uint8_t* sX1 = smem_bwd;             // own rows: Q (query side) / K (key side)
    uint8_t* sX2 = sX1 + TILE;           // own rows: dO           / V
    uint8_t* sY = sX2 + TILE;            // two stages of the other side: [stage][K, V] / [stage][Q, dO]
    float* sStat = reinterpret_cast<float*>(sY + 4 * TILE);  // [2 stages][lse (natural log) | delta][64] of QUERY rows

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t bh = blockIdx.y, N = p.seq;
    const int64_t own0 = (int64_t)blockIdx.x * kRows;
    const int64_t base = bh * N * D;
    const __nv_bfloat16* X1 = (kKeySide ? p.k : p.q) + base;
    const __nv_bfloat16* X2 = (kKeySide ? p.v : p.d_out) + base;
    const __nv_bfloat16* Y1 = (kKeySide ? p.q : p.k) + base;
    const __nv_bfloat16* Y2 = (kKeySide ? p.d_out : p.v) + base;

    load_tile<D>(sX1, X1, own0, N);
    load_tile<D>(sX2, X2, own0, N);
    // query statistics: of the own rows (query side, loaded once into stage 0) or of each tile (key side)
    auto load_stats = [&](int stage, int64_t r0) {
        if (threadIdx.x < kRows) {
            const int64_t r = r0 + threadIdx.x;
            sStat[stage * 2 * kRows + threadIdx.x] = r < N ? p.lse[bh * N + r] : -INFINITY;
            sStat[stage * 2 * kRows + kRows + threadIdx.x] = r < N ? p.delta[bh * N + r] : 0.f;
        }
    };
    if (!kKeySide) load_stats(0, own0);

    // other-side tile range
    int64_t t_lo = 0, t_hi = N;
    if (p.causal) {
        if (kKeySide) t_lo = own0;                                   // queries >= the first own key
        else t_hi = own0 + kRows < N ? own0 + kRows : N;             // keys <= the last own query
    }

    float z1[NT_D][4];                    // query side: dQ; key side: dK
    float z2[kKeySide ? NT_D : 1][4];     // key side: dV
#pragma unroll
    for (int j = 0; j < NT_D; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) z1[j][e] = 0.f;
#pragma unroll
    for (int j = 0; j < (kKeySide ? NT_D : 1); ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) z2[j][e] = 0.f;

    const uint32_t x1_a = smem_u32(sX1), x2_a = smem_u32(sX2);
    const int lr = lane & 7, lm = lane >> 3;          // ldmatrix: this lane addresses row lr of matrix lm
    const int a_row = warp * 16 + (lm & 1) * 8 + lr;  // A operand: matrices 0,2 rows 0-7; 1,3 rows 8-15

    auto prefetch = [&](int stage, int64_t t0) {
        load_tile_async<D>(sY + (stage * 2) * TILE, Y1, t0, N);
        load_tile_async<D>(sY + (stage * 2 + 1) * TILE, Y2, t0, N);
        if (kKeySide) load_stats(stage, t0);
        cp_async_commit();
    };
    if (t_lo < t_hi) prefetch(0, t_lo);
    int stage = 0;
    for (int64_t t0 = t_lo; t0 < t_hi; t0 += kRows, stage ^= 1) {
        // the other stage was last read in the previous iteration; every warp has passed its barrier below
        if (t0 + kRows < t_hi) {
            prefetch(stage ^ 1, t0 + kRows);
            cp_async_wait<1>();  // this iteration's tile has landed (the prefetch just issued may be in flight)
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();  // copies and statistics of all threads visible (also orders the X loads before first use)
        const uint32_t y1_a = smem_u32(sY + (stage * 2) * TILE), y2_a = smem_u32(sY + (stage * 2 + 1) * TILE);
        const float* sLse = sStat + (kKeySide ? stage * 2 * kRows : 0);
        const float* sDelta = sLse + kRows;

#pragma unroll
        for (int half = 0; half < 2; ++half) {  // 32 columns of the other tile at a time (register budget)
            float t1[4][4], t2[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) t1[j][e] = t2[j][e] = 0.f;

            // ---- T1 = X1 Y1^T, T2 = X2 Y2^T over the head dim (D/16 k-steps, two per B ldmatrix)
#pragma unroll
            for (int kp = 0; kp < D / 32; ++kp) {
                uint32_t a1[2][4], a2[2][4];
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    const int chunk = (kp * 2 + s) * 2 + (lm >> 1);
                    ldmatrix_x4(x1_a + tile_off(a_row, chunk), a1[s][0], a1[s][1], a1[s][2], a1[s][3]);
                    ldmatrix_x4(x2_a + tile_off(a_row, chunk), a2[s][0], a2[s][1], a2[s][2], a2[s][3]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int n_row = half * 32 + j * 8 + lr;
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(y1_a + tile_off(n_row, kp * 4 + lm), b0, b1, b2, b3);
                    mma_bf16(t1[j], a1[0], b0, b1);
                    mma_bf16(t1[j], a1[1], b2, b3);
                    ldmatrix_x4(y2_a + tile_off(n_row, kp * 4 + lm), b0, b1, b2, b3);
                    mma_bf16(t2[j], a2[0], b0, b1);
                    mma_bf16(t2[j], a2[1], b2, b3);
                }
            }

            // ---- P and dS on the accumulator fragments; element e of n-tile j sits at
            //      own row g + 8*(e>>1), other column half*32 + j*8 + 2t + (e&1)
            uint32_t wp[2][4], wd[2][4];  // A fragments (two k-steps of 16 columns): P (key side only) and dS
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float pv[4], dv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r_own = warp * 16 + g + 8 * (e >> 1);
                    const int c_oth = half * 32 + j * 8 + 2 * t + (e & 1);
                    const int64_t own = own0 + r_own, oth = t0 + c_oth;
                    const int64_t qi = kKeySide ? oth : own, kj = kKeySide ? own : oth;
                    const int stat = kKeySide ? c_oth : r_own;
                    const float lse = sLse[stat];
                    const bool vis = own < N && oth < N && !(p.causal && kj > qi) && lse != -INFINITY;
                    const float prob = vis ? fast_exp2(t1[j][e] * p.scale_log2 - lse * kLog2e) : 0.f;
                    pv[e] = prob;
                    dv[e] = prob * (t2[j][e] - sDelta[stat]) * p.scale;
                }
                // n-tiles 2s and 2s+1 of this half form k-step s of the accumulating product
                const int s = j >> 1, hi = (j & 1) * 2;
                if (kKeySide) {
                    wp[s][hi] = float2_to_bf16x2(pv[0], pv[1]);
                    wp[s][hi + 1] = float2_to_bf16x2(pv[2], pv[3]);
                }
                wd[s][hi] = float2_to_bf16x2(dv[0], dv[1]);
                wd[s][hi + 1] = float2_to_bf16x2(dv[2], dv[3]);
            }

            // ---- Z1 += dS Y1 (dQ += dS K / dK += dS^T Q);  key side also Z2 += P^T Y2 (dV += P^T dO)
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                const int k_row = half * 32 + s * 16 + (lm & 1) * 8 + lr;  // matrices 0,2: k 0-7; 1,3: k 8-15
#pragma unroll
                for (int jp = 0; jp < NT_D / 2; ++jp) {  // two n-tiles of the head dim per ldmatrix.trans
                    const int chunk = jp * 2 + (lm >> 1);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(y1_a + tile_off(k_row, chunk), b0, b1, b2, b3);
                    mma_bf16(z1[2 * jp], wd[s], b0, b1);
                    mma_bf16(z1[2 * jp + 1], wd[s], b2, b3);
                    if (kKeySide) {
                        ldmatrix_x4_trans(y2_a + tile_off(k_row, chunk), b0, b1, b2, b3);
                        mma_bf16(z2[2 * jp], wp[s], b0, b1);
                        mma_bf16(z2[2 * jp + 1], wp[s], b2, b3);
                    }
                }
            }
        }
        __syncthreads();  // every warp is done with this stage before the next iteration refills it
    }

    // ---- write the own rows: element e of n-tile j = row g + 8*(e>>1), column j*8 + 2t + (e&1)
    float* out1 = (kKeySide ? p.dk : p.dq) + base;
#pragma unroll
    for (int j = 0; j < NT_D; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t r = own0 + warp * 16 + g + 8 * h;
            if (r < N) {
                *reinterpret_cast<float2*>(out1 + r * D + j * 8 + 2 * t) = make_float2(z1[j][2 * h], z1[j][2 * h + 1]);
                if (kKeySide)
                    *reinterpret_cast<float2*>(p.dv + base + r * D + j * 8 + 2 * t) =
                        make_float2(z2[j][2 * h], z2[j][2 * h + 1]);
            }
        }
    }
}

template <int D>
static cudaError_t launch_bwd_tc(const BwdTcParams& p, int64_t bh, cudaStream_t stream) {
    const size_t smem = (size_t)6 * kRows * D * 2 + 4 * kRows * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(bwd_tc_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(bwd_tc_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dim3 grid((unsigned)((p.seq + kRows - 1) / kRows), (unsigned)bh);
    bwd_tc_kernel<D, false><<<grid, 128, smem, stream>>>(p);
    bwd_tc_kernel<D, true><<<grid, 128, smem, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_backward_bf16(const void* q, const void* k, const void* v, const void* out, const void* d_out,
                                 const float* lse, float* dq, float* dk, float* dv, float* delta_ws, int64_t batch,
                                 int64_t heads, int64_t seq, int dim, int causal, float scale, cudaStream_t stream) {
    const int64_t bh = batch * heads;
    if (bh == 0 || seq == 0) return cudaSuccess;
    if (bh > 65535) return cudaErrorInvalidValue;
    const int64_t rows = bh * seq;
    if (dim != 64 && dim != 128) return cudaErrorInvalidValue;
    {
        const int rows_per_cta = 8 * 2 * (32 / (dim / 8));
        const unsigned grid = (unsigned)((rows + rows_per_cta - 1) / rows_per_cta);
        if (dim == 128)
            bwd_delta_bf16_kernel<128><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)d_out,
                                                                 delta_ws, rows);
        else
            bwd_delta_bf16_kernel<64><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)d_out,
                                                                delta_ws, rows);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    // The tcgen05 / TMEM / TMA kernel (backward_tcgen05.cu) is the path; RT_ATTN_BACKWARD_IMPL=mma_sync keeps
    // this file's mma.sync kernel for comparisons, and it also serves shapes the other one does not cover.
    static const bool legacy = [] {
        const char* s = getenv("RT_ATTN_BACKWARD_IMPL");
        return s && s[0] == 'm';
    }();
    if (!legacy) {
        e = launch_backward_tcgen05(q, k, v, d_out, lse, delta_ws, dq, dk, dv, batch, heads, seq, dim, causal, scale, stream);
        if (e != cudaErrorNotSupported) return e;
    }
    BwdTcParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                  (const __nv_bfloat16*)d_out, lse, delta_ws, dq, dk, dv, seq, causal, scale, scale * kLog2e};
    if (dim == 128) return launch_bwd_tc<128>(p, bh, stream);
    if (dim == 64) return launch_bwd_tc<64>(p, bh, stream);
    return cudaErrorInvalidValue;
}

}  // namespace rt
