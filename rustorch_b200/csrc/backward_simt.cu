// f32 flash-attention backward on CUDA cores: (dQ, dK, dV) from Q, K, V, O, dO and the saved
// row statistics LSE = m + ln(l) of the forward pass.
//
// Replaces rustorch_attention::flash_backward (crates/rustorch-attention/src/cpu_backward.rs:46-185),
// which recomputes the full N x N probability matrix per (batch, head).  Same math (:16-27):
//   P = exp(scale * Q K^T - LSE),  dV = P^T dO,  dP = dO V^T,
//   dS = P o (dP - delta),  delta_i = sum_j P_ij dP_ij = dO_i . O_i,
//   dQ = scale * dS K,  dK = scale * dS^T Q
// evaluated tile by tile, so nothing of size N x N is stored.  Two deterministic passes (no
// atomics): one warp per query row accumulates dQ_i over key tiles, then one warp per key row
// accumulates dK_j and dV_j over query tiles; each pass recomputes the scores it needs.  The lane
// index runs over the 32 rows of the opposite tile, which sit in shared memory with a padded
// pitch.  A causal launch skips the tiles above the diagonal.
#include "common.cuh"
#include "kernels.h"

namespace rt {

constexpr int kBwdRows = 8;    // rows (warps) per CTA
constexpr int kBwdTile = 32;   // rows of the opposite operand per tile (one per lane)

struct BwdParams {
    const float *q, *k, *v, *out, *d_out, *lse;
    float *dq, *dk, *dv, *delta;
    int64_t seq;
    int dim, causal;
    float scale;
};

// delta_i = dO_i . O_i (the row sum of P o dP), one warp per row.
__global__ void __launch_bounds__(256) bwd_delta_kernel(const float* __restrict__ out, const float* __restrict__ d_out,
                                                        float* __restrict__ delta, int64_t rows, int dim) {
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    float acc = 0.f;
    for (int d = lane; d < dim; d += 32) acc = fmaf(out[row * dim + d], d_out[row * dim + d], acc);
#pragma unroll
    for (int off = 16; off; off >>= 1) acc += __shfl_xor_sync(kFullMask, acc, off);
    if (lane == 0) delta[row] = acc;
}

// Pass over the rows of one side (kQuerySide: a warp owns query row i and walks key tiles to form
// dQ_i; otherwise it owns key row j and walks query tiles to form dK_j and dV_j).
template <bool kQuerySide>
__global__ void __launch_bounds__(kBwdRows * 32) bwd_pass_kernel(const BwdParams p) {
    extern __shared__ float smem[];
    const int D = p.dim;
    const int P1 = D + 1;
    float* tA = smem;                        // [32][D+1]  K tile (query side) / Q tile (key side)
    float* tB = tA + kBwdTile * P1;          // [32][D+1]  V tile               / dO tile
    float* rA = tB + kBwdTile * P1;          // [rows][D]  Q rows               / K rows
    float* rB = rA + kBwdRows * D;           // [rows][D]  dO rows              / V rows
    float* tLse = rB + kBwdRows * D;         // [32]  (key side) LSE of the tile's query rows
    float* tDelta = tLse + kBwdTile;         // [32]  (key side) delta of the tile's query rows

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t bh = blockIdx.y;
    const int64_t N = p.seq;
    const int64_t row0 = (int64_t)blockIdx.x * kBwdRows;
    const int64_t r = row0 + warp;           // the row this warp owns
    const bool row_valid = r < N;
    const int64_t base = bh * N * D;

    const float* ownA = (kQuerySide ? p.q : p.k) + base;
    const float* ownB = (kQuerySide ? p.d_out : p.v) + base;
    const float* othA = (kQuerySide ? p.k : p.q) + base;
    const float* othB = (kQuerySide ? p.v : p.d_out) + base;

    for (int i = threadIdx.x; i < kBwdRows * D; i += blockDim.x) {
        const int64_t rr = row0 + i / D;
        rA[i] = rr < N ? ownA[rr * D + i % D] : 0.f;
        rB[i] = rr < N ? ownB[rr * D + i % D] : 0.f;
    }
    float own_lse = 0.f, own_delta = 0.f;
    if (kQuerySide && row_valid) {
        own_lse = p.lse[bh * N + r];
        own_delta = p.delta[bh * N + r];
    }

    // tile range of the opposite side that this CTA's rows can see / be seen by
    int64_t t_lo = 0, t_hi = N;
    if (p.causal) {
        if (kQuerySide) {
            t_hi = row0 + kBwdRows < N ? row0 + kBwdRows : N;  // keys <= last query row of the CTA
        } else {
            t_lo = (row0 / kBwdTile) * kBwdTile;               // queries >= first key row of the CTA
        }
    }

    float acc0[8], acc1[8];  // query side: dQ_i; key side: dK_j (acc0) and dV_j (acc1); d = lane + 32*t
#pragma unroll
    for (int t = 0; t < 8; ++t) acc0[t] = acc1[t] = 0.f;

    for (int64_t t0 = t_lo; t0 < t_hi; t0 += kBwdTile) {
        __syncthreads();
        for (int i = threadIdx.x; i < kBwdTile * D; i += blockDim.x) {
            const int rr = i / D, d = i % D;
            const bool in = t0 + rr < N;
            tA[rr * P1 + d] = in ? othA[(t0 + rr) * D + d] : 0.f;
            tB[rr * P1 + d] = in ? othB[(t0 + rr) * D + d] : 0.f;
        }
        if (!kQuerySide && threadIdx.x < kBwdTile) {
            const bool in = t0 + threadIdx.x < N;
            tLse[threadIdx.x] = in ? p.lse[bh * N + t0 + threadIdx.x] : 0.f;
            tDelta[threadIdx.x] = in ? p.delta[bh * N + t0 + threadIdx.x] : 0.f;
        }
        __syncthreads();
        if (!row_valid) continue;

        const int64_t o = t0 + lane;  // the opposite row this lane handles
        const int64_t qi = kQuerySide ? r : o, kj = kQuerySide ? o : r;
        const float* a_own = rA + warp * D;
        const float* b_own = rB + warp * D;
        const float* a_oth = tA + lane * P1;
        const float* b_oth = tB + lane * P1;
        // s = q_i . k_j ; dp = dO_i . v_j  (query side: own = (q, dO), other = (k, v); key side: own = (k, v))
        float s = 0.f, dp = 0.f;
        for (int d = 0; d < D; ++d) {
            s = fmaf(a_own[d], a_oth[d], s);
            dp = fmaf(b_own[d], b_oth[d], dp);
        }
        const float lse = kQuerySide ? own_lse : tLse[lane];
        const float delta = kQuerySide ? own_delta : tDelta[lane];
        const bool visible = o < N && !(p.causal && kj > qi) && lse != -INFINITY;
        const float prob = visible ? expf(s * p.scale - lse) : 0.f;
        const float ds = prob * (dp - delta) * p.scale;

        if (kQuerySide) {
            // dQ_i += sum_j dS_ij K_j
            for (int jj = 0; jj < kBwdTile; ++jj) {
                const float w = __shfl_sync(kFullMask, ds, jj);
                const float* krow = tA + jj * P1;
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    const int d = lane + 32 * t;
                    if (d < D) acc0[t] = fmaf(w, krow[d], acc0[t]);
                }
            }
        } else {
            // dK_j += sum_i dS_ij Q_i ; dV_j += sum_i P_ij dO_i
            for (int ii = 0; ii < kBwdTile; ++ii) {
                const float w = __shfl_sync(kFullMask, ds, ii);
                const float pw = __shfl_sync(kFullMask, prob, ii);
                const float* qrow = tA + ii * P1;
                const float* dorow = tB + ii * P1;
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    const int d = lane + 32 * t;
                    if (d < D) {
                        acc0[t] = fmaf(w, qrow[d], acc0[t]);
                        acc1[t] = fmaf(pw, dorow[d], acc1[t]);
                    }
                }
            }
        }
    }

    if (!row_valid) return;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        const int d = lane + 32 * t;
        if (d < D) {
            if (kQuerySide) {
                p.dq[base + r * D + d] = acc0[t];
            } else {
                p.dk[base + r * D + d] = acc0[t];
                p.dv[base + r * D + d] = acc1[t];
            }
        }
    }
}

cudaError_t launch_backward_f32(const float* q, const float* k, const float* v, const float* out, const float* d_out,
                                const float* lse, float* dq, float* dk, float* dv, float* delta_ws, int64_t batch,
                                int64_t heads, int64_t seq, int dim, int causal, float scale, cudaStream_t stream) {
    const int64_t bh = batch * heads;
    if (bh == 0 || seq == 0) return cudaSuccess;
    if (bh > 65535) return cudaErrorInvalidValue;
    const int64_t rows = bh * seq;
    bwd_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(out, d_out, delta_ws, rows, dim);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    BwdParams p{q, k, v, out, d_out, lse, dq, dk, dv, delta_ws, seq, dim, causal, scale};
    const size_t smem = sizeof(float) * ((size_t)2 * kBwdTile * (dim + 1) + (size_t)2 * kBwdRows * dim + 2 * kBwdTile);
    e = cudaFuncSetAttribute(bwd_pass_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(bwd_pass_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dim3 grid((unsigned)((seq + kBwdRows - 1) / kBwdRows), (unsigned)bh);
    bwd_pass_kernel<true><<<grid, kBwdRows * 32, smem, stream>>>(p);
    bwd_pass_kernel<false><<<grid, kBwdRows * 32, smem, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace rt
