// Split-KV GQA decode, TMA-staged and tensor-core assisted (head dim 64, 128 or 256).
//
// Same contract and partial format as gqa_decode_splitkv_kernel (decode.cu) — it replaces the
// reference's per-head scalar decode kernels (crates/rustorch-cuda/src/llm_kernels.rs:376-536)
// and decode_attn_row (crates/rustorch-nn/src/gqa.rs:216-270) — but built to be limited by HBM
// rather than by instruction issue:
//   * K and V rows travel global -> shared memory as TMA tiles (16 tokens x 64 dims, 128-byte
//     swizzle) through a per-warp ring of mbarrier-tracked stages, so many kilobytes per SM are
//     in flight without holding registers;
//   * q.k and p.v run on mma.sync.m16n8k16 (bf16 in, f32 accumulate): M = the G <= 8 query heads
//     of the GQA group (padded to 16), N = 8 tokens (scores) or 8 dims (output), fragments
//     fetched with ldmatrix (transposed for V), about 5 warp instructions per 512-byte token row;
//   * online softmax in the log2 domain on the accumulator fragments; the O rescale is skipped
//     (warp-uniformly) when no row maximum moved.
// One CTA = 4 independent warps = one (sequence, KV head, chunk); warp states are merged through
// shared memory and written as a normalised (O f32, LSE) partial, or as the final output when
// the launch has a single chunk.  Rows past the visible range are masked in the scores and
// zeroed in V (uninitialised cache memory may hold NaN bit patterns).  Waits are bounded.
#include <cuda.h>
#include <cstdlib>

#include "kernels.h"
#include "mma_sync.cuh"
#include "tc_ptx.cuh"
#include "tensor_map.h"

namespace rt {

using namespace ptx;

struct DecodeTcParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out_bf16;
    float* out_f32;
    float* lse;
    float* part_o;
    float* part_lse;
    const int32_t* kv_lens;
    int64_t kv_len_uniform;
    int64_t kv_begin, kv_end;
    int64_t max_seq;
    int n_heads, n_kv;
    int chunk, n_chunks;
    int64_t rows;
    int64_t of_stride, lse_stride;  // floats between consecutive rows of out_f32 / lse
    float scale_log2;
    int* status;
    int* counters;  // NULL, or [B * Hkv] zeroed before the launch: the last chunk of a group merges its partials
};

// Called by every CTA of a multi-chunk launch once its partial is written.  The CTA that completes
// its (sequence, KV head) group combines the group's chunk partials with the (m, l) merge of
// online_softmax.rs:105-131 and writes the final rows, so no separate merge launch is needed:
// for short chunks that launch costs as much as the streaming itself.  Partials of other CTAs are
// read with cache-global loads after a device-scope fence.
template <int D, int G>
__device__ __forceinline__ void finish_group(const DecodeTcParams& p, int b, int kvh, int64_t row0, float* scratch) {
    __shared__ int s_last;
    __shared__ float s_red[4];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(&p.counters[b * p.n_kv + kvh], 1) == p.n_chunks - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float* w_sm = scratch;  // [n_chunks]
    for (int gg = 0; gg < G; ++gg) {
        const int64_t row = row0 + gg;
        float m = -INFINITY;
        for (int c = tid; c < p.n_chunks; c += 128) {
            const float x = __ldcg(p.part_lse + (int64_t)c * p.rows + row);
            w_sm[c] = x;
            m = fmaxf(m, x);
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(kFullMask, m, off));
        __syncthreads();  // s_red free (previous row), w_sm written
        if (lane == 0) s_red[warp] = m;
        __syncthreads();
        m = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
        float l = 0.f;
        if (m != -INFINITY) {
            for (int c = tid; c < p.n_chunks; c += 128) {
                const float x = w_sm[c];
                const float w = (x == -INFINITY) ? 0.f : expf(x - m);
                w_sm[c] = w;
                l += w;
            }
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) l += __shfl_xor_sync(kFullMask, l, off);
        __syncthreads();  // everyone has read s_red (max); weights written
        if (lane == 0) s_red[warp] = l;
        __syncthreads();
        l = (s_red[0] + s_red[1]) + (s_red[2] + s_red[3]);
        const float inv = (l > 0.f) ? 1.f / l : 0.f;
        for (int d = tid; d < D; d += 128) {
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            if (l > 0.f) {
                const float* src = p.part_o + row * D + d;
                const int64_t cs = p.rows * D;
                int c = 0;
                for (; c + 4 <= p.n_chunks; c += 4) {  // four independent loads in flight; empty chunks may be uninitialised
                    const float w0 = w_sm[c], w1 = w_sm[c + 1], w2 = w_sm[c + 2], w3 = w_sm[c + 3];
                    const float x0 = w0 != 0.f ? __ldcg(src + (int64_t)c * cs) : 0.f;
                    const float x1 = w1 != 0.f ? __ldcg(src + (int64_t)(c + 1) * cs) : 0.f;
                    const float x2 = w2 != 0.f ? __ldcg(src + (int64_t)(c + 2) * cs) : 0.f;
                    const float x3 = w3 != 0.f ? __ldcg(src + (int64_t)(c + 3) * cs) : 0.f;
                    a0 = fmaf(w0, x0, a0);
                    a1 = fmaf(w1, x1, a1);
                    a2 = fmaf(w2, x2, a2);
                    a3 = fmaf(w3, x3, a3);
                }
                for (; c < p.n_chunks; ++c) {
                    const float w0 = w_sm[c];
                    if (w0 != 0.f) a0 = fmaf(w0, __ldcg(src + (int64_t)c * cs), a0);
                }
            }
            const float outv = ((a0 + a1) + (a2 + a3)) * inv;
            if (p.out_bf16) p.out_bf16[row * D + d] = __float2bfloat16(outv);
            if (p.out_f32) p.out_f32[row * p.of_stride + d] = outv;
        }
        if (tid == 0 && p.lse) p.lse[row * p.lse_stride] = (l > 0.f) ? m + logf(l) : -INFINITY;
        __syncthreads();  // w_sm and s_red are reused by the next row
    }
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

template <int D>
struct DecodeTcCfg {
    static constexpr int NW = 4;               // warps per CTA
    static constexpr int BLK = 16;             // tokens per warp step (one MMA K extent of P.V)
    static constexpr int STAGES = 3;
    static constexpr int NSUB = D / 64;        // 64-column swizzled boxes per row
    static constexpr int BOX_BYTES = BLK * 128;             // 16 rows x 128 B
    static constexpr int KV_BYTES = NSUB * BOX_BYTES;        // K (or V) of one block
    static constexpr int STAGE_BYTES = 2 * KV_BYTES;
    static constexpr int RING_BYTES = NW * STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = RING_BYTES + NW * STAGES * 8 + 1024;
};

enum { kToDecFull = 301 };

template <int D, int G>
__global__ void __launch_bounds__(128, 2)
gqa_decode_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const DecodeTcParams p) {
    using C = DecodeTcCfg<D>;
    constexpr int NW = C::NW, BLK = C::BLK, STAGES = C::STAGES, NSUB = C::NSUB;
    constexpr int NT = D / 8;  // output n-tiles (8 dims each)

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::RING_BYTES);

    const int chunk_idx = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tig = lane & 3;  // mma fragment coordinates: g = head row, tig = column pair
    const int64_t row0 = (int64_t)b * p.n_heads + (int64_t)kvh * G;
    const bool direct = (p.n_chunks == 1);

    int64_t len = p.kv_lens ? (int64_t)p.kv_lens[b] : p.kv_len_uniform;
    if (len > p.max_seq) len = p.max_seq;
    const int64_t hi = (p.kv_end >= 0 && p.kv_end < len) ? p.kv_end : len;
    const int64_t c0 = p.kv_begin + (int64_t)chunk_idx * p.chunk;
    int64_t c1 = c0 + p.chunk;
    if (c1 > hi) c1 = hi;

    if (c0 >= c1) {  // nothing visible in this chunk: identity partial
        if (direct) {
            for (int i = tid; i < G * D; i += 128) {
                const int64_t o = (row0 + i / D) * D + i % D;
                if (p.out_bf16) p.out_bf16[o] = __float2bfloat16(0.f);
                if (p.out_f32) p.out_f32[(row0 + i / D) * p.of_stride + i % D] = 0.f;
            }
            if (tid < G && p.lse) p.lse[(row0 + tid) * p.lse_stride] = -INFINITY;
        } else if (tid < G) {
            p.part_lse[(int64_t)chunk_idx * p.rows + row0 + tid] = -INFINITY;
        }
        if (!direct && p.counters) finish_group<D, G>(p, b, kvh, row0, reinterpret_cast<float*>(smem));
        return;
    }

    uint8_t* ring = smem + warp * (STAGES * C::STAGE_BYTES);
    uint64_t* full = bars + warp * STAGES;
    if (lane == 0) {
        if (warp == 0) {
            prefetch_tensormap(&tm_k);
            prefetch_tensormap(&tm_v);
        }
        for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncwarp();

    // Q fragments of the group's heads (A operand rows 0..G-1; rows G..15 are zero).
    uint32_t qa[D / 16][2];
    {
        const __nv_bfloat16* qrow = p.q + (row0 + g) * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            qa[ks][0] = (g < G) ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + tig * 2) : 0u;
            qa[ks][1] = (g < G) ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + tig * 2) : 0u;
        }
    }

    // This warp's blocks: block i covers tokens [c0 + (i*NW + warp)*BLK, +BLK).
    const int64_t span = c1 - c0;
    const int n_blocks_cta = (int)((span + BLK - 1) / BLK);
    const int n_my = (n_blocks_cta > warp) ? (n_blocks_cta - warp + NW - 1) / NW : 0;
    const int64_t cache_row0 = ((int64_t)b * p.n_kv + kvh) * p.max_seq;

    auto issue = [&](int it) {  // lane 0 only
        const int st = it % STAGES;
        const int64_t t0 = c0 + ((int64_t)it * NW + warp) * BLK;
        uint8_t* dst = ring + st * C::STAGE_BYTES;
        mbar_arrive_expect_tx(&full[st], C::STAGE_BYTES);
#pragma unroll
        for (int s = 0; s < NSUB; ++s) {
            tma_load_2d(dst + s * C::BOX_BYTES, &tm_k, &full[st], s * 64, (int)(cache_row0 + t0));
            tma_load_2d(dst + C::KV_BYTES + s * C::BOX_BYTES, &tm_v, &full[st], s * 64, (int)(cache_row0 + t0));
        }
    };
    int issued_upto = -1;  // lane 0: highest iteration whose loads have been issued
    if (lane == 0)
        for (int it = 0; it < STAGES && it < n_my; ++it) {
            issue(it);
            issued_upto = it;
        }

    float m_run = -INFINITY, l_part = 0.f;  // state of head g (all four lanes of a group agree on m_run)
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

    bool ok = true;
    for (int it = 0; it < n_my; ++it) {
        const int st = it % STAGES;
        const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
        if (!__all_sync(kFullMask, mbar_wait(&full[st], ph, p.status, kToDecFull))) {
            ok = false;
            break;
        }
        const int64_t t0 = c0 + ((int64_t)it * NW + warp) * BLK;
        const int valid = (int)((c1 - t0 < BLK) ? (c1 - t0) : BLK);
        uint8_t* kst = ring + st * C::STAGE_BYTES;
        uint8_t* vst = kst + C::KV_BYTES;
        if (valid < BLK) {  // zero the V rows past the visible range (may hold NaN bit patterns)
            for (int i = lane; i < (BLK - valid) * NSUB * 8; i += 32) {
                const int r = valid + i / (NSUB * 8), rem = i % (NSUB * 8);
                *reinterpret_cast<uint4*>(vst + (rem / 8) * C::BOX_BYTES + r * 128 + (rem % 8) * 16) =
                    make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }
        const uint32_t k_a = smem_u32(kst), v_a = smem_u32(vst);

        // ---- S[heads x 16 tokens] = Q K^T : two 8-token tiles, D/16 k-steps each
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const int r = lane & 7, mtx = lane >> 3;  // ldmatrix: this lane addresses row r of matrix mtx
#pragma unroll
            for (int kp = 0; kp < D / 32; ++kp) {     // two k-steps (32 dims = 4 chunks of 16 B) per ldmatrix.x4
                const int sub = kp / 2, chunk = (kp % 2) * 4 + mtx;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(k_a + sub * C::BOX_BYTES + r * 128 + ((chunk ^ r) << 4), b0, b1, b2, b3);
                mma_16816(s0, qa[2 * kp][0], qa[2 * kp][1], b0, b1);
                mma_16816(s0, qa[2 * kp + 1][0], qa[2 * kp + 1][1], b2, b3);
                ldmatrix_x4(k_a + sub * C::BOX_BYTES + (8 + r) * 128 + ((chunk ^ r) << 4), b0, b1, b2, b3);
                mma_16816(s1, qa[2 * kp][0], qa[2 * kp][1], b0, b1);
                mma_16816(s1, qa[2 * kp + 1][0], qa[2 * kp + 1][1], b2, b3);
            }
        }

        // ---- online softmax for head g over tokens {tig*2, tig*2+1, 8+tig*2, 8+tig*2+1}
        float sc[4];
        sc[0] = (tig * 2 < valid) ? s0[0] * p.scale_log2 : -INFINITY;
        sc[1] = (tig * 2 + 1 < valid) ? s0[1] * p.scale_log2 : -INFINITY;
        sc[2] = (8 + tig * 2 < valid) ? s1[0] * p.scale_log2 : -INFINITY;
        sc[3] = (8 + tig * 2 + 1 < valid) ? s1[1] * p.scale_log2 : -INFINITY;
        float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        if (__any_sync(kFullMask, m_new != m_run)) {
            const float alpha = fast_exp2(m_run - m_use);  // m_run = -inf -> 0 (O and l are 0 then)
            l_part *= alpha;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                o[j][0] *= alpha;
                o[j][1] *= alpha;
            }
            m_run = m_new;
        }
        const float p0 = fast_exp2(sc[0] - m_use), p1 = fast_exp2(sc[1] - m_use);
        const float p2 = fast_exp2(sc[2] - m_use), p3 = fast_exp2(sc[3] - m_use);
        l_part += (p0 + p1) + (p2 + p3);
        const uint32_t pa0 = float2_to_bf16x2(p0, p1);  // A fragment: tokens tig*2, tig*2+1
        const uint32_t pa2 = float2_to_bf16x2(p2, p3);  //             tokens 8+tig*2, 8+tig*2+1

        // ---- O[heads x D] += P V : D/8 n-tiles, one k-step of 16 tokens
        {
            const int r = lane & 7, mtx = lane >> 3;
            const int trow = (mtx & 1) * 8 + r;  // matrices 0,2: tokens 0-7; 1,3: tokens 8-15
#pragma unroll
            for (int jp = 0; jp < NT / 2; ++jp) {  // two n-tiles per ldmatrix.x4.trans
                const int ch = jp * 2 + (mtx >> 1);  // 16-byte chunk (8 dims) across the row
                const int sub = ch / 8, chunk = ch % 8;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(v_a + sub * C::BOX_BYTES + trow * 128 + ((chunk ^ (trow & 7)) << 4), b0, b1, b2, b3);
                mma_16816(o[2 * jp], pa0, pa2, b0, b1);
                mma_16816(o[2 * jp + 1], pa0, pa2, b2, b3);
            }
        }

        __syncwarp();
        if (lane == 0 && it + STAGES < n_my) {
            fence_proxy_async();  // order this warp's reads of the stage before the refill
            issue(it + STAGES);
            issued_upto = it + STAGES;
        }
    }
    if (!ok && lane == 0) {
        // Drain: every copy this warp issued must land before the ring is reused below and before the
        // CTA may exit.  The last load into stage s was iteration `last`; it completes phase last/STAGES
        // of that stage's barrier, so that parity (and no other) is what to wait for, bounded.
        const int issued = issued_upto + 1;  // iterations 0 .. issued-1 have loads in flight or landed
        for (int s = 0; s < STAGES; ++s) {
            if (issued <= s) continue;  // this stage was never loaded
            const int last = s + ((issued - 1 - s) / STAGES) * STAGES;
            const uint32_t par = (uint32_t)(last / STAGES) & 1u;
            const long long t0 = clock64();
            while (!mbar_try_wait(&full[s], par) && clock64() - t0 < (1ll << 28)) {
            }
        }
    }

    // ---- merge the four warp states through shared memory (the ring is idle now)
    l_part += __shfl_xor_sync(kFullMask, l_part, 1);
    l_part += __shfl_xor_sync(kFullMask, l_part, 2);
    __syncthreads();
    float* sm_o = reinterpret_cast<float*>(smem);  // [NW][G][D]
    float* sm_m = sm_o + NW * G * D;               // [NW][G]
    float* sm_l = sm_m + NW * G;                   // [NW][G]
    if (g < G) {
        if (tig == 0) {
            sm_m[warp * G + g] = m_run;
            sm_l[warp * G + g] = l_part;
        }
#pragma unroll
        for (int j = 0; j < NT; ++j)
            *reinterpret_cast<float2*>(&sm_o[(warp * G + g) * D + j * 8 + tig * 2]) = make_float2(o[j][0], o[j][1]);
    }
    __syncthreads();
    for (int i = tid; i < G * D; i += 128) {
        const int gg = i / D, d = i % D;
        float m = -INFINITY;
#pragma unroll
        for (int x = 0; x < NW; ++x) m = fmaxf(m, sm_m[x * G + gg]);
        float l = 0.f, acc = 0.f;
        if (m != -INFINITY) {
#pragma unroll
            for (int x = 0; x < NW; ++x) {
                const float w = fast_exp2(sm_m[x * G + gg] - m);
                l += w * sm_l[x * G + gg];
                acc += w * sm_o[(x * G + gg) * D + d];
            }
        }
        const float outv = (l > 0.f) ? acc / l : 0.f;
        const float lse = (l > 0.f) ? (m + fast_log2(l)) * kLn2 : -INFINITY;
        const int64_t row = row0 + gg;
        if (direct) {
            if (p.out_bf16) p.out_bf16[row * D + d] = __float2bfloat16(outv);
            if (p.out_f32) p.out_f32[row * p.of_stride + d] = outv;
            if (d == 0 && p.lse) p.lse[row * p.lse_stride] = lse;
        } else {
            p.part_o[((int64_t)chunk_idx * p.rows + row) * D + d] = outv;
            if (d == 0) p.part_lse[(int64_t)chunk_idx * p.rows + row] = lse;
        }
    }
    if (!direct && p.counters) {
        __syncthreads();  // the warp-merge scratch at the start of the ring is free again
        finish_group<D, G>(p, b, kvh, row0, reinterpret_cast<float*>(smem));
    }
}

// The cache viewed as a 2-D bf16 tensor [rows = B*Hkv*max_seq, D]; box = 16 rows x 64 columns.
static bool make_cache_map(CUtensorMap* map, const void* base, int64_t rows, int dim) {
    const uint64_t dims[2] = {(uint64_t)dim, (uint64_t)rows};
    const uint64_t strides[1] = {(uint64_t)dim * 2};
    const uint32_t box[2] = {64, 16};
    return encode_bf16_map_cached(map, 2, base, dims, strides, box);
}

template <int D, int G>
static cudaError_t launch_dg(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeTcParams& p, int64_t batch,
                             cudaStream_t stream) {
    auto kern = gqa_decode_tc_kernel<D, G>;
    cudaError_t e = set_max_dynamic_smem_once<gqa_decode_tc_kernel<D, G>>(DecodeTcCfg<D>::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    dim3 grid(p.n_chunks, p.n_kv, (unsigned)batch);
    kern<<<grid, 128, DecodeTcCfg<D>::SMEM_BYTES, stream>>>(mk, mv, p);
    return cudaGetLastError();
}

template <int D>
static cudaError_t launch_d(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeTcParams& p, int group,
                            int64_t batch, cudaStream_t stream) {
    switch (group) {
        case 1: return launch_dg<D, 1>(mk, mv, p, batch, stream);
        case 2: return launch_dg<D, 2>(mk, mv, p, batch, stream);
        case 4: return launch_dg<D, 4>(mk, mv, p, batch, stream);
        case 8: return launch_dg<D, 8>(mk, mv, p, batch, stream);
    }
    return cudaErrorInvalidValue;
}

// Returns cudaErrorNotSupported when this kernel does not cover the shape (the caller then
// uses the CUDA-core kernel).
cudaError_t launch_gqa_decode_tc(const void* q, const void* k, const void* v, void* out_bf16, float* out_f32,
                                 float* lse, int64_t batch, int n_heads, int n_kv, int head_dim, int64_t max_seq,
                                 const int32_t* kv_lens, int64_t kv_len_uniform, int64_t kv_begin, int64_t kv_end,
                                 float scale, float* part_o, float* part_lse, int* counters, int chunk, int n_chunks,
                                 int64_t of_stride, int64_t lse_stride, bool* merged, cudaStream_t stream) {
    *merged = false;
    const int64_t cache_rows = batch * n_kv * max_seq;
    if ((head_dim != 64 && head_dim != 128 && head_dim != 256) || cache_rows >= (1ll << 31) - 64)
        return cudaErrorNotSupported;
    CUtensorMap mk, mv;
    if (!make_cache_map(&mk, k, cache_rows, head_dim) || !make_cache_map(&mv, v, cache_rows, head_dim))
        return cudaErrorNotSupported;
    DecodeTcParams p;
    p.q = (const __nv_bfloat16*)q;
    p.out_bf16 = (__nv_bfloat16*)out_bf16;
    p.out_f32 = out_f32;
    p.lse = lse;
    p.part_o = part_o;
    p.part_lse = part_lse;
    p.kv_lens = kv_lens;
    p.kv_len_uniform = kv_len_uniform;
    p.kv_begin = kv_begin;
    p.kv_end = kv_end;
    p.max_seq = max_seq;
    p.n_heads = n_heads;
    p.n_kv = n_kv;
    p.chunk = chunk;
    p.n_chunks = n_chunks;
    p.rows = batch * n_heads;
    p.of_stride = of_stride;
    p.lse_stride = lse_stride;
    p.scale_log2 = scale * kLog2e;
    p.status = device_status_ptr();
    if (!p.status) return cudaErrorInvalidSymbol;
    // The in-kernel merge is serial per (sequence, KV head): worth it for the few chunks of a batched
    // decode (config 4 has at most 8), not for the dozens of chunks of one long sequence, which the
    // merge kernel spreads over many more threads (batch 1, kv_len 4096 = 32 chunks: 20.5 us fused,
    // 14.4 us with the merge kernel).
    constexpr int kMaxFusedChunks = 8;
    static const bool fused_off = [] {
        const char* s = getenv("RT_ATTN_DECODE_FUSED_MERGE");
        return s && s[0] == '0';
    }();
    // ... and only for grids of several waves: a small launch (batch 1) is latency-bound, and there the
    // memset node plus the serial tail cost more than the second launch (14.4 us against 10.3 us).
    const bool many_ctas = batch * n_kv * (int64_t)n_chunks >= 4 * (int64_t)sm_count();
    p.counters = (n_chunks > 1 && n_chunks <= kMaxFusedChunks && many_ctas && !fused_off) ? counters : nullptr;
    if (p.counters) {
        cudaError_t e = cudaMemsetAsync(p.counters, 0, sizeof(int) * (size_t)batch * n_kv, stream);
        if (e != cudaSuccess) return e;
        *merged = true;
    }
    return head_dim == 256   ? launch_d<256>(mk, mv, p, n_heads / n_kv, batch, stream)
           : head_dim == 128 ? launch_d<128>(mk, mv, p, n_heads / n_kv, batch, stream)
                             : launch_d<64>(mk, mv, p, n_heads / n_kv, batch, stream);
}

}  // namespace rt
