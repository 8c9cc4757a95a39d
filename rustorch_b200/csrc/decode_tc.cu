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
    MergePush push; // world > 0: the merged rows (record layout, out_f32 = this rank's slot) also go to the peers
};

// Called by every CTA of a multi-chunk launch once its partial is written.  The CTA that completes
// its (sequence, KV head) group combines the group's chunk partials with the (m, l) merge of
// online_softmax.rs:105-131 and writes the final rows, so no separate merge launch is needed.
// The combine is spread over the CTA: chunk c goes to warp c % 4, each lane owns D/32 consecutive
// dims and keeps up to eight 16-byte loads in flight, the four warp sums meet in shared memory.
// Partials of other CTAs are read with cache-global loads after a device-scope fence.
// With p.push.world > 0 the launch is one rank of a split-KV decode: the rows are the rank's (O | LSE)
// record; the finishing CTA also stores them into the slot every peer keeps for this rank (one warp per
// peer in turn, 16-byte stores over NVLink, nothing is ever loaded from a peer), and the CTA that
// finishes the launch's last group raises every peer's flag with a system-scope release.
// scratch: G * n_chunks + 4 * G * D floats of shared memory (decode_merge_smem_bytes).
template <int D, int G>
__device__ __forceinline__ void finish_group(const DecodeTcParams& p, int b, int kvh, int64_t row0, float* scratch) {
    __shared__ int s_last;
    __shared__ float s_red[4][G];
    constexpr int VPL = D / 32;  // dims per lane
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = p.n_chunks;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(&p.counters[b * p.n_kv + kvh], 1) == n - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float* w_sm = scratch;                                   // [G][n]: LSE of (row, chunk), then its weight
    float* acc_sm = scratch + G * n;                         // [4 warps][G][D]
    float* stage = scratch + ((G * n + 4 * G * D + 3) & ~3);  // [G][D + 1]: the record rows on their way to the peers

    // ---- weights: per row the maximum LSE, exp(LSE_c - max) and their sum
    float mrow[G], lrow[G];
#pragma unroll
    for (int gg = 0; gg < G; ++gg) {
        float m = -INFINITY;
        for (int c = tid; c < n; c += 128) {
            const float x = __ldcg(p.part_lse + (int64_t)c * p.rows + row0 + gg);
            w_sm[gg * n + c] = x;
            m = fmaxf(m, x);
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(kFullMask, m, off));
        if (lane == 0) s_red[warp][gg] = m;
    }
    __syncthreads();
#pragma unroll
    for (int gg = 0; gg < G; ++gg) {
        const float m = fmaxf(fmaxf(s_red[0][gg], s_red[1][gg]), fmaxf(s_red[2][gg], s_red[3][gg]));
        mrow[gg] = m;
        float l = 0.f;
        if (m != -INFINITY) {
            for (int c = tid; c < n; c += 128) {  // the same thread wrote these entries above
                const float x = w_sm[gg * n + c];
                const float w = (x == -INFINITY) ? 0.f : expf(x - m);
                w_sm[gg * n + c] = w;
                l += w;
            }
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) l += __shfl_xor_sync(kFullMask, l, off);
        lrow[gg] = l;
    }
    __syncthreads();  // every thread has read the maxima: s_red is free for the sums; weights are visible
#pragma unroll
    for (int gg = 0; gg < G; ++gg)
        if (lane == 0) s_red[warp][gg] = lrow[gg];

    // ---- weighted sum of the partial rows: warp x takes chunks x, x+4, ...
    float acc[G][VPL];
#pragma unroll
    for (int gg = 0; gg < G; ++gg)
#pragma unroll
        for (int i = 0; i < VPL; ++i) acc[gg][i] = 0.f;
    const int64_t cs = p.rows * D;  // floats between consecutive chunks of part_o
    const float* src = p.part_o + row0 * D + lane * VPL;
    constexpr int kLoadsPerChunk = G * (VPL >= 4 ? VPL / 4 : 1);         // 16-byte (8-byte at D = 64) loads per lane
    constexpr int kInFlight = kLoadsPerChunk >= 8 ? 1 : 8 / kLoadsPerChunk;  // chunks loaded per round
    for (int c0 = warp; c0 < n; c0 += 4 * kInFlight) {
        float v[kInFlight][G][VPL], wgt[kInFlight][G];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const int c = c0 + 4 * u;
#pragma unroll
            for (int gg = 0; gg < G; ++gg) {
                wgt[u][gg] = (c < n && mrow[gg] != -INFINITY) ? w_sm[gg * n + c] : 0.f;
                const float* q = src + (int64_t)c * cs + gg * D;
                if (wgt[u][gg] != 0.f) {  // an empty chunk's partial row may be uninitialised
                    if constexpr (VPL == 2) {
                        const float2 t = __ldcg(reinterpret_cast<const float2*>(q));
                        v[u][gg][0] = t.x; v[u][gg][1] = t.y;
                    } else {
#pragma unroll
                        for (int i = 0; i < VPL; i += 4) {
                            const float4 t = __ldcg(reinterpret_cast<const float4*>(q + i));
                            v[u][gg][i] = t.x; v[u][gg][i + 1] = t.y; v[u][gg][i + 2] = t.z; v[u][gg][i + 3] = t.w;
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < VPL; ++i) v[u][gg][i] = 0.f;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u)
#pragma unroll
            for (int gg = 0; gg < G; ++gg)
#pragma unroll
                for (int i = 0; i < VPL; ++i) acc[gg][i] = fmaf(wgt[u][gg], v[u][gg][i], acc[gg][i]);
    }
#pragma unroll
    for (int gg = 0; gg < G; ++gg)
#pragma unroll
        for (int i = 0; i < VPL; ++i) acc_sm[(warp * G + gg) * D + lane * VPL + i] = acc[gg][i];
    __syncthreads();

    // ---- final rows: O = sum of the four warp sums / l, LSE = m + ln l
    const bool do_push = p.push.world > 0;
    for (int i = tid; i < G * D; i += 128) {
        const int gg = i / D, d = i % D;
        const float l = (s_red[0][gg] + s_red[1][gg]) + (s_red[2][gg] + s_red[3][gg]);
        const float sum = (acc_sm[(0 * G + gg) * D + d] + acc_sm[(1 * G + gg) * D + d]) +
                          (acc_sm[(2 * G + gg) * D + d] + acc_sm[(3 * G + gg) * D + d]);
        const float outv = (l > 0.f) ? sum / l : 0.f;
        const int64_t row = row0 + gg;
        if (p.out_bf16) p.out_bf16[row * D + d] = __float2bfloat16(outv);
        if (p.out_f32) p.out_f32[row * p.of_stride + d] = outv;
        if (do_push) stage[gg * (D + 1) + d] = outv;
    }
    if (tid < G) {
        const float l = (s_red[0][tid] + s_red[1][tid]) + (s_red[2][tid] + s_red[3][tid]);
        const float lse = (l > 0.f) ? mrow[tid] + logf(l) : -INFINITY;
        if (p.lse) p.lse[(row0 + tid) * p.lse_stride] = lse;
        if (do_push) stage[tid * (D + 1) + D] = lse;
    }
    if (!do_push) return;

    // ---- delivery: the G record rows are contiguous ([rows, D + 1] layout) and 16-byte aligned as a block
    // when G * (D + 1) is a multiple of 4 (checked by the launcher)
    __syncthreads();
    {
        const float4* stage4 = reinterpret_cast<const float4*>(stage);
        constexpr int kVec = G * (D + 1) / 4;
        for (int r = warp; r < p.push.world; r += 4) {
            float* base = p.push.dst[r];
            if (base == p.out_f32) continue;  // this rank's own slot was written above
            float4* dst = reinterpret_cast<float4*>(base + row0 * (D + 1));
            for (int i = lane; i < kVec; i += 32) dst[i] = stage4[i];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        const int groups = (int)(p.rows / G);
        if (atomicAdd(p.push.done_counter, 1) == groups - 1) {
            *p.push.done_counter = 0;  // ready for the next launch
            __threadfence_system();    // the rows of every group are ordered before the flags
            for (int r = 0; r < p.push.world; ++r)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.push.flag[r]), "r"(p.push.epoch) : "memory");
        }
    }
}

// Shared memory finish_group needs: weights, four warp sums, the staged record rows.
static size_t decode_merge_smem_bytes(int G, int D, int n_chunks) {
    return sizeof(float) * ((size_t)G * (size_t)n_chunks + 4 * (size_t)G * (size_t)D + 4 + (size_t)G * (size_t)(D + 1));
}

__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

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

    // Launched with programmatic stream serialisation, the CTA may be resident before the kernel ahead of it in
    // the stream has finished (the append of this token's K and V rows, the previous step's merge): this
    // returns once that kernel has completed and its writes are visible (at once under a normal launch).
    // Nothing is read from global memory before it.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    int64_t len = p.kv_lens ? (int64_t)p.kv_lens[b] : p.kv_len_uniform;
    if (len > p.max_seq) len = p.max_seq;
    const int64_t hi = (p.kv_end >= 0 && p.kv_end < len) ? p.kv_end : len;
    const int64_t c0 = p.kv_begin + (int64_t)chunk_idx * p.chunk;
    int64_t c1 = c0 + p.chunk;
    if (c1 > hi) c1 = hi;

    if (c0 >= c1) {  // nothing visible in this chunk: identity partial
        launch_dependents();
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

    // This CTA has streamed its share of the cache: a kernel launched behind this one with programmatic
    // stream serialisation (the cross-rank merge, which only waits on flags) may be scheduled once every CTA
    // has got here, instead of after the whole grid has drained.
    launch_dependents();

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
    // RT_ATTN_DECODE_PDL=0 launches without programmatic stream serialisation.
    static const bool pdl = [] {
        const char* e = getenv("RT_ATTN_DECODE_PDL");
        return !(e && e[0] == '0');
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.n_chunks, p.n_kv, (unsigned)batch);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = DecodeTcCfg<D>::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kern, mk, mv, p);
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
                                 int64_t of_stride, int64_t lse_stride, bool* merged, const MergePush* push,
                                 cudaStream_t stream) {
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
    // The CTA that completes a (sequence, KV head) group can merge the group's chunk partials itself
    // (finish_group), which makes a multi-chunk decode one kernel.  It costs a memset node for the counters
    // and a tail in which one CTA per group works alone, so it is used where that is cheaper than a second
    // launch: grids of several waves with few chunks per group (batched decode), and launches whose rows
    // also go to the peers of a split-KV decode, where it also replaces the copy kernel.  A small batch-1
    // launch is latency-bound and keeps the separate merge kernel.  RT_ATTN_DECODE_FUSED_MERGE=0 forces the
    // separate kernel everywhere.  The merge scratch must fit the (then idle) ring, and rows delivered to
    // peers must be 16-byte aligned group by group (group size 4 or 8).
    static const bool fused_off = [] {
        const char* s = getenv("RT_ATTN_DECODE_FUSED_MERGE");
        return s && s[0] == '0';
    }();
    const int group = n_heads / n_kv;
    const size_t ring = head_dim == 256 ? DecodeTcCfg<256>::RING_BYTES
                                        : head_dim == 128 ? DecodeTcCfg<128>::RING_BYTES : DecodeTcCfg<64>::RING_BYTES;
    const bool fits = decode_merge_smem_bytes(group, head_dim, n_chunks) <= ring;
    const bool pushing = push && push->world > 0;
    // Delivery from inside the decode kernel is built and tested but measured slower than the chunk-merge
    // kernel delivering the rows (its tail is one CTA per group); RT_ATTN_DECODE_PUSH_IN_KERNEL=1 selects it.
    static const bool push_in_kernel = [] {
        const char* s = getenv("RT_ATTN_DECODE_PUSH_IN_KERNEL");
        return s && s[0] == '1';
    }();
    const bool push_ok = pushing && push_in_kernel && group % 4 == 0 && out_f32 && of_stride == head_dim + 1;
    constexpr int kMaxFusedChunks = 8;
    const bool many_ctas = batch * n_kv * (int64_t)n_chunks >= 4 * (int64_t)sm_count();
    const bool batched = n_chunks <= kMaxFusedChunks && many_ctas && !pushing;
    p.counters = (n_chunks > 1 && fits && (batched || push_ok) && !fused_off) ? counters : nullptr;
    p.push = MergePush{};
    if (p.counters) {
        cudaError_t e = cudaMemsetAsync(p.counters, 0, sizeof(int) * (size_t)batch * n_kv, stream);
        if (e != cudaSuccess) return e;
        *merged = true;
        if (push) p.push = *push;
    }
    return head_dim == 256   ? launch_d<256>(mk, mv, p, n_heads / n_kv, batch, stream)
           : head_dim == 128 ? launch_d<128>(mk, mv, p, n_heads / n_kv, batch, stream)
                             : launch_d<64>(mk, mv, p, n_heads / n_kv, batch, stream);
}

}  // namespace rt
