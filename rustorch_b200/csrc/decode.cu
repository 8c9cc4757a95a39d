// Split-KV GQA decode for a bf16 KV cache, plus the (O, LSE) merge kernel.
//
// Replaces the reference's one-CTA-per-query-head decode kernels
// (crates/rustorch-cuda/src/llm_kernels.rs:376-536) and the seq_q == 1 branch of
// gqa_forward_f32 (crates/rustorch-nn/src/gqa.rs:190-270).
//
// The path is HBM-bound (4 FLOP per KV byte at Hq/Hkv = 4), so the design is about
// streaming the cache once, fully coalesced, with many bytes in flight:
//   * one CTA per (sequence, KV head, KV chunk); the G = Hq/Hkv query heads of a group are
//     processed together so every K/V element is fetched once (the reference re-reads the
//     cache once per query head);
//   * a token row (D bf16) is spread over D/8 lanes, 16 bytes per lane, so one warp load
//     instruction covers 512 contiguous bytes; the next block of K and V rows is prefetched
//     into registers while the current one is consumed;
//   * the q.k partial sums of G heads x T tokens are reduced across the D/8 lanes with a
//     recursive-halving exchange (V-1 shuffles instead of V*log2(D/8)), which also leaves
//     exactly one (head, token) score per lane, so each exponential is evaluated once;
//   * per lane-group online softmax in the log2 domain with a warp-uniform lazy rescale;
//   * chunk results are written as normalised (O f32, LSE) partials and merged by
//     merge_partials_kernel, the same kernel that merges per-GPU partials.
#include "common.cuh"
#include "kernels.h"

namespace rt {

template <int D, int G>
struct DecodeCfg {
    static constexpr int LPT = D / 8;                 // lanes per token row
    static constexpr int TPI = 32 / LPT;              // token rows per warp load instruction
    static constexpr int T = (LPT / G >= 4) ? 4 : ((LPT / G >= 1) ? LPT / G : 1);  // rows per lane-group per step
    static constexpr int V = G * T;                   // scores reduced per step
    static constexpr int R = LPT / V;                 // replication of a score after the reduce
    static constexpr int TOK = TPI * T;               // token rows per warp step
    static constexpr int NW = 4;                      // warps per CTA
    static constexpr int NG = NW * TPI;               // lane-groups per CTA
    static_assert(V <= LPT, "scores per step must not exceed lanes per token");
};

struct DecodeParams {
    const __nv_bfloat16* q;
    const __nv_bfloat16* k;
    const __nv_bfloat16* v;
    __nv_bfloat16* out_bf16;
    float* out_f32;
    float* lse;
    float* part_o;    // [n_chunks, rows, D]
    float* part_lse;  // [n_chunks, rows]
    const int32_t* kv_lens;
    int64_t kv_len_uniform;
    int64_t kv_begin, kv_end;
    int64_t max_seq;
    int n_heads, n_kv;
    int chunk, n_chunks;
    int64_t rows;  // B * Hq
    int64_t of_stride, lse_stride;  // floats between consecutive rows of out_f32 / lse (D and 1 unless packed)
    float scale_log2;
};

template <int D, int G>
__global__ void __launch_bounds__(128) gqa_decode_splitkv_kernel(const DecodeParams p) {
    using C = DecodeCfg<D, G>;
    constexpr int LPT = C::LPT, TPI = C::TPI, T = C::T, V = C::V, R = C::R, TOK = C::TOK, NW = C::NW,
                  NG = C::NG;

    __shared__ float sm_m[NG][G];
    __shared__ float sm_l[NG][G];
    __shared__ __align__(16) float sm_o[NG][G][D];

    const int chunk_idx = blockIdx.x;
    const int kvh = blockIdx.y;
    const int b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gi = lane / LPT;   // lane-group within the warp
    const int lig = lane % LPT;  // lane within the group: owns dims [lig*8, lig*8+8)
    const int64_t row0 = (int64_t)b * p.n_heads + (int64_t)kvh * G;  // first output row of the group
    const bool direct = (p.n_chunks == 1);

    int64_t len = p.kv_lens ? (int64_t)p.kv_lens[b] : p.kv_len_uniform;
    if (len > p.max_seq) len = p.max_seq;
    int64_t hi = (p.kv_end >= 0 && p.kv_end < len) ? p.kv_end : len;
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
        return;
    }

    // q of the G heads, my 8 dims, pre-multiplied by scale*log2(e).
    float2 q2[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint4 w = *reinterpret_cast<const uint4*>(p.q + (row0 + g) * D + lig * 8);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = bf16x2_to_float2(ww[i]);
            q2[g][i] = make_float2(f.x * p.scale_log2, f.y * p.scale_log2);
        }
    }

    const __nv_bfloat16* kbase = p.k + ((int64_t)b * p.n_kv + kvh) * p.max_seq * D + lig * 8;
    const __nv_bfloat16* vbase = p.v + ((int64_t)b * p.n_kv + kvh) * p.max_seq * D + lig * 8;

    // Online-softmax state of this lane-group.  A lane tracks the head g_own of the one
    // score it receives from the reduce; O accumulators cover all G heads for my 8 dims.
    const int idx_own = lig / R;      // which of the V scores lands here
    const int g_own = idx_own / T;
    float m_run = -INFINITY;          // running max (log2 domain) of head g_own
    float l_part = 0.f;               // my share of the running sum of head g_own
    float2 o2[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i) o2[g][i] = make_float2(0.f, 0.f);

    uint4 kreg[T], vreg[T], knext[T], vnext[T];
    auto load_block = [&](int64_t tb, uint4(&kk)[T], uint4(&vv)[T]) {
#pragma unroll
        for (int j = 0; j < T; ++j) {
            const int64_t t = tb + j * TPI + gi;
            if (t < c1) {
                kk[j] = ld_stream_16B(kbase + t * D);
                vv[j] = ld_stream_16B(vbase + t * D);
            } else {
                kk[j] = make_uint4(0, 0, 0, 0);
                vv[j] = make_uint4(0, 0, 0, 0);
            }
        }
    };

    int64_t tb = c0 + (int64_t)warp * TOK;
    if (tb < c1) load_block(tb, knext, vnext);
    for (; tb < c1; tb += NW * TOK) {
#pragma unroll
        for (int j = 0; j < T; ++j) {
            kreg[j] = knext[j];
            vreg[j] = vnext[j];
        }
        if (tb + NW * TOK < c1) load_block(tb + NW * TOK, knext, vnext);

        // ---- scores: partial dot products over my 8 dims, then reduce across the group
        float s[V];
#pragma unroll
        for (int j = 0; j < T; ++j) {
            const uint32_t kw[4] = {kreg[j].x, kreg[j].y, kreg[j].z, kreg[j].w};
            float2 k2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) k2[i] = bf16x2_to_float2(kw[i]);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float2 acc = __fmul2_rn(q2[g][0], k2[0]);
#pragma unroll
                for (int i = 1; i < 4; ++i) acc = __ffma2_rn(q2[g][i], k2[i], acc);
                s[g * T + j] = acc.x + acc.y;
            }
        }
        {
            int n = V;
#pragma unroll
            for (int off = LPT / 2; off >= 1; off >>= 1) {
                if (n > 1) {
                    const bool up = (lig & off) != 0;
#pragma unroll
                    for (int i = 0; i < n / 2; ++i) {
                        const float send = up ? s[i] : s[i + n / 2];
                        const float keep = up ? s[i + n / 2] : s[i];
                        s[i] = keep + __shfl_xor_sync(kFullMask, send, off);
                    }
                    n /= 2;
                } else {
                    s[0] += __shfl_xor_sync(kFullMask, s[0], off);
                }
            }
        }
        // s[0] is now the full score of (head g_own, token slot j_own).
        const int j_own = idx_own % T;
        const int64_t t_own = tb + j_own * TPI + gi;
        float sc = (t_own < c1) ? s[0] : -INFINITY;

        // ---- online softmax for head g_own over the T tokens of this step
        float m_step = sc;
#pragma unroll
        for (int off = R; off < R * T; off <<= 1) m_step = fmaxf(m_step, __shfl_xor_sync(kFullMask, m_step, off));
        const float m_new = fmaxf(m_run, m_step);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float pexp = fast_exp2(sc - m_use);
        const bool changed = (m_new != m_run);
        if (__any_sync(kFullMask, changed)) {  // warp-uniform lazy rescale
            const float alpha = fast_exp2(m_run - m_use);  // m_run = -inf -> 0, O is 0 then anyway
            l_part *= alpha;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float a = __shfl_sync(kFullMask, alpha, (g * T) * R, LPT);
                const float2 a2 = make_float2(a, a);
#pragma unroll
                for (int i = 0; i < 4; ++i) o2[g][i] = __fmul2_rn(o2[g][i], a2);
            }
            m_run = m_new;
        }
        l_part += pexp;

        // ---- O += P V
#pragma unroll
        for (int j = 0; j < T; ++j) {
            const uint32_t vw[4] = {vreg[j].x, vreg[j].y, vreg[j].z, vreg[j].w};
            float2 v2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) v2[i] = bf16x2_to_float2(vw[i]);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float pj = __shfl_sync(kFullMask, pexp, (g * T + j) * R, LPT);
                const float2 p2 = make_float2(pj, pj);
#pragma unroll
                for (int i = 0; i < 4; ++i) o2[g][i] = __ffma2_rn(p2, v2[i], o2[g][i]);
            }
        }
    }

    // ---- merge the NG lane-group states of the CTA
#pragma unroll
    for (int off = R; off < R * T; off <<= 1) l_part += __shfl_xor_sync(kFullMask, l_part, off);
    const int grp = warp * TPI + gi;
    if (lig == (g_own * T) * R) {
        sm_m[grp][g_own] = m_run;
        sm_l[grp][g_own] = l_part;
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float4* dst = reinterpret_cast<float4*>(&sm_o[grp][g][lig * 8]);
        dst[0] = make_float4(o2[g][0].x, o2[g][0].y, o2[g][1].x, o2[g][1].y);
        dst[1] = make_float4(o2[g][2].x, o2[g][2].y, o2[g][3].x, o2[g][3].y);
    }
    __syncthreads();

    for (int i = tid; i < G * D; i += 128) {
        const int g = i / D, d = i % D;
        float m = -INFINITY;
#pragma unroll
        for (int x = 0; x < NG; ++x) m = fmaxf(m, sm_m[x][g]);
        float l = 0.f, o = 0.f;
        if (m != -INFINITY) {
#pragma unroll
            for (int x = 0; x < NG; ++x) {
                const float w = fast_exp2(sm_m[x][g] - m);  // -inf -> 0
                l += w * sm_l[x][g];
                o += w * sm_o[x][g][d];
            }
        }
        const float outv = (l > 0.f) ? o / l : 0.f;
        const float lse = (l > 0.f) ? (m + fast_log2(l)) * kLn2 : -INFINITY;
        const int64_t row = row0 + g;
        if (direct) {
            if (p.out_bf16) p.out_bf16[row * D + d] = __float2bfloat16(outv);
            if (p.out_f32) p.out_f32[row * p.of_stride + d] = outv;
            if (d == 0 && p.lse) p.lse[row * p.lse_stride] = lse;
        } else {
            p.part_o[((int64_t)chunk_idx * p.rows + row) * D + d] = outv;
            if (d == 0) p.part_lse[(int64_t)chunk_idx * p.rows + row] = lse;
        }
    }
}

// O = sum_r exp(LSE_r - LSE) O_r, LSE = logsumexp_r LSE_r; one CTA of 256 threads per output row.
// The weights exp(LSE_r - LSE) are computed once into shared memory; the accumulation then runs
// over the partials with 8 warps in parallel (part r goes to warp r % 8) and four independent
// loads in flight per lane, so a row with hundreds of partials (long-context split-KV) costs a few
// memory latencies instead of one per partial.  Each lane owns dims lane, lane+32, ...
// A partial with LSE_r = -inf gets weight 0 and its O is never read (it may be uninitialised).
constexpr int kToPeerFlag = 401;  // device status code: a peer's record did not arrive in time

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

constexpr int kMergeWarps = 8;
constexpr int kMergeMaxDimPerLane = 8;  // dim <= 256

// Merge of one output row over n_parts partials (the CTA's 8 warps in parallel, see above).  On return every
// thread holds the row's LSE; thread d < dim holds O[d] (normalised; zeros and LSE = -inf when every part is
// empty).  part r of the row lies at o_row + r * part_stride (dim floats), its LSE at lse_row[r * lse_part_stride].
// sm: kMergeWarps * dim + n_parts floats; red / s_ml: small CTA-shared scratch.  Ends with a __syncthreads-free
// state in which sm may be reused after the next barrier.
__device__ __forceinline__ float merge_row(const float* o_row, const float* lse_row, int n_parts, int64_t part_stride,
                                           int64_t lse_part_stride, int dim, float* sm, float* red, float* s_ml,
                                           float& lse_out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* acc_sm = sm;                    // [kMergeWarps][dim]
    float* w_sm = sm + kMergeWarps * dim;  // [n_parts]: LSE_r, then the weight of part r
    float m = -INFINITY;
    for (int r = tid; r < n_parts; r += kMergeWarps * 32) {
        const float x = lse_row[(int64_t)r * lse_part_stride];
        w_sm[r] = x;
        m = fmaxf(m, x);
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(kFullMask, m, off));
    __syncthreads();  // red / s_ml / sm of an earlier merge in this kernel are no longer read
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (tid == 0) {
        float x = red[0];
        for (int i = 1; i < kMergeWarps; ++i) x = fmaxf(x, red[i]);
        s_ml[0] = x;
    }
    __syncthreads();
    m = s_ml[0];
    if (m == -INFINITY) {  // every partial empty
        lse_out = -INFINITY;
        return 0.f;
    }
    float l = 0.f;
    for (int r = tid; r < n_parts; r += kMergeWarps * 32) {
        const float x = w_sm[r];
        const float w = (x == -INFINITY) ? 0.f : expf(x - m);
        w_sm[r] = w;
        l += w;
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) l += __shfl_xor_sync(kFullMask, l, off);
    __syncthreads();  // weights visible; red[] free again
    if (lane == 0) red[warp] = l;

    float acc[kMergeMaxDimPerLane];
#pragma unroll
    for (int i = 0; i < kMergeMaxDimPerLane; ++i) acc[i] = 0.f;
    for (int r0 = warp; r0 < n_parts; r0 += 4 * kMergeWarps) {
        float w[4];
        float v[4][kMergeMaxDimPerLane];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int r = r0 + u * kMergeWarps;
            w[u] = (r < n_parts) ? w_sm[r] : 0.f;
#pragma unroll
            for (int i = 0; i < kMergeMaxDimPerLane; ++i) {
                const int d = lane + 32 * i;
                v[u][i] = (w[u] != 0.f && d < dim) ? o_row[(int64_t)r * part_stride + d] : 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int i = 0; i < kMergeMaxDimPerLane; ++i) acc[i] = fmaf(w[u], v[u][i], acc[i]);
    }
#pragma unroll
    for (int i = 0; i < kMergeMaxDimPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < dim) acc_sm[warp * dim + d] = acc[i];
    }
    __syncthreads();
    if (tid == 0) {
        float x = 0.f;
        for (int i = 0; i < kMergeWarps; ++i) x += red[i];
        s_ml[1] = x;
    }
    __syncthreads();
    const float s_l = s_ml[1];
    lse_out = m + logf(s_l);
    float o = 0.f;
    if (tid < dim) {
#pragma unroll
        for (int x = 0; x < kMergeWarps; ++x) o += acc_sm[x * dim + tid];
        o *= 1.f / s_l;
    }
    return o;
}

// Bounded wait for arrival flags: thread t < n waits until flag_of(t) >= epoch.  Returns false (for the whole
// CTA) when a wait ran out; the code is then in the device status word.
__device__ __forceinline__ bool wait_for_flags(const uint32_t* flags, int n, int64_t flag_stride, uint32_t epoch,
                                               long long max_clocks, int* status) {
    __shared__ int wait_failed;
    const int tid = threadIdx.x;
    if (tid == 0) wait_failed = 0;
    __syncthreads();
    if (tid < n) {
        const long long t0 = clock64();
        while (ld_acquire_sys_u32(flags + tid * flag_stride) < epoch) {
            if (clock64() - t0 > max_clocks) {
                report_timeout(status, kToPeerFlag);
                wait_failed = 1;
                break;
            }
        }
    }
    __syncthreads();
    return !wait_failed;
}

__global__ void __launch_bounds__(kMergeWarps * 32) merge_partials_kernel(const float* __restrict__ o_parts,
                                                                         const float* __restrict__ lse_parts,
                                                                         int n_parts, int64_t rows, int dim,
                                                                         int64_t in_row_stride, int64_t in_lse_stride,
                                                                         __nv_bfloat16* out_bf16, float* out_f32,
                                                                         float* lse_out, int64_t of_stride,
                                                                         int64_t lse_stride, MergeWait wait,
                                                                         MergePush push) {
    const int64_t row = blockIdx.x;
    const int tid = threadIdx.x;
    // Delivery of this row to the peers (record layout: out_f32 rows of of_stride floats, LSE at column dim).
    auto push_row_value = [&](int d, float x) {
        for (int r = 0; r < push.world; ++r)
            if (push.dst[r] != out_f32) push.dst[r][row * of_stride + d] = x;
    };
    if (!wait.flags) {
        // A merge of partials that the kernel before it in the stream wrote: under programmatic stream
        // serialisation its CTAs may be resident early, and this returns once that kernel has completed and
        // its writes are visible (at once under a normal launch).
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    // what follows in the stream (the next step's decode) may be scheduled; it waits before it reads anything
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (wait.flags) {
        // Part r of this merge is written into local memory by rank r (on that GPU), which then raises
        // flags[r] (or, with per-row flags, flags[r * rows + row]) to the epoch with a system-scope release.
        // The wait is bounded: on expiry the kernel records the code and returns without touching the outputs.
        const uint32_t* f = wait.flags + (wait.per_row ? row : 0);
        if (!wait_for_flags(f, wait.n_flags, wait.per_row ? rows : 1, wait.epoch, wait.max_clocks, wait.status)) return;
    }
    __shared__ float red[kMergeWarps];
    __shared__ float s_ml[2];
    extern __shared__ float merge_sm[];
    float lse;
    const float o = merge_row(o_parts + row * in_row_stride, lse_parts + row * in_lse_stride, n_parts,
                              rows * in_row_stride, rows * in_lse_stride, dim, merge_sm, red, s_ml, lse);
    if (tid < dim) {
        if (out_bf16) out_bf16[row * dim + tid] = __float2bfloat16(o);
        if (out_f32) out_f32[row * of_stride + tid] = o;
        if (push.world) push_row_value(tid, o);
    }
    if (tid == 0 && lse_out) lse_out[row * lse_stride] = lse;
    if (push.world) {
        if (tid == 0) push_row_value(dim, lse);
        __threadfence_system();  // every thread of the CTA, once its stores are issued
        __syncthreads();
        if (tid == 0 && atomicAdd(push.done_counter, 1) == (int)rows - 1) {
            *push.done_counter = 0;  // ready for the next launch
            __threadfence_system();  // all rows of all CTAs are ordered before the flags
            for (int r = 0; r < push.world; ++r)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(push.flag[r]), "r"(push.epoch) : "memory");
        }
    }
}

// The tail of a split-KV decode in ONE kernel, one CTA per output row: merge the rank's chunk partials of the
// row, store the row (O | LSE) into the slot every rank keeps for this rank (plain stores, NVLink for the peers;
// nothing is ever loaded from a peer) and raise that rank's flag for (this rank, row); then wait, bounded, for
// the row from every rank and merge the `world` rows out of local memory.  Rows are independent, so nothing
// waits for a whole record, no counter is shared between CTAs, and the chunk merge, the delivery and the
// cross-rank merge need no kernel boundary between them.
// With do_wait = 0 the kernel stops after the delivery; merge_partials_kernel with per-row flags then does
// the second half (used where several ranks are emulated on one GPU: a kernel must not wait for a flag that a
// later launch on the same GPU raises).
struct RowExchange {
    float* slot[kMaxPeers];          // on rank p: the [rows, dim + 1] slot p keeps for this rank (p = this rank: local)
    uint32_t* flag[kMaxPeers];       // on rank p: the [rows] flags p keeps for this rank
    const float* local_slots;        // this rank's slots for all ranks: [world][rows][dim + 1]
    const uint32_t* local_flags;     // [world][rows]
    int world;
    uint32_t epoch;
    long long max_clocks;
    int* status;
    int do_wait;
};

__global__ void __launch_bounds__(kMergeWarps * 32) splitkv_row_exchange_kernel(
    const float* __restrict__ o_parts, const float* __restrict__ lse_parts, int n_parts, int64_t rows, int dim,
    int64_t in_row_stride, int64_t in_lse_stride, __nv_bfloat16* out_bf16, float* out_f32, float* lse_out,
    RowExchange x) {
    const int64_t row = blockIdx.x;
    const int tid = threadIdx.x;
    __shared__ float red[kMergeWarps];
    __shared__ float s_ml[2];
    extern __shared__ float merge_sm[];
    // Launched with programmatic stream serialisation: the CTAs may already be resident when the decode kernel
    // before this one finishes (it lets its dependents go once every CTA has streamed its chunk); this wait
    // returns when that kernel has completed and its partials are visible (at once under a normal launch).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float lse;
    const float o = merge_row(o_parts + row * in_row_stride, lse_parts + row * in_lse_stride, n_parts,
                              rows * in_row_stride, rows * in_lse_stride, dim, merge_sm, red, s_ml, lse);
    const int64_t rec = row * (dim + 1);
    for (int r = 0; r < x.world; ++r) {
        if (tid < dim) x.slot[r][rec + tid] = o;
        if (tid == 0) x.slot[r][rec + dim] = lse;
    }
    __threadfence_system();
    __syncthreads();
    if (tid < x.world)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(x.flag[tid] + row), "r"(x.epoch) : "memory");
    if (!x.do_wait) return;
    if (!wait_for_flags(x.local_flags + row, x.world, rows, x.epoch, x.max_clocks, x.status)) return;
    const float o2 = merge_row(x.local_slots + rec, x.local_slots + rec + dim, x.world, rows * (dim + 1),
                               rows * (dim + 1), dim, merge_sm, red, s_ml, lse);
    if (tid < dim) {
        if (out_bf16) out_bf16[row * dim + tid] = __float2bfloat16(o2);
        if (out_f32) out_f32[row * dim + tid] = o2;
    }
    if (tid == 0 && lse_out) lse_out[row] = lse;
}

// ---------------------------------------------------------------------------------------------
// The same row exchange with the flag inside the data ("low-latency" words, as NCCL's LL protocol): every
// element of a row travels as one 8-byte word {value bits, epoch}.  An aligned 8-byte store is a single
// access, so a reader that sees the epoch in a word also sees the value that came with it: no system-scope
// fence between data and flag, no flag store, and the reader needs no acquire - one NVLink round trip less
// on the critical path of every step.  Slots are [rows][dim + 1] words; the two slot sets still alternate
// with the epoch, and a stale word (epoch - 2 or older) simply does not match.
struct LlExchange {
    unsigned long long* words[kMaxPeers];   // on rank p: the [rows][dim + 1] words p keeps for this rank
    const unsigned long long* local_words;  // this rank's words for all ranks: [world][rows][dim + 1]
    int world;
    uint32_t epoch;
    long long max_clocks;
    int* status;
    int do_wait;
};

__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Waits (bounded) until element tid of row `row` has arrived from every rank, then merges the rows by their
// LSEs: o is the merged element tid (tid < dim), lse the merged LSE.  All threads of the CTA call it.
__device__ __forceinline__ bool ll_wait_merge(const unsigned long long* local_words, int world, int64_t rows, int dim,
                                              int64_t row, uint32_t epoch, long long max_clocks, int* status, float& o,
                                              float& lse) {
    __shared__ float s_lse[kMaxPeers];
    __shared__ int s_fail;
    const int tid = threadIdx.x;
    if (tid == 0) s_fail = 0;
    __syncthreads();
    float v[kMaxPeers];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) v[r] = 0.f;
    if (tid <= dim) {
        const long long t0 = clock64();
        bool alive = true;
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r) {
            if (r >= world || !alive) continue;
            const unsigned long long* p = local_words + ((int64_t)r * rows + row) * (dim + 1) + tid;
            unsigned long long w = ld_relaxed_sys_u64(p);
            while ((uint32_t)(w >> 32) != epoch) {
                if (clock64() - t0 > max_clocks) {
                    report_timeout(status, kToPeerFlag);
                    s_fail = 1;
                    alive = false;
                    break;
                }
                w = ld_relaxed_sys_u64(p);
            }
            v[r] = __uint_as_float((uint32_t)w);
            if (tid == dim) s_lse[r] = v[r];
        }
    }
    __syncthreads();
    if (s_fail) return false;
    float m = -INFINITY;
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
        if (r < world) m = fmaxf(m, s_lse[r]);
    float l = 0.f, acc = 0.f;
    if (m > -INFINITY) {
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r) {
            if (r >= world) continue;
            const float w = (s_lse[r] == -INFINITY) ? 0.f : expf(s_lse[r] - m);
            l += w;
            acc = fmaf(w, v[r], acc);
        }
    }
    o = (l > 0.f) ? acc / l : 0.f;
    lse = (l > 0.f) ? m + logf(l) : -INFINITY;
    return true;
}

__global__ void __launch_bounds__(kMergeWarps * 32) splitkv_row_exchange_ll_kernel(
    const float* __restrict__ o_parts, const float* __restrict__ lse_parts, int n_parts, int64_t rows, int dim,
    int64_t in_row_stride, int64_t in_lse_stride, __nv_bfloat16* out_bf16, float* out_f32, float* lse_out,
    LlExchange x) {
    const int64_t row = blockIdx.x;
    const int tid = threadIdx.x;
    __shared__ float red[kMergeWarps];
    __shared__ float s_ml[2];
    extern __shared__ float merge_sm[];
    asm volatile("griddepcontrol.wait;" ::: "memory");  // see splitkv_row_exchange_kernel
    float lse;
    const float o = merge_row(o_parts + row * in_row_stride, lse_parts + row * in_lse_stride, n_parts,
                              rows * in_row_stride, rows * in_lse_stride, dim, merge_sm, red, s_ml, lse);
    const int64_t rec = row * (dim + 1);
    const unsigned long long tag = (unsigned long long)x.epoch << 32;
    for (int r = 0; r < x.world; ++r) {
        if (tid < dim) st_relaxed_sys_u64(x.words[r] + rec + tid, tag | __float_as_uint(o));
        if (tid == 0) st_relaxed_sys_u64(x.words[r] + rec + dim, tag | __float_as_uint(lse));
    }
    if (!x.do_wait) return;
    float o2, lse2;
    if (!ll_wait_merge(x.local_words, x.world, rows, dim, row, x.epoch, x.max_clocks, x.status, o2, lse2)) return;
    if (tid < dim) {
        if (out_bf16) out_bf16[row * dim + tid] = __float2bfloat16(o2);
        if (out_f32) out_f32[row * dim + tid] = o2;
    }
    if (tid == 0 && lse_out) lse_out[row] = lse2;
}

// Second half alone (after a delivery with do_wait = 0: several ranks emulated on one GPU).
__global__ void __launch_bounds__(kMergeWarps * 32) splitkv_ll_merge_kernel(
    const unsigned long long* __restrict__ local_words, int world, int64_t rows, int dim, uint32_t epoch,
    long long max_clocks, int* status, __nv_bfloat16* out_bf16, float* out_f32, float* lse_out) {
    const int64_t row = blockIdx.x;
    const int tid = threadIdx.x;
    float o, lse;
    if (!ll_wait_merge(local_words, world, rows, dim, row, epoch, max_clocks, status, o, lse)) return;
    if (tid < dim) {
        if (out_bf16) out_bf16[row * dim + tid] = __float2bfloat16(o);
        if (out_f32) out_f32[row * dim + tid] = o;
    }
    if (tid == 0 && lse_out) lse_out[row] = lse;
}

static size_t merge_smem_bytes(int64_t n_parts, int dim) {
    return sizeof(float) * ((size_t)kMergeWarps * dim + (size_t)n_parts);
}

bool merge_fits(int64_t n_parts, int dim) {
    return dim <= 32 * kMergeMaxDimPerLane && merge_smem_bytes(n_parts, dim) <= 48 * 1024;
}

// Writes one token's K and V rows into the caches (llm_kernels.rs:345-373, batched).
__global__ void kv_append_kernel(__nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
                                 const __nv_bfloat16* k_in, const __nv_bfloat16* v_in, int n_kv,
                                 int head_dim, int64_t max_seq, int64_t pos, const int32_t* positions) {
    // the decode that follows may be scheduled at once; it waits for this kernel's completion before it reads
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int kvh = blockIdx.x, b = blockIdx.y;
    const int64_t at = positions ? (int64_t)positions[b] : pos;
    if (at < 0 || at >= max_seq) return;
    const int64_t src = ((int64_t)b * n_kv + kvh) * head_dim;
    const int64_t dst = (((int64_t)b * n_kv + kvh) * max_seq + at) * head_dim;
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
        k_cache[dst + i] = k_in[src + i];
        v_cache[dst + i] = v_in[src + i];
    }
}

// One decode step's preparation in a single launch: rotary embedding of q (in place) and of the new K
// row, then the K and V rows go into the caches at each sequence's position.  The reference issues
// three kernels per layer and token for this (rope on Q, rope on K, kv_append:
// crates/rustorch-llm/src/cuda_backend.rs:917-966).  angle = pos * inv_freq[k] in f32, accurate sincosf.
//   style 0: pairs (k, k + D/2) (crates/rustorch-nn/src/rope.rs:162-205, the CPU model's convention)
//   style 1: pairs (2k, 2k+1)   (crates/rustorch-cuda/src/llm_kernels.rs:109-143)
// Grid (Hq + Hkv, B), D/2 threads: CTA y handles one head row; rows >= Hq are the KV heads.
__global__ void rope_kv_append_kernel(__nv_bfloat16* q, const __nv_bfloat16* k_in, const __nv_bfloat16* v_in,
                                      __nv_bfloat16* k_cache, __nv_bfloat16* v_cache, const float* inv_freq,
                                      const int32_t* positions, int64_t pos_uniform, int n_heads, int n_kv,
                                      int head_dim, int64_t max_seq, int style) {
    // the decode that follows may be scheduled at once; it waits for this kernel's completion before it reads
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int b = blockIdx.y, hrow = blockIdx.x, half = head_dim / 2;
    const int64_t pos = positions ? (int64_t)positions[b] : pos_uniform;
    if (pos < 0 || pos >= max_seq) return;
    const bool is_q = hrow < n_heads;
    const int h = is_q ? hrow : hrow - n_heads;
    const __nv_bfloat16* src = is_q ? q + ((int64_t)b * n_heads + h) * head_dim
                                    : k_in + ((int64_t)b * n_kv + h) * head_dim;
    __nv_bfloat16* dst = is_q ? q + ((int64_t)b * n_heads + h) * head_dim
                              : k_cache + (((int64_t)b * n_kv + h) * max_seq + pos) * head_dim;
    for (int k = threadIdx.x; k < half; k += blockDim.x) {
        const int i0 = style == 0 ? k : 2 * k, i1 = style == 0 ? k + half : 2 * k + 1;
        float s, c;
        sincosf((float)pos * inv_freq[k], &s, &c);
        const float x0 = __bfloat162float(src[i0]), x1 = __bfloat162float(src[i1]);
        dst[i0] = __float2bfloat16_rn(x0 * c - x1 * s);
        dst[i1] = __float2bfloat16_rn(x1 * c + x0 * s);
    }
    if (!is_q) {
        const __nv_bfloat16* vs = v_in + ((int64_t)b * n_kv + h) * head_dim;
        __nv_bfloat16* vd = v_cache + (((int64_t)b * n_kv + h) * max_seq + pos) * head_dim;
        for (int i = threadIdx.x; i < head_dim; i += blockDim.x) vd[i] = vs[i];
    }
}

cudaError_t launch_rope_kv_append(void* q, const void* k_in, const void* v_in, void* k_cache, void* v_cache,
                                  const float* inv_freq, const int32_t* positions, int64_t pos_uniform,
                                  int64_t batch, int n_heads, int n_kv, int head_dim, int64_t max_seq, int style,
                                  cudaStream_t stream) {
    if (batch == 0 || n_heads + n_kv == 0) return cudaSuccess;
    dim3 grid(n_heads + n_kv, (unsigned)batch);
    int threads = head_dim / 2;
    threads = threads < 32 ? 32 : (threads > 128 ? 128 : threads);
    rope_kv_append_kernel<<<grid, threads, 0, stream>>>((__nv_bfloat16*)q, (const __nv_bfloat16*)k_in,
                                                        (const __nv_bfloat16*)v_in, (__nv_bfloat16*)k_cache,
                                                        (__nv_bfloat16*)v_cache, inv_freq, positions, pos_uniform,
                                                        n_heads, n_kv, head_dim, max_seq, style);
    return cudaGetLastError();
}

// Tokens per KV chunk (one CTA per chunk).  Large chunks amortise the per-CTA prologue and the
// partial traffic (1024 tokens measured best on the ragged batched workload); the choice walks
// down from 1024 until the grid both covers the SMs x 2 resident CTAs and fills its last wave
// to at least 95 % (a long single sequence otherwise loses up to a quarter of a wave).  It depends
// only on (batch, n_kv, max_seq) so that rt_gqa_decode_workspace_bytes can size the scratch.
// RT_ATTN_DECODE_CHUNK=<multiple of 64> overrides it.
int decode_chunk_tokens(int64_t batch, int n_kv, int64_t max_seq) {
    static int forced = [] {
        const char* e = getenv("RT_ATTN_DECODE_CHUNK");
        int c = e ? atoi(e) : 0;
        return (c >= 64 && c % 64 == 0) ? c : 0;
    }();
    if (forced) return forced;
    const int64_t base = (batch > 0 ? batch : 1) * (int64_t)(n_kv > 0 ? n_kv : 1);
    const int64_t slots = (int64_t)sm_count() * 2;
    int best = 128;
    double best_eff = -1.0;
    for (int c = 1024; c >= 128; c -= 64) {
        const int64_t ctas = base * ((max_seq + c - 1) / c);
        if (ctas < slots && c > 128) continue;
        const double waves = (double)ctas / (double)slots;
        const double eff = waves / (double)((ctas + slots - 1) / slots);
        if (eff >= 0.95) return c;
        if (eff > best_eff) {
            best_eff = eff;
            best = c;
        }
    }
    return best;
}

// RT_ATTN_DECODE_IMPL=simt selects the CUDA-core kernel for every shape (A/B comparisons).
static bool decode_use_tensor_cores() {
    static bool use = [] {
        const char* e = getenv("RT_ATTN_DECODE_IMPL");
        return !(e && e[0] == 's');
    }();
    return use;
}

int decode_num_chunks(int64_t batch, int n_kv, int64_t max_seq) {
    const int chunk = decode_chunk_tokens(batch, n_kv, max_seq);
    int64_t n = (max_seq + chunk - 1) / chunk;
    return (int)(n < 1 ? 1 : n);
}

template <int D, int G>
static cudaError_t launch_decode_dg(const DecodeParams& p, int64_t batch, cudaStream_t stream) {
    dim3 grid(p.n_chunks, p.n_kv, (unsigned)batch);
    gqa_decode_splitkv_kernel<D, G><<<grid, 128, 0, stream>>>(p);
    return cudaGetLastError();
}

template <int D>
static cudaError_t launch_decode_d(const DecodeParams& p, int group, int64_t batch, cudaStream_t stream) {
    switch (group) {
        case 1: return launch_decode_dg<D, 1>(p, batch, stream);
        case 2: return launch_decode_dg<D, 2>(p, batch, stream);
        case 4: return launch_decode_dg<D, 4>(p, batch, stream);
        case 8: return launch_decode_dg<D, 8>(p, batch, stream);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_gqa_decode(const void* q, const void* k, const void* v, void* out_bf16, float* out_f32,
                              float* lse, int64_t batch, int n_heads, int n_kv, int head_dim,
                              int64_t max_seq, const int32_t* kv_lens, int64_t kv_len_uniform,
                              int64_t kv_begin, int64_t kv_end, float scale, void* workspace,
                              int64_t of_stride, int64_t lse_stride, cudaStream_t stream, const MergePush* push,
                              bool* pushed, DecodeTail* tail) {
    if (pushed) *pushed = false;
    DecodeParams p;
    p.q = (const __nv_bfloat16*)q;
    p.k = (const __nv_bfloat16*)k;
    p.v = (const __nv_bfloat16*)v;
    p.out_bf16 = (__nv_bfloat16*)out_bf16;
    p.out_f32 = out_f32;
    p.lse = lse;
    p.kv_lens = kv_lens;
    p.kv_len_uniform = kv_len_uniform;
    p.kv_begin = kv_begin;
    p.kv_end = kv_end;
    p.max_seq = max_seq;
    p.n_heads = n_heads;
    p.n_kv = n_kv;
    p.chunk = decode_chunk_tokens(batch, n_kv, max_seq);
    // The visible range can be no longer than this; chunks past it would all be empty.
    int64_t span = max_seq - kv_begin;
    if (!kv_lens && kv_len_uniform - kv_begin < span) span = kv_len_uniform - kv_begin;
    if (kv_end >= 0 && kv_end - kv_begin < span) span = kv_end - kv_begin;
    if (span < 1) span = 1;
    // A few long sequences (fewer (sequence, KV head) groups than resident CTAs): one wave of longer chunks
    // streams as fast as several waves of short ones and leaves a fraction of the partials to merge
    // (one sequence of 131072 positions: 37 chunks instead of 147).  The chunk only ever grows here, so the
    // chunk count stays within what rt_gqa_decode_workspace_bytes sized the scratch for.
    {
        const int64_t groups = batch * (int64_t)n_kv, slots = (int64_t)sm_count() * 2;
        if (groups < slots) {
            const int64_t per_group = slots / groups;
            const int64_t want = ((span + per_group - 1) / per_group + 63) / 64 * 64;
            if (want > p.chunk && want <= (1 << 20)) p.chunk = (int)want;
        }
    }
    p.n_chunks = (int)((span + p.chunk - 1) / p.chunk);
    p.rows = batch * n_heads;
    p.of_stride = of_stride > 0 ? of_stride : head_dim;
    p.lse_stride = lse_stride > 0 ? lse_stride : 1;
    p.scale_log2 = scale * kLog2e;
    p.part_o = (float*)workspace;
    p.part_lse = p.part_o ? p.part_o + (int64_t)decode_num_chunks(batch, n_kv, max_seq) * p.rows * head_dim : nullptr;
    const int group = n_heads / n_kv;
    // after the partials: one completion counter per (sequence, KV head) for the in-kernel merge
    int* counters = p.part_lse ? reinterpret_cast<int*>(p.part_lse + (int64_t)decode_num_chunks(batch, n_kv, max_seq) * p.rows)
                               : nullptr;
    bool merged = false;
    if (tail) {  // the caller merges the chunk partials itself (split-KV row exchange)
        counters = nullptr;
        tail->n_chunks = p.n_chunks;
        tail->part_o = p.part_o;
        tail->part_lse = p.part_lse;
    }
    cudaError_t e = cudaErrorNotSupported;
    if (decode_use_tensor_cores())
        e = launch_gqa_decode_tc(q, k, v, out_bf16, out_f32, lse, batch, n_heads, n_kv, head_dim, max_seq, kv_lens,
                                 kv_len_uniform, kv_begin, kv_end, scale, p.part_o, p.part_lse, counters, p.chunk,
                                 p.n_chunks, p.of_stride, p.lse_stride, &merged, push, stream);
    if (e == cudaErrorNotSupported) {  // a cache too large for 32-bit TMA row coordinates, or RT_ATTN_DECODE_IMPL=simt
        switch (head_dim) {
            case 64: e = launch_decode_d<64>(p, group, batch, stream); break;
            case 128: e = launch_decode_d<128>(p, group, batch, stream); break;
            case 256: e = launch_decode_d<256>(p, group, batch, stream); break;
            default: return cudaErrorInvalidValue;
        }
    }
    if (e != cudaSuccess) return e;
    if (merged && push && push->world > 0 && pushed) *pushed = true;  // delivered by the decode kernel itself
    if (p.n_chunks > 1 && !merged && !tail) {
        e = launch_merge_partials(p.part_o, p.part_lse, p.n_chunks, p.rows, head_dim, head_dim, 1, p.out_bf16, p.out_f32, lse,
                                  stream, nullptr, push, p.of_stride, p.lse_stride);
        if (e != cudaSuccess) return e;
        if (push && pushed) *pushed = true;
    }
    return e;
}

cudaError_t launch_merge_partials(const float* o_parts, const float* lse_parts, int64_t n_parts, int64_t rows,
                                  int dim, int64_t in_row_stride, int64_t in_lse_stride, void* out_bf16,
                                  float* out_f32, float* lse, cudaStream_t stream, const MergeWait* wait,
                                  const MergePush* push, int64_t of_stride, int64_t lse_stride) {
    if (rows == 0) return cudaSuccess;
    if (of_stride <= 0) of_stride = dim;
    if (lse_stride <= 0) lse_stride = 1;
    if (!merge_fits(n_parts, dim)) return cudaErrorInvalidValue;
    if (wait && wait->n_flags > kMergeWarps * 32) return cudaErrorInvalidValue;
    const MergeWait w = wait ? *wait : MergeWait{nullptr, 0, 0u, 0, nullptr, 0};
    const MergePush ps = push ? *push : MergePush{};
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(kMergeWarps * 32);
    cfg.dynamicSmemBytes = merge_smem_bytes(n_parts, dim);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    // RT_ATTN_MERGE_PDL=0 launches the plain merge without programmatic stream serialisation (measured with
    // it: the 131 072-position shard 91.1 -> 89.3 us, batch-1 decode at 8192 positions 12.4 -> 10.7 us).
    static const bool merge_pdl = [] {
        const char* e = getenv("RT_ATTN_MERGE_PDL");
        return !(e && e[0] == '0');
    }();
    if (wait || merge_pdl) {
        // A merge that waits on arrival flags reads nothing the kernel before it in the stream wrote except
        // through those flags (acquire loads), so it may be scheduled as soon as that kernel lets its
        // dependents go (the decode kernel does once every CTA has streamed its chunk).  Its wait is bounded,
        // and the CTAs it waits for are resident by then.
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, merge_partials_kernel, o_parts, lse_parts, (int)n_parts, rows, dim, in_row_stride,
                              in_lse_stride, (__nv_bfloat16*)out_bf16, out_f32, lse, of_stride, lse_stride, w, ps);
}

cudaError_t launch_row_exchange(const float* o_parts, const float* lse_parts, int64_t n_parts, int64_t rows, int dim,
                                int64_t in_row_stride, int64_t in_lse_stride, void* out_bf16, float* out_f32, float* lse,
                                void* const* peer_slots, void* const* peer_flags, const float* local_slots,
                                const uint32_t* local_flags, int world, uint32_t epoch, long long wait_clocks,
                                int do_wait, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    const int64_t most = n_parts > world ? n_parts : world;
    if (world <= 0 || world > kMaxPeers || !merge_fits(most, dim)) return cudaErrorInvalidValue;
    RowExchange x;
    for (int r = 0; r < kMaxPeers; ++r) {
        x.slot[r] = r < world ? static_cast<float*>(peer_slots[r]) : nullptr;
        x.flag[r] = r < world ? static_cast<uint32_t*>(peer_flags[r]) : nullptr;
    }
    x.local_slots = local_slots;
    x.local_flags = local_flags;
    x.world = world;
    x.epoch = epoch;
    x.max_clocks = wait_clocks > 0 ? wait_clocks : (1ll << 31);
    x.status = device_status_ptr();
    x.do_wait = do_wait;
    if (!x.status) return cudaErrorInvalidSymbol;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(kMergeWarps * 32);
    cfg.dynamicSmemBytes = merge_smem_bytes(most, dim);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    static const bool pdl = [] {
        const char* e = getenv("RT_ATTN_EXCHANGE_PDL");
        return !(e && e[0] == '0');
    }();
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, splitkv_row_exchange_kernel, o_parts, lse_parts, (int)n_parts, rows, dim, in_row_stride,
                              in_lse_stride, (__nv_bfloat16*)out_bf16, out_f32, lse, x);
}

cudaError_t launch_row_exchange_ll(const float* o_parts, const float* lse_parts, int64_t n_parts, int64_t rows, int dim,
                                   int64_t in_row_stride, int64_t in_lse_stride, void* out_bf16, float* out_f32,
                                   float* lse, void* const* peer_words, const void* local_words, int world,
                                   uint32_t epoch, long long wait_clocks, int do_wait, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    if (world <= 0 || world > kMaxPeers || dim + 1 > kMergeWarps * 32 || !merge_fits(n_parts, dim))
        return cudaErrorInvalidValue;
    LlExchange x;
    for (int r = 0; r < kMaxPeers; ++r) x.words[r] = r < world ? static_cast<unsigned long long*>(peer_words[r]) : nullptr;
    x.local_words = static_cast<const unsigned long long*>(local_words);
    x.world = world;
    x.epoch = epoch;
    x.max_clocks = wait_clocks > 0 ? wait_clocks : (1ll << 31);
    x.status = device_status_ptr();
    x.do_wait = do_wait;
    if (!x.status) return cudaErrorInvalidSymbol;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(kMergeWarps * 32);
    cfg.dynamicSmemBytes = merge_smem_bytes(n_parts, dim);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // as launch_row_exchange
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, splitkv_row_exchange_ll_kernel, o_parts, lse_parts, (int)n_parts, rows, dim,
                              in_row_stride, in_lse_stride, (__nv_bfloat16*)out_bf16, out_f32, lse, x);
}

cudaError_t launch_ll_merge(const void* local_words, int world, int64_t rows, int dim, uint32_t epoch,
                            long long wait_clocks, void* out_bf16, float* out_f32, float* lse, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    if (world <= 0 || world > kMaxPeers || dim + 1 > kMergeWarps * 32) return cudaErrorInvalidValue;
    int* status = device_status_ptr();
    if (!status) return cudaErrorInvalidSymbol;
    splitkv_ll_merge_kernel<<<(unsigned)rows, kMergeWarps * 32, 0, stream>>>(
        static_cast<const unsigned long long*>(local_words), world, rows, dim, epoch,
        wait_clocks > 0 ? wait_clocks : (1ll << 31), status, (__nv_bfloat16*)out_bf16, out_f32, lse);
    return cudaGetLastError();
}

// Copies this rank's packed (O | LSE) record into the slot every peer keeps for it and raises the
// peer's flag.  One CTA per destination; plain peer stores over NVLink (no multicast, no multimem),
// a system-scope fence, then one release store of the epoch.  The kernel never waits.
struct PushParams {
    const float* src;
    float* dst[kMaxPeers];
    uint32_t* flag[kMaxPeers];
    int64_t n_vec4;
    uint32_t epoch;
};

__global__ void __launch_bounds__(256) push_records_kernel(const PushParams p) {
    const int peer = blockIdx.x;
    float4* dst = reinterpret_cast<float4*>(p.dst[peer]);
    const float4* src = reinterpret_cast<const float4*>(p.src);
    if (reinterpret_cast<const float4*>(dst) != src)
        for (int64_t i = threadIdx.x; i < p.n_vec4; i += blockDim.x) dst[i] = src[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flag[peer]), "r"(p.epoch) : "memory");
}

cudaError_t launch_push_records(const float* record, void* const* peer_slots, void* const* peer_flags, int world,
                                int64_t record_floats, uint32_t epoch, cudaStream_t stream) {
    if (world <= 0 || world > kMaxPeers || (record_floats & 3)) return cudaErrorInvalidValue;
    PushParams p;
    p.src = record;
    for (int r = 0; r < kMaxPeers; ++r) {
        p.dst[r] = r < world ? static_cast<float*>(peer_slots[r]) : nullptr;
        p.flag[r] = r < world ? static_cast<uint32_t*>(peer_flags[r]) : nullptr;
    }
    p.n_vec4 = record_floats / 4;
    p.epoch = epoch;
    push_records_kernel<<<world, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_kv_append(void* k_cache, void* v_cache, const void* k_in, const void* v_in, int64_t batch,
                             int n_kv, int head_dim, int64_t max_seq, int64_t pos, const int32_t* positions,
                             cudaStream_t stream) {
    if (batch == 0 || n_kv == 0) return cudaSuccess;
    dim3 grid(n_kv, (unsigned)batch);
    kv_append_kernel<<<grid, 64, 0, stream>>>((__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
                                              (const __nv_bfloat16*)k_in, (const __nv_bfloat16*)v_in, n_kv,
                                              head_dim, max_seq, pos, positions);
    return cudaGetLastError();
}

}  // namespace rt
