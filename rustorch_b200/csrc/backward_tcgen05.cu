// bf16 flash-attention backward on the Blackwell tensor cores (tcgen05 + TMEM + TMA).
//
// Same math as rustorch_attention::flash_backward (crates/rustorch-attention/src/cpu_backward.rs:16-27,
// 96-189) with the saved row statistics in place of the N x N probability matrix:
//   P = exp(scale * Q K^T - LSE),  dP = dO V^T,  dS = P o (dP - delta),  delta_i = dO_i . O_i,
//   dV = P^T dO,  dQ = scale * dS K,  dK = scale * dS^T Q.
// Two deterministic passes (no atomics, fixed summation order) share one kernel template.  A CTA owns
// 128 rows of one side, keeps them in shared memory, and walks the other side in 64-row steps that TMA
// streams through a four-slot ring:
//   query side: own X1 = Q_i, X2 = dO_i;  per key tile (Y1 = K_j, Y2 = V_j)
//               T1 = Q K^T, T2 = dO V^T (SS MMAs into TMEM) -> dS (bf16, back into TMEM) -> dQ += dS K_j (TS MMA)
//   key side:   own X1 = K_j, X2 = V_j;   per query tile (Y1 = Q_i, Y2 = dO_i)
//               T1 = K Q^T = S^T, T2 = V dO^T = dP^T -> P^T, dS^T (bf16, into TMEM)
//               -> dV += P^T dO_i, dK += dS^T Q_i (TS MMAs)
// Every product is "own rows x other tile": the score-like ones take both operands K-major from
// 128-byte-swizzled shared memory, the accumulating ones take A from TMEM and the other tile MN-major,
// exactly as TMA lands it (the forward's P V product has the same shape).  The thread that owns TMEM lane
// r owns own-row r: on the query side the statistics (LSE_i, delta_i) are per thread, on the key side
// they belong to the columns and are staged in shared memory per tile.  P and dS are rounded to bf16 for
// the accumulating products, as the forward rounds P.  A causal launch skips the tiles beyond the diagonal.
// An other-side tile is consumed in two 64-row steps, and the score-like results are double-buffered in
// TMEM, so the element-wise work of step u+1 runs while the accumulating MMAs of step u and the score
// MMAs of step u+2 occupy the tensor pipe (the forward kernel pipelines S and P the same way).
// TMEM (512 columns): buffer b of step u (b = u & 1) holds T1 at [128 b, 128 b + 64) and T2 at
// [128 b + 64, 128 b + 128); accumulators from 256 (dQ, or dV then dK), D columns each; P^T / dS (bf16)
// overwrite 32 of the columns of T1 / T2.  320 threads: warps 0-7 element-wise work and the final read-out,
// two threads per own row (warp w owns rows 32 (w % 4).. and the 32 score columns of half w / 4; its bf16
// results go back into the first 16 of its OWN columns, so the two threads of a row never touch each other's
// inputs, and the accumulating MMAs take K elements 0-31 from columns [0,16) and 32-63 from [32,48));
// warp 8 TMA producer, warp 9 TMEM allocation and MMA issue.
// Every mbarrier wait is bounded; on expiry the kernel records a code in the device status word and
// leaves through the common teardown.
#include <cuda.h>
#include <cstdlib>

#include "kernels.h"
#include "tc_ptx.cuh"

namespace rt {

using namespace ptx;

bool make_tensor_map_bf16_4d(CUtensorMap* map, const void* base, int64_t batch, int64_t heads, int64_t seq, int dim,
                             int64_t stride_b, int64_t stride_h, int64_t stride_row, int box_rows);  // prefill_tc.cu

namespace {

enum { kToBwdX = 201, kToBwdYFull, kToBwdYEmpty, kToBwdT, kToBwdA, kToBwdAcc, kToBwdDrain, kToBwdStat };

template <int D>
struct BwdCfg {
    static constexpr int TILE_BYTES = 128 * D * 2;
    static constexpr int SUB_BYTES = 128 * 64 * 2;  // one 64-column (128-byte) swizzled sub-tile
    static constexpr int NSUB = D / 64;
    static constexpr int HALF_BYTES = 64 * D * 2;   // 64 other-side rows: NSUB sub-tiles of 64 rows x 128 bytes
    static constexpr int HSUB_BYTES = 64 * 64 * 2;
    static constexpr int STAGES = 4;                // ring slots, each (Y1 | Y2) of one 64-row step
    static constexpr int NBARS = 1 + 2 * STAGES + 6;
    static constexpr int STAT_BYTES = 2 * 2 * 128 * 4;  // two slots of LSE * log2(e) and delta of a 128-row other tile
    static constexpr int SMEM_BYTES = 2 * TILE_BYTES + STAGES * 2 * HALF_BYTES + STAT_BYTES + NBARS * 8 + 16 + 1024;
    static constexpr uint32_t COL_T = 0, COL_ACC = 256;  // T1 of buffer b at COL_T + 128 b, T2 64 columns further
};

struct Bwd5Params {
    const float* lse;    // [B*H, N]
    const float* delta;  // [B*H, N]
    float* out1;         // query side: dQ; key side: dV   ([B*H, N, D] f32)
    float* out2;         // key side: dK
    int seq, heads;
    int causal;
    float scale, scale_log2;
    int* status;
    int head_group;      // heads per group of the CTA order
};

template <int D, bool kKeySide>
__global__ void __launch_bounds__(320, 1)
bwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_x1, const __grid_constant__ CUtensorMap tm_x2,
                   const __grid_constant__ CUtensorMap tm_y1, const __grid_constant__ CUtensorMap tm_y2,
                   const Bwd5Params p) {
    using C = BwdCfg<D>;
    constexpr int TILE = C::TILE_BYTES, SUB = C::SUB_BYTES, STAGES = C::STAGES, HALFT = C::HALF_BYTES, HSUB = C::HSUB_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sX1 = smem;
    uint8_t* sX2 = sX1 + TILE;
    uint8_t* sY = sX2 + TILE;  // [STAGES][Y1 | Y2], 64 rows each
    float* stat = reinterpret_cast<float*>(sY + STAGES * 2 * HALFT);  // [2][lse2[128] | delta[128]]
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(stat) + C::STAT_BYTES);
    uint64_t* x_full = bars;                // [1]
    uint64_t* y_full = x_full + 1;          // [STAGES]
    uint64_t* y_empty = y_full + STAGES;    // [STAGES]
    uint64_t* t_full = y_empty + STAGES;    // [2] per buffer, one phase per use: T1, T2 are in TMEM
    uint64_t* a_full = t_full + 2;          // [2] per buffer, one phase per use: the bf16 A operands are in TMEM
    uint64_t* acc_done = a_full + 2;        // [1] the last accumulating MMA has retired
    uint64_t* stat_bar = acc_done + 1;      // [1] one phase per step: the column statistics are in shared memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stat_bar + 1);

    const int warp = __shfl_sync(kFullMask, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int N = p.seq;
    const int n_tiles = (N + 127) / 128;
    // heaviest tiles first: under a causal mask the query side's last tiles and the key side's first tiles
    // walk the most other-side tiles
    // CTA order: heads in groups of p.head_group (RT_ATTN_BACKWARD_HEAD_GROUP, default 4); inside a group tile rank r (0 = heaviest) of every head comes
    // before rank r + 1.  A group's Q, K, V, dO (a few MB per head) stay in L2 while its CTAs run, and the grid's
    // last wave holds the group's lightest tiles instead of a head's heaviest.
    const int kHeadGroup = p.head_group;
    const int n_bh = (int)gridDim.x / n_tiles;
    const int grp = (int)blockIdx.x / (kHeadGroup * n_tiles);
    const int rem = (int)blockIdx.x - grp * kHeadGroup * n_tiles;
    const int in_grp = min(kHeadGroup, n_bh - grp * kHeadGroup);
    const int rank = rem / in_grp;
    const int own = kKeySide ? rank : (p.causal ? n_tiles - 1 - rank : rank);
    const int bh = grp * kHeadGroup + rem % in_grp, b = bh / p.heads, h = bh % p.heads;
    const int own0 = own * 128;
    // other-side tiles [t_lo, t_hi)
    const int t_lo = (kKeySide && p.causal) ? own : 0;
    const int t_hi = (!kKeySide && p.causal) ? own + 1 : n_tiles;
    const int n_steps = t_hi - t_lo;  // other-side tiles; each is two 64-row steps
    const int n_u = 2 * n_steps;

    if (warp == 8 && lane == 0) {
        prefetch_tensormap(&tm_x1);
        prefetch_tensormap(&tm_x2);
        prefetch_tensormap(&tm_y1);
        prefetch_tensormap(&tm_y2);
        mbar_init(x_full, 1);
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&y_full[i], 1);
            mbar_init(&y_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&t_full[i], 1);
            mbar_init(&a_full[i], 256);
        }
        mbar_init(acc_done, 1);
        mbar_init(stat_bar, 256);
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 8) {
        // ============================================================== TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(x_full, 2 * TILE);
#pragma unroll
            for (int s = 0; s < C::NSUB; ++s) {
                tma_load_4d(sX1 + s * SUB, &tm_x1, x_full, s * 64, own0, h, b);
                tma_load_4d(sX2 + s * SUB, &tm_x2, x_full, s * 64, own0, h, b);
            }
            int issued = 0;
            for (int u = 0; u < n_u; ++u) {
                const int st = u % STAGES;
                if (u >= STAGES && !mbar_wait(&y_empty[st], (uint32_t)(u / STAGES - 1) & 1u, p.status, kToBwdYEmpty)) break;
                mbar_arrive_expect_tx(&y_full[st], 2 * HALFT);
                uint8_t* dst = sY + st * 2 * HALFT;
                const int r0 = (t_lo + (u >> 1)) * 128 + (u & 1) * 64;
#pragma unroll
                for (int s = 0; s < C::NSUB; ++s) {
                    tma_load_4d(dst + s * HSUB, &tm_y1, &y_full[st], s * 64, r0, h, b);
                    tma_load_4d(dst + HALFT + s * HSUB, &tm_y2, &y_full[st], s * 64, r0, h, b);
                }
                issued = u + 1;
            }
            // Drain: every copy this thread issued must have landed before the CTA may exit.
            mbar_wait(x_full, 0, p.status, kToBwdDrain);
            for (int u = max(0, issued - STAGES); u < issued; ++u)
                mbar_wait(&y_full[u % STAGES], (uint32_t)(u / STAGES) & 1u, p.status, kToBwdDrain);
        }
    } else if (warp == 9) {
        // ============================================================== MMA issuer
        const bool leader = elect_one();
        constexpr uint32_t idesc_t = make_idesc_bf16(128, 64, 0, 0);
        constexpr uint32_t idesc_a = make_idesc_bf16(128, D, 0, 1);
        const uint64_t dx1 = make_smem_desc_sw128(smem_u32(sX1), 16, 1024);
        const uint64_t dx2 = make_smem_desc_sw128(smem_u32(sX2), 16, 1024);
        const uint64_t dy_k = make_smem_desc_sw128(smem_u32(sY), 16, 1024);    // other tile as a K-major operand
        const uint64_t dy_mn = make_smem_desc_sw128(smem_u32(sY), HSUB, 1024);  // the same rows as an MN-major operand
        const uint32_t tT = tmem_base + C::COL_T, tAcc = tmem_base + C::COL_ACC;
        auto commit = [&](uint64_t* bar) {
            if (leader) mma_commit(bar);
        };
        auto wait = [&](uint64_t* bar, uint32_t parity, int code) {
            return __all_sync(kFullMask, mbar_wait(bar, parity, p.status, code));
        };
        // T1 = X1 Y1^T, T2 = X2 Y2^T over the 64 other-side rows of step u, into buffer u & 1 (they overwrite
        // the A operands of step u - 2: the pipe runs this thread's MMAs in issue order, after the accumulating
        // MMAs of that step)
        auto issue_T = [&](int u) {
            const int st = u % STAGES;
            const uint64_t y1 = dy_k + (uint64_t)((st * 2 * HALFT) >> 4), y2 = y1 + (uint64_t)(HALFT >> 4);
            const uint32_t t1 = tT + (u & 1) * 128, t2 = t1 + 64;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t offx = (uint32_t)(((kk / 4) * SUB + (kk % 4) * 32) >> 4);
                const uint32_t offy = (uint32_t)(((kk / 4) * HSUB + (kk % 4) * 32) >> 4);
                if (leader) mma_ss(t1, dx1 + offx, y1 + offy, idesc_t, kk > 0);
            }
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t offx = (uint32_t)(((kk / 4) * SUB + (kk % 4) * 32) >> 4);
                const uint32_t offy = (uint32_t)(((kk / 4) * HSUB + (kk % 4) * 32) >> 4);
                if (leader) mma_ss(t2, dx2 + offx, y2 + offy, idesc_t, kk > 0);
            }
        };
        bool ok = wait(x_full, 0, kToBwdX);
        auto wait_rows = [&](int u) {  // the rows of step u have landed
            const bool got = wait(&y_full[u % STAGES], (uint32_t)(u / STAGES) & 1u, kToBwdYFull);
            tc_fence_after();
            return got;
        };
        if (ok && n_u > 0) {
            ok = wait_rows(0);
            if (ok) {
                issue_T(0);
                commit(&t_full[0]);
                ok = wait_rows(1);
            }
            if (ok) {
                issue_T(1);
                commit(&t_full[1]);
            }
        }
        for (int u = 0; u < n_u && ok; ++u) {
            const int st = u % STAGES;
            if (!wait(&a_full[u & 1], (uint32_t)(u >> 1) & 1u, kToBwdA)) break;
            tc_fence_after();
            const uint64_t y1 = dy_mn + (uint64_t)((st * 2 * HALFT) >> 4), y2 = y1 + (uint64_t)(HALFT >> 4);
            const uint32_t t1 = tT + (u & 1) * 128, t2 = t1 + 64;
            const uint32_t acc0 = u > 0 ? 1u : 0u;
            if (kKeySide) {
                // dV += P^T dO (A = P^T in the first 32 columns of T1, B = Y2 = dO), dK += dS^T Q (A in T2, B = Y1 = Q)
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    if (leader)
                        mma_ts(tAcc, t1 + kk * 8 + (kk >= 2 ? 16 : 0), y2 + (uint64_t)((kk * 2048) >> 4), idesc_a, kk > 0 ? 1u : acc0);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    if (leader)
                        mma_ts(tAcc + D, t2 + kk * 8 + (kk >= 2 ? 16 : 0), y1 + (uint64_t)((kk * 2048) >> 4), idesc_a, kk > 0 ? 1u : acc0);
            } else {
                // dQ += dS K (A = dS in the first 32 columns of T2, B = Y1 = K)
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    if (leader)
                        mma_ts(tAcc, t2 + kk * 8 + (kk >= 2 ? 16 : 0), y1 + (uint64_t)((kk * 2048) >> 4), idesc_a, kk > 0 ? 1u : acc0);
            }
            commit(&y_empty[st]);  // the step's rows are free once these MMAs (and the score MMAs before them) retire
            if (u + 2 < n_u) {
                if (!wait_rows(u + 2)) break;
                issue_T(u + 2);
                commit(&t_full[u & 1]);
            }
            if (u == n_u - 1) commit(acc_done);
        }
        if (n_u == 0) commit(acc_done);
    } else {
        // ============================================================== element-wise warps (two threads per own row)
        const int half = warp >> 2;  // which 32 of a step's 64 score columns
        const int r = (warp & 3) * 32 + lane;
        const int own_row = own0 + r;
        const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tT = tmem_base + lane_sel + C::COL_T;
        const uint32_t tAcc = tmem_base + lane_sel + C::COL_ACC;
        const float c = p.scale_log2;
        const int64_t stat_base = (int64_t)bh * N;
        float my_lse2 = 0.f, my_delta = 0.f;  // query side: this row's statistics
        if (!kKeySide && own_row < N) {
            const float x = p.lse[stat_base + own_row];
            my_lse2 = (x > -INFINITY && x < INFINITY) ? x * kLog2e : INFINITY;  // no visible key (or NaN): P = 0
            my_delta = p.delta[stat_base + own_row];
        }
        bool ok = true;
        for (int u = 0; u < n_u && ok; ++u) {
            const int t = u >> 1, st = t & 1, buf = u & 1;
            const int other0 = (t_lo + t) * 128 + buf * 64;  // first other-side row of this step
            float* s_lse2 = stat + st * 256;
            float* s_delta = s_lse2 + 128;
            if (kKeySide && buf == 0) {
                // the statistics of this tile's 128 queries (columns); the slot was last read two tiles ago, and
                // every thread has passed the a_full arrivals of that tile's successor by now
                if (half == 0) {
                    const int qi = other0 + r;
                    const float x = qi < N ? p.lse[stat_base + qi] : INFINITY;
                    s_lse2[r] = (x > -INFINITY && x < INFINITY) ? x * kLog2e : INFINITY;  // +inf -> P = 0
                    s_delta[r] = qi < N ? p.delta[stat_base + qi] : 0.f;
                }
                mbar_arrive(stat_bar);  // an mbarrier rather than bar.sync, so that this wait is bounded as well
                if (!__all_sync(kFullMask, mbar_wait(stat_bar, (uint32_t)t & 1u, p.status, kToBwdStat))) {
                    ok = false;
                    break;
                }
            }
            if (!__all_sync(kFullMask, mbar_wait(&t_full[buf], (uint32_t)(u >> 1) & 1u, p.status, kToBwdT))) {
                ok = false;
                break;
            }
            tc_fence_after();
            // Is any (own row, other index) pair of this step masked?  Only the diagonal tile of a causal
            // launch and the last tile of a ragged sequence are.
            const bool diag = p.causal && (t_lo + t) == own;
            const bool ragged = other0 + 64 > N;
            const uint32_t t1 = tT + buf * 128, t2 = t1 + 64;
            const float2 c2 = make_float2(c, c);
            {
                constexpr int ch = 0;  // this thread's single chunk: score columns [32 half, 32 half + 32) of the step
                const int cbase = half * 32;
                uint32_t a1[32], a2[32];
                tmem_ld32(t1 + cbase, a1);
                tmem_ld32(t2 + cbase, a2);
                tc_wait_ld();
                uint32_t pk_p[16], pk_ds[16];
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    // statistics of four columns: the row's own on the query side, one 16-byte broadcast read each
                    // on the key side (an LSE of +inf makes the probability 0: absent queries, rows without a key)
                    float4 l4, d4;
                    if (kKeySide) {
                        l4 = *reinterpret_cast<const float4*>(s_lse2 + buf * 64 + cbase + i);
                        d4 = *reinterpret_cast<const float4*>(s_delta + buf * 64 + cbase + i);
                    } else {
                        l4 = make_float4(my_lse2, my_lse2, my_lse2, my_lse2);
                        d4 = make_float4(my_delta, my_delta, my_delta, my_delta);
                    }
                    const float2 xa = __ffma2_rn(make_float2(__uint_as_float(a1[i]), __uint_as_float(a1[i + 1])), c2,
                                                 make_float2(-l4.x, -l4.y));
                    const float2 xb = __ffma2_rn(make_float2(__uint_as_float(a1[i + 2]), __uint_as_float(a1[i + 3])), c2,
                                                 make_float2(-l4.z, -l4.w));
                    float2 pa = make_float2(fast_exp2(xa.x), fast_exp2(xa.y));
                    float2 pb = make_float2(fast_exp2(xb.x), fast_exp2(xb.y));
                    if (diag || ragged) {
                        const int o0 = other0 + cbase + i;
                        auto hidden = [&](int other) {
                            return other >= N || (p.causal && (kKeySide ? own_row > other : other > own_row));
                        };
                        if (hidden(o0)) pa.x = 0.f;
                        if (hidden(o0 + 1)) pa.y = 0.f;
                        if (hidden(o0 + 2)) pb.x = 0.f;
                        if (hidden(o0 + 3)) pb.y = 0.f;
                    }
                    const float2 ta = __fadd2_rn(make_float2(__uint_as_float(a2[i]), __uint_as_float(a2[i + 1])),
                                                 make_float2(-d4.x, -d4.y));
                    const float2 tb = __fadd2_rn(make_float2(__uint_as_float(a2[i + 2]), __uint_as_float(a2[i + 3])),
                                                 make_float2(-d4.z, -d4.w));
                    const float2 da = __fmul2_rn(pa, ta), db = __fmul2_rn(pb, tb);
                    pk_p[i / 2] = float2_to_bf16x2(pa.x, pa.y);
                    pk_p[i / 2 + 1] = float2_to_bf16x2(pb.x, pb.y);
                    pk_ds[i / 2] = float2_to_bf16x2(da.x, da.y);
                    pk_ds[i / 2 + 1] = float2_to_bf16x2(db.x, db.y);
                }
                // the 32 bf16 values go into the first 16 of this thread's own 32 columns (in registers by now)
                (void)ch;
                if (kKeySide) tmem_st16(t1 + cbase, pk_p);
                tmem_st16(t2 + cbase, pk_ds);
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(&a_full[buf]);
        }
        // ---- read-out: accumulators -> f32 global (scale folded into dQ and dK)
        if (ok && __all_sync(kFullMask, mbar_wait(acc_done, 0, p.status, kToBwdAcc))) {
            tc_fence_after();
            constexpr int kOuts = kKeySide ? 2 : 1;
            constexpr int OC = D / 2;  // accumulator columns per thread
#pragma unroll
            for (int o = 0; o < kOuts; ++o) {
                float* dst = (o == 0 ? p.out1 : p.out2) + ((int64_t)bh * N + own_row) * D + half * OC;
                const float mul = (kKeySide && o == 0) ? 1.f : p.scale;  // dV is not scaled
#pragma unroll
                for (int ch = 0; ch < OC / 32; ++ch) {
                    uint32_t a[32];
                    tmem_ld32(tAcc + o * D + half * OC + ch * 32, a);
                    tc_wait_ld();
                    if (own_row < N) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4*>(dst + ch * 32 + i) =
                                make_float4(__uint_as_float(a[i]) * mul, __uint_as_float(a[i + 1]) * mul,
                                            __uint_as_float(a[i + 2]) * mul, __uint_as_float(a[i + 3]) * mul);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <int D, bool kKeySide>
cudaError_t launch_side(const CUtensorMap& x1, const CUtensorMap& x2, const CUtensorMap& y1, const CUtensorMap& y2,
                        const Bwd5Params& p, int64_t bh, cudaStream_t stream) {
    cudaError_t e = set_max_dynamic_smem_once<bwd_tcgen05_kernel<D, kKeySide>>(BwdCfg<D>::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const int64_t n_ctas = ((p.seq + 127) / 128) * bh;
    if (n_ctas > 0x7fffffff) return cudaErrorInvalidValue;
    dim3 grid((unsigned)n_ctas);
    bwd_tcgen05_kernel<D, kKeySide><<<grid, 320, BwdCfg<D>::SMEM_BYTES, stream>>>(x1, x2, y1, y2, p);
    return cudaGetLastError();
}

}  // namespace

// Returns cudaErrorNotSupported when this kernel does not cover the shape (the caller then uses the
// mma.sync kernel).
cudaError_t launch_backward_tcgen05(const void* q, const void* k, const void* v, const void* d_out, const float* lse,
                                    const float* delta, float* dq, float* dk, float* dv, int64_t batch, int64_t heads,
                                    int64_t seq, int dim, int causal, float scale, cudaStream_t stream) {
    const int64_t bh = batch * heads;
    if ((dim != 64 && dim != 128) || bh > 65535 || seq > (1 << 30)) return cudaErrorNotSupported;
    // own-side tiles are 128-row boxes, other-side steps 64-row boxes of the same tensors
    CUtensorMap mq, mk, mv, mdo, hq, hk, hv, hdo;
    const TensorStrides s = TensorStrides::contiguous(heads, seq, dim);
    const void* ptrs[4] = {q, k, v, d_out};
    CUtensorMap* full[4] = {&mq, &mk, &mv, &mdo};
    CUtensorMap* half[4] = {&hq, &hk, &hv, &hdo};
    for (int i = 0; i < 4; ++i)
        if (!make_tensor_map_bf16_4d(full[i], ptrs[i], batch, heads, seq, dim, s.batch, s.head, s.row, 128) ||
            !make_tensor_map_bf16_4d(half[i], ptrs[i], batch, heads, seq, dim, s.batch, s.head, s.row, 64))
            return cudaErrorNotSupported;
    Bwd5Params p;
    p.lse = lse;
    p.delta = delta;
    p.seq = (int)seq;
    p.heads = (int)heads;
    p.causal = causal;
    p.scale = scale;
    p.scale_log2 = scale * kLog2e;
    p.status = device_status_ptr();
    if (!p.status) return cudaErrorInvalidSymbol;
    static const int env_group = [] {
        const char* e = getenv("RT_ATTN_BACKWARD_HEAD_GROUP");
        const int v = e ? atoi(e) : 0;
        return v > 0 ? v : 4;  // measured: 2-4 about 1 % ahead of 1 (head-major), 16 level, 128 slower by 20 % (L2)
    }();
    p.head_group = env_group;
    // query side: own (Q, dO), other (K, V) -> dQ
    p.out1 = dq;
    p.out2 = nullptr;
    cudaError_t e = dim == 128 ? launch_side<128, false>(mq, mdo, hk, hv, p, bh, stream)
                               : launch_side<64, false>(mq, mdo, hk, hv, p, bh, stream);
    if (e != cudaSuccess) return e;
    // key side: own (K, V), other (Q, dO) -> dV, dK
    p.out1 = dv;
    p.out2 = dk;
    return dim == 128 ? launch_side<128, true>(mk, mv, hq, hdo, p, bh, stream)
                      : launch_side<64, true>(mk, mv, hq, hdo, p, bh, stream);
}

}  // namespace rt
