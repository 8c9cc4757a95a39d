// Flash-attention forward on the Blackwell tensor cores (tcgen05 + TMEM + TMA), bf16.
//
// Replaces rustorch_attention::flash_forward_masked (crates/rustorch-attention/src/cpu_forward.rs:193-425)
// for bf16 device tensors of head dim 64 or 128.  The recurrence is the reference's online
// softmax (cpu_forward.rs:355-386) evaluated in the log2 domain; unlike the reference, KV tiles
// that a causal mask or a per-batch kv_len hides completely are never visited.
//
// CTA = 256 query rows of one (batch, head) = two 128-row Q tiles that ping-pong on the tensor
// pipe, so the softmax of one tile overlaps the MMAs of the other.  384 threads = 3 warpgroups:
//   warps 0-3  : softmax + lazy O rescale + epilogue of Q tile 0 (one thread per query row)
//   warps 4-7  : the same for Q tile 1
//   warp  8    : TMA producer (Q once, then K_j / V_j through their rings)
//   warp  9    : TMEM allocation and the single thread that issues every tcgen05.mma
//   warps 10-11: idle (they complete the third warpgroup so that setmaxnreg can move its
//                registers to the softmax warpgroups: 72 vs 216 registers per thread)
// TMEM (512 columns x 128 lanes, f32): per Q tile two 64-column S buffers (S[w][b] at w*128 + b*64),
// O0 [256,256+D), O1 [256+D,256+2D).  K/V are loaded as 128-key tiles but multiplied in 64-key
// steps; P (bf16) overwrites the first 32 columns of its S buffer and feeds the PV MMA from TMEM.
// S = Q K^T is an SS MMA with both operands K-major in 128-byte-swizzled shared memory; O += P V
// is a TS MMA whose B operand (V) is MN-major, i.e. V is used exactly as TMA lands it.
// Every mbarrier wait is bounded; on expiry the kernel records a code in the device status
// word, drains its own copies and MMAs, frees TMEM and returns.
#include <cuda.h>
#include <mutex>

#include "kernels.h"
#include "tc_ptx.cuh"

namespace rt {

using namespace ptx;

template <int D>
struct TcCfg {
    static constexpr int BM = 128;                      // query rows per tile
    static constexpr int BL = 128;                      // keys per TMA-loaded K/V tile
    static constexpr int BN = 64;                       // keys per MMA / softmax step
    static constexpr int KS = (D == 128) ? 3 : 4;       // K ring depth (runs one tile ahead of V)
    static constexpr int VS = (D == 128) ? 2 : 4;       // V ring depth
    static constexpr int TILE_BYTES = 128 * D * 2;
    static constexpr int SUB_BYTES = 128 * 64 * 2;      // one 64-column (128-byte) swizzled sub-tile
    static constexpr int HALF_BYTES = 64 * 128;         // 64 rows inside a sub-tile
    static constexpr int NSUB = D / 64;
    static constexpr int NBARS = 2 + 2 * KS + 2 * VS + 4 + 4 + 2 + 2 + 1;
    static constexpr int SMEM_BYTES = (2 + KS + VS) * TILE_BYTES + NBARS * 8 + 16 + 1024;
    static constexpr uint32_t TMEM_COLS = 512;
    static constexpr uint32_t COL_S = 0, COL_O = 256;   // S: tile w, buffer b at COL_S + w*128 + b*64
};

struct TcParams {
    __nv_bfloat16* out;
    float* lse;
    const int32_t* kv_lens;
    const uint8_t* key_keep;
    int64_t keep_batch_stride;
    int seq, heads;        // query rows per head, query heads
    int seq_kv, heads_kv;  // key rows per KV head, KV heads (query head h reads KV head h / (heads/heads_kv))
    const int32_t* q_offsets;  // NULL or [B]: causal position of query row 0 inside the key sequence
    float scale_log2;  // scale * log2(e)
    int* status;       // device status word (bounded-wait expiry codes)
#ifdef RT_TC_TIMELINE
    long long* timeline;  // profiling builds only: clock64 stamps of CTA 0 (see TL_* below)
#endif
};

#ifdef RT_TC_TIMELINE
// Profiling aid, compiled only with -DRT_TC_TIMELINE: one thread per role of CTA 0 stamps clock64
// at the phase boundaries of every step.  Layout: [role 0..2][step][8] (role 0/1 = softmax of Q
// tile 0/1, role 2 = MMA issuer).
#define TL_STAMP(role, step, slot)                                                                     \
    do {                                                                                               \
        if (p.timeline && blockIdx.x == 0 && (step) < 256)                                             \
            p.timeline[(((role) * 256) + (step)) * 8 + (slot)] = clock64();                            \
    } while (0)
static long long* g_tc_timeline = nullptr;
extern "C" void rt_debug_set_tc_timeline(void* ptr) { g_tc_timeline = (long long*)ptr; }
#else
#define TL_STAMP(role, step, slot) do { } while (0)
#endif

// Timeout codes written to the device status word (100 + site).
enum { kToQ = 101, kToKFull, kToKEmpty, kToVFull, kToVEmpty, kToSFull, kToPFull, kToOFull, kToDone, kToDrain };

// Pipeline, per Q tile w and 64-key step u (buffer b = u & 1):
//   MMA:     S_w(u) -> TMEM S[w][b]            (SS, N = 64, D/16 k-steps)       commit s_full[w][b]
//   softmax: S[w][b] -> registers -> P (bf16) over the first 32 columns of S[w][b]   arrive p_full[w][b]
//   MMA:     O_w += P V(u)                      (TS, N = D, 4 k-steps)           commit o_full[w]
//            then S_w(u+2) into the same buffer (in-order after the PV that read P from it)
// S is double-buffered, so the softmax of step u+1 never waits for the PV of step u; the
// softmax warps of both tiles keep the MUFU pipe busy while the tensor pipe runs behind them.
template <int D, bool kCausal, bool kKeep>
__global__ void __launch_bounds__(384, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                  const TcParams p) {
    using C = TcCfg<D>;
    constexpr int KS = C::KS, VS = C::VS, TILE = C::TILE_BYTES, SUB = C::SUB_BYTES, HALF = C::HALF_BYTES;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + 2 * TILE;
    uint8_t* sV = sK + KS * TILE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + VS * TILE);
    uint64_t* q_full = bars;              // [2]
    uint64_t* k_full = q_full + 2;        // [KS]
    uint64_t* k_empty = k_full + KS;      // [KS]
    uint64_t* v_full = k_empty + KS;      // [VS]
    uint64_t* v_empty = v_full + VS;      // [VS]
    uint64_t* s_full = v_empty + VS;      // [2 tiles][2 buffers]
    uint64_t* p_full = s_full + 4;        // [2 tiles][2 buffers]
    uint64_t* o_full = p_full + 4;        // [2]  one phase per PV step (O at rest for a rescale)
    uint64_t* o_done = o_full + 2;        // [2]  single phase: the last PV of the tile has retired
    uint64_t* done_bar = o_done + 2;      // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);

    // Broadcasting the warp index makes it provably warp-uniform, so role dispatch and the MMA
    // operands stay on the uniform datapath.
    const int warp = __shfl_sync(kFullMask, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int N = p.seq;
    const int n_qb = (N + 255) / 256;
    const int bh = blockIdx.x / n_qb;
    const int qb = n_qb - 1 - (int)(blockIdx.x % n_qb);  // heaviest causal block of a head first
    const int b = bh / p.heads;
    const int bh_kv = b * p.heads_kv + (bh % p.heads) / (p.heads / p.heads_kv);
    const int q0 = qb * 256;
    const int Nkv = p.seq_kv;

    int kv_hi = Nkv;
    if (p.kv_lens) {
        const int l = p.kv_lens[b];
        kv_hi = l < 0 ? 0 : (l < Nkv ? l : Nkv);
    }
    const int q_off = p.q_offsets ? p.q_offsets[b] : 0;  // query row i sits at key position i + q_off
    const int n_steps = (kv_hi + 63) / 64;  // 64-key steps that hold a visible key
    int U[2];                               // steps of each Q tile (U[0] <= U[1])
#pragma unroll
    for (int w = 0; w < 2; ++w) {
        const int last_key = q0 + 128 * w + 127 + q_off;  // last key the tile's last row may see
        U[w] = !kCausal ? n_steps : (last_key < 0 ? 0 : min(n_steps, last_key / 64 + 1));
    }
    const int u_max = U[1];
    const int n_tiles = (u_max + 1) / 2;    // 128-key K/V tiles to load

    if (u_max == 0) {  // no visible key at all: NaN rows, LSE = -inf (cpu_forward.rs:411-420)
        if (warp < 8) {
            const int row = q0 + warp * 32 + lane;
            if (row < N) {
                uint4 nan4 = make_uint4(0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u);
                uint4* dst = reinterpret_cast<uint4*>(p.out + ((int64_t)bh * N + row) * D);
#pragma unroll
                for (int i = 0; i < D / 8; ++i) dst[i] = nan4;
                if (p.lse) p.lse[(int64_t)bh * N + row] = -INFINITY;
            }
        }
        return;
    }

    // ------------------------------------------------------------------ setup
    if (warp == 8 && lane == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_o);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&q_full[i], 1);
            mbar_init(&o_full[i], 1);
            mbar_init(&o_done[i], 1);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
        }
        for (int i = 0; i < KS; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
        }
        for (int i = 0; i < VS; ++i) {
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        mbar_init(done_bar, 1);
        fence_barrier_init();
        fence_proxy_async();
        // Q and the first K tile are requested right away, so their latency overlaps the TMEM
        // allocation and the CTA-wide barrier below (the producer loop starts at K tile 1).
        for (int w = 0; w < 2; ++w) {
            mbar_arrive_expect_tx(&q_full[w], TILE);
#pragma unroll
            for (int s = 0; s < C::NSUB; ++s)
                tma_load_3d(sQ + w * TILE + s * SUB, &tm_q, &q_full[w], s * 64, q0 + w * 128, bh);
            if (w == 0) {
                mbar_arrive_expect_tx(&k_full[0], TILE);
#pragma unroll
                for (int s = 0; s < C::NSUB; ++s)
                    tma_load_3d(sK + s * SUB, &tm_k, &k_full[0], s * 64, 0, bh_kv);
            }
        }
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // The register hand-over sits inside each role's own branch: the compiler budgets the code
    // that follows a setmaxnreg only when no path with a different budget merges into it.
    if (warp >= 8) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
      if (warp == 8) {
        // ============================================================== TMA producer
        if (lane == 0) {
            int k_issued = 1, v_issued = 0;  // Q and K tile 0 were requested during setup
            for (int j = 0; j < n_tiles; ++j) {
                const int ks = j % KS, vs = j % VS;
                if (j > 0) {
                    if (!mbar_wait(&k_empty[ks], ((uint32_t)(j / KS) & 1u) ^ 1u, p.status, kToKEmpty)) break;
                    mbar_arrive_expect_tx(&k_full[ks], TILE);
#pragma unroll
                    for (int s = 0; s < C::NSUB; ++s)
                        tma_load_3d(sK + ks * TILE + s * SUB, &tm_k, &k_full[ks], s * 64, j * 128, bh_kv);
                    k_issued = j + 1;
                }
                if (!mbar_wait(&v_empty[vs], ((uint32_t)(j / VS) & 1u) ^ 1u, p.status, kToVEmpty)) break;
                mbar_arrive_expect_tx(&v_full[vs], TILE);
#pragma unroll
                for (int s = 0; s < C::NSUB; ++s)
                    tma_load_3d(sV + vs * TILE + s * SUB, &tm_v, &v_full[vs], s * 64, j * 128, bh_kv);
                v_issued = j + 1;
            }
            // Drain: every copy this thread issued must have landed before the CTA may exit.
            mbar_wait(&q_full[0], 0, p.status, kToDrain);
            mbar_wait(&q_full[1], 0, p.status, kToDrain);
            for (int j = max(0, k_issued - KS); j < k_issued; ++j)
                mbar_wait(&k_full[j % KS], (uint32_t)(j / KS) & 1u, p.status, kToDrain);
            for (int j = max(0, v_issued - VS); j < v_issued; ++j)
                mbar_wait(&v_full[j % VS], (uint32_t)(j / VS) & 1u, p.status, kToDrain);
        }
      } else if (warp == 9) {
        // ============================================================== MMA issuer
        // The whole warp runs this loop with uniform control flow and only the elected lane
        // executes the tcgen05 instructions: descriptors, addresses and loop state then live in
        // uniform registers, which is what the MMA instruction takes its operands from.
        {
            const bool leader = elect_one();
            constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);
            constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
            // Descriptors are built once; each MMA only adds an offset (in 16-byte units) to the
            // start-address field, so the issuing thread keeps ahead of the tensor pipe.
            const uint64_t dq = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);
            const uint64_t dk = make_smem_desc_sw128(smem_u32(sK), 16, 1024);
            const uint64_t dv = make_smem_desc_sw128(smem_u32(sV), SUB, 1024);
            const uint32_t tS0 = tmem_base + C::COL_S, tO0 = tmem_base + C::COL_O;
            // S_w(u): keys [64u, 64u+64) = rows (u&1)*64.. of K tile u/2
            auto issue_S = [&](int w, int u) {
                const uint64_t a = dq + (uint64_t)((w * TILE) >> 4);
                const uint64_t bk = dk + (uint64_t)((((u >> 1) % KS) * TILE + (u & 1) * HALF) >> 4);
                const uint32_t d = tS0 + w * 128 + (u & 1) * 64;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (uint32_t)(((kk / 4) * SUB + (kk % 4) * 32) >> 4);
                    if (leader) mma_ss(d, a + off, bk + off, idesc_s, kk > 0);
                }
            };
            // O_w += P V(u): P (bf16) sits in the first 32 columns of S[w][u&1]
            auto issue_PV = [&](int w, int u) {
                const uint64_t bv = dv + (uint64_t)((((u >> 1) % VS) * TILE + (u & 1) * HALF) >> 4);
                const uint32_t a = tS0 + w * 128 + (u & 1) * 64;
                const uint32_t acc0 = u > 0 ? 1u : 0u;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    if (leader) mma_ts(tO0 + w * D, a + kk * 8, bv + (uint64_t)((kk * 2048) >> 4), idesc_o, kk > 0 ? 1u : acc0);
            };
            auto commit = [&](uint64_t* bar) {
                if (leader) mma_commit(bar);
            };
            auto wait = [&](uint64_t* bar, uint32_t parity, int code) {
                return __all_sync(kFullMask, mbar_wait(bar, parity, p.status, code));
            };
            auto last_use = [&](int u) { return (u & 1) || u == U[1] - 1; };  // of a 128-key tile, by Q tile 1

            bool ok = wait(&k_full[0], 0, kToKFull);
            if (ok && U[0] > 0) {
                ok = wait(&q_full[0], 0, kToQ);
                if (ok) {
                    tc_fence_after();
                    issue_S(0, 0);
                    commit(&s_full[0]);
                    if (U[0] > 1) {
                        issue_S(0, 1);
                        commit(&s_full[1]);
                    }
                }
            }
            if (ok) ok = wait(&q_full[1], 0, kToQ);
            if (ok) {
                tc_fence_after();
                issue_S(1, 0);
                commit(&s_full[2]);
                if (last_use(0)) commit(&k_empty[0]);
                if (U[1] > 1) {
                    issue_S(1, 1);
                    commit(&s_full[3]);
                    commit(&k_empty[0]);
                }
            }
            int k_waited = 0, v_waited = -1;
            for (int u = 0; u < u_max && ok; ++u) {
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    if (!ok || u >= U[w]) continue;
                    const int vt = u >> 1;
                    if (vt > v_waited) {
                        if (!wait(&v_full[vt % VS], (uint32_t)(vt / VS) & 1u, kToVFull)) { ok = false; continue; }
                        v_waited = vt;
                    }
                    TL_STAMP(2, u, w * 4 + 0);
                    if (!wait(&p_full[w * 2 + (u & 1)], (uint32_t)(u >> 1) & 1u, kToPFull)) { ok = false; continue; }
                    TL_STAMP(2, u, w * 4 + 1);
                    tc_fence_after();
                    issue_PV(w, u);
                    commit(&o_full[w]);
                    if (u == U[w] - 1) commit(&o_done[w]);
                    if (w == 1 && last_use(u)) commit(&v_empty[vt % VS]);
                    if (u + 2 < U[w]) {
                        const int kt = (u + 2) >> 1;
                        if (kt > k_waited) {
                            if (!wait(&k_full[kt % KS], (uint32_t)(kt / KS) & 1u, kToKFull)) { ok = false; continue; }
                            k_waited = kt;
                            tc_fence_after();
                        }
                        TL_STAMP(2, u, w * 4 + 2);
                        issue_S(w, u + 2);
                        commit(&s_full[w * 2 + (u & 1)]);
                        if (w == 1 && last_use(u + 2)) commit(&k_empty[kt % KS]);
                    }
                    TL_STAMP(2, u, w * 4 + 3);
                }
            }
            // All MMAs issued by this thread must retire before TMEM is freed.
            commit(done_bar);
            wait(done_bar, 0, kToDone);
        }
      }  // warps 10-11 idle: they only complete the warpgroup for setmaxnreg
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        // ============================================================== softmax / epilogue warps
        const int w = warp >> 2;                       // Q tile
        const int row_in_tile = (warp & 3) * 32 + lane;
        const int row = q0 + w * 128 + row_in_tile;    // query index within the sequence
        const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tS = tmem_base + lane_sel + C::COL_S + w * 128;
        const uint32_t tO = tmem_base + lane_sel + C::COL_O + w * D;
        const float c = p.scale_log2;
        const uint8_t* keep = kKeep ? p.key_keep + (int64_t)b * p.keep_batch_stride : nullptr;

        float m_ref = -INFINITY;  // reference max (raw score units) the running sums are relative to
        float l = 0.f;
        bool ok = true;
        const int n_iter = U[w];

        for (int u = 0; u < n_iter; ++u) {
            const int buf = u & 1;
            if ((warp & 3) == 0 && lane == 0) TL_STAMP(w, u, 0);
            if (!__all_sync(kFullMask, mbar_wait(&s_full[w * 2 + buf], (uint32_t)(u >> 1) & 1u, p.status, kToSFull))) {
                ok = false;
                break;
            }
            tc_fence_after();
            if ((warp & 3) == 0 && lane == 0) TL_STAMP(w, u, 1);

            uint32_t s[64];
            {
                uint32_t(&s0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[0]);
                uint32_t(&s1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[32]);
                tmem_ld32(tS + buf * 64, s0);
                tmem_ld32(tS + buf * 64 + 32, s1);
                tc_wait_ld();
            }
            if ((warp & 3) == 0 && lane == 0) TL_STAMP(w, u, 2);

            // ---- masks: keys beyond kv_hi, causal diagonal, keep flags
            const int col0 = u * 64;
            int lim = kv_hi - 1 - col0;                       // last visible column in this step
            if (kCausal) lim = min(lim, row + q_off - col0);
            if (lim < 63) {
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (i > lim) s[i] = 0xff800000u;  // -inf
            }
            if (kKeep) {  // Mask::Padding keep flags (mask.rs:44); every thread reads the same bytes
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (col0 + i < Nkv && __ldg(keep + col0 + i) == 0) s[i] = 0xff800000u;
            }

            // ---- row max (three-input max halves the instruction count)
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 64; i += 8) {
                mx0 = max3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
                mx1 = max3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
                mx2 = max3(mx2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
                mx3 = max3(mx3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));

            // ---- lazy rescale: move the reference max only when it would grow by > 2^8
            if (u == 0) {
                m_ref = mx;
            } else {
                const bool need = (mx > m_ref) && ((mx - m_ref) * c > 8.0f || m_ref == -INFINITY);
                if (__any_sync(kFullMask, need)) {
                    // O must be at rest: the PV of the previous step has to be complete.
                    if (!__all_sync(kFullMask, mbar_wait(&o_full[w], (uint32_t)(u - 1) & 1u, p.status, kToOFull))) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const float m_new = fmaxf(m_ref, mx);
                    const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2((m_ref - m_new) * c);
                    l *= alpha;
                    m_ref = m_new;
#pragma unroll
                    for (int ch = 0; ch < D / 32; ++ch) {
                        uint32_t o[32];
                        tmem_ld32(tO + ch * 32, o);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(tO + ch * 32, o);
                    }
                    tc_wait_st();
                }
            }

            if ((warp & 3) == 0 && lane == 0) TL_STAMP(w, u, 3);
            // ---- P = exp2(s*c - m*c), row sum, bf16 pack, store to TMEM over S (packed f32x2 math)
            const float mc = (m_ref == -INFINITY) ? 0.f : m_ref * c;
            const float2 c2 = make_float2(c, c), nmc2 = make_float2(-mc, -mc);
            float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    const float2 xa = __ffma2_rn(
                        make_float2(__uint_as_float(s[ch * 32 + 2 * i]), __uint_as_float(s[ch * 32 + 2 * i + 1])), c2, nmc2);
                    const float2 xb = __ffma2_rn(
                        make_float2(__uint_as_float(s[ch * 32 + 2 * i + 2]), __uint_as_float(s[ch * 32 + 2 * i + 3])), c2,
                        nmc2);
                    const float2 pa = make_float2(fast_exp2(xa.x), fast_exp2(xa.y));
                    const float2 pb = make_float2(fast_exp2(xb.x), fast_exp2(xb.y));
                    sum_a = __fadd2_rn(sum_a, pa);
                    sum_b = __fadd2_rn(sum_b, pb);
                    pk[i] = float2_to_bf16x2(pa.x, pa.y);
                    pk[i + 1] = float2_to_bf16x2(pb.x, pb.y);
                }
                tmem_st16(tS + buf * 64 + ch * 16, pk);
            }
            l += (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
            if ((warp & 3) == 0 && lane == 0) TL_STAMP(w, u, 4);
            tc_wait_st();
            if ((warp & 3) == 0 && lane == 0) TL_STAMP(w, u, 5);
            tc_fence_before();
            mbar_arrive(&p_full[w * 2 + buf]);
        }

        if (n_iter == 0) {  // this tile sees no key (its rows lie before the first visible position)
            if (row < N) {
                uint4* dst = reinterpret_cast<uint4*>(p.out + ((int64_t)bh * N + row) * D);
#pragma unroll
                for (int i = 0; i < D / 8; ++i) dst[i] = make_uint4(0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u);
                if (p.lse) p.lse[(int64_t)bh * N + row] = -INFINITY;
            }
            ok = false;
        }
        // ---- epilogue: O / l -> bf16 into the (now idle) shared-memory tile of Q_w in the swizzled
        // layout of the output tensor map, then one TMA store per 64-column half: 16-byte shared stores
        // instead of row-strided global stores, and rows past N are clipped by the hardware.
        // (o_full cannot be used for the wait: up to two PV steps may still be in flight, which a
        // parity wait cannot tell from none.)
        bool stored = false;
        if (ok && __all_sync(kFullMask, mbar_wait(&o_done[w], 0, p.status, kToOFull))) {
            tc_fence_after();
            const bool valid = (l > 0.f);
            const float inv = valid ? 1.f / l : 0.f;
            uint8_t* stage = sQ + w * TILE + row_in_tile * 128;  // every score MMA that read Q_w has retired
#pragma unroll
            for (int ch = 0; ch < D / 32; ++ch) {
                uint32_t o[32];
                tmem_ld32(tO + ch * 32, o);
                tc_wait_ld();
#pragma unroll
                for (int v4 = 0; v4 < 4; ++v4) {
                    uint4 pack;
                    uint32_t* pw = reinterpret_cast<uint32_t*>(&pack);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float a = __uint_as_float(o[v4 * 8 + 2 * i]) * inv;
                        const float bb = __uint_as_float(o[v4 * 8 + 2 * i + 1]) * inv;
                        pw[i] = valid ? float2_to_bf16x2(a, bb) : 0x7fc07fc0u;
                    }
                    const int cc = ch * 4 + v4;  // 16-byte chunk of the row: sub-tile cc/8, chunk cc%8
                    *reinterpret_cast<uint4*>(stage + (cc / 8) * SUB + (((cc % 8) ^ (row_in_tile & 7)) << 4)) = pack;
                }
            }
            if (p.lse && row < N)
                p.lse[(int64_t)bh * N + row] =
                    valid ? (m_ref * c + fast_log2(l)) * kLn2 : (l == 0.f ? -INFINITY : NAN);
            fence_proxy_async();  // generic-proxy writes above -> visible to the TMA (async proxy) read
            stored = true;
        }
        named_barrier_sync(1 + w, 128);  // all four warps of the tile, whatever happened above
        if (row_in_tile == 0 && stored) {
#pragma unroll
            for (int s = 0; s < C::NSUB; ++s)
                tma_store_3d(&tm_o, sQ + w * TILE + s * SUB, s * 64, q0 + w * 128, bh);
            tma_store_commit_and_wait();  // the tile must be read out before the CTA gives up its shared memory
        }
    }

    // ------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------- host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

EncodeTiledFn tensor_map_encoder() { return get_encode_fn(); }

// View of a [B*H, N, D] bf16 tensor as a 3-D TMA tensor; box = 64 columns x 128 rows of one
// (b,h), 128-byte swizzle.  Rows past N are zero-filled, so tiles never read a neighbour head.
bool make_tensor_map_bf16_3d(CUtensorMap* map, const void* base, int64_t bh, int64_t seq, int dim) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return false;
    cuuint64_t dims[3] = {(cuuint64_t)dim, (cuuint64_t)seq, (cuuint64_t)bh};
    cuuint64_t strides[2] = {(cuuint64_t)dim * 2, (cuuint64_t)seq * dim * 2};
    cuuint32_t box[3] = {64, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D, bool kCausal, bool kKeep>
static cudaError_t launch_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                             const TcParams& p, int64_t n_ctas, cudaStream_t stream) {
    auto kern = prefill_tc_kernel<D, kCausal, kKeep>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<D>::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)n_ctas, 384, TcCfg<D>::SMEM_BYTES, stream>>>(mq, mk, mv, mo, p);
    return cudaGetLastError();
}

cudaError_t launch_prefill_tc(const void* q, const void* k, const void* v, void* out, float* lse, int64_t batch,
                              int64_t heads, int64_t heads_kv, int64_t seq, int64_t seq_kv, int dim, int causal,
                              const int32_t* kv_lens, const int32_t* q_offsets, const uint8_t* key_keep,
                              int64_t keep_batch_stride, float scale, cudaStream_t stream) {
    const int64_t bh = batch * heads;
    if (bh == 0 || seq == 0) return cudaSuccess;
    CUtensorMap mq, mk, mv, mo;
    if (!make_tensor_map_bf16_3d(&mq, q, bh, seq, dim) || !make_tensor_map_bf16_3d(&mo, out, bh, seq, dim) ||
        !make_tensor_map_bf16_3d(&mk, k, batch * heads_kv, seq_kv, dim) ||
        !make_tensor_map_bf16_3d(&mv, v, batch * heads_kv, seq_kv, dim))
        return cudaErrorInvalidValue;
    TcParams p;
    p.out = (__nv_bfloat16*)out;
    p.lse = lse;
    p.kv_lens = kv_lens;
    p.key_keep = key_keep;
    p.keep_batch_stride = keep_batch_stride;
    p.seq = (int)seq;
    p.heads = (int)heads;
    p.seq_kv = (int)seq_kv;
    p.heads_kv = (int)heads_kv;
    p.q_offsets = q_offsets;
    p.scale_log2 = scale * kLog2e;
    p.status = device_status_ptr();
    if (!p.status) return cudaErrorInvalidSymbol;
#ifdef RT_TC_TIMELINE
    p.timeline = g_tc_timeline;
#endif
    const int64_t n_ctas = bh * ((seq + 255) / 256);
    if (n_ctas > 0x7fffffff) return cudaErrorInvalidValue;
    const bool keep = key_keep != nullptr;
#define RT_TC_DISPATCH(DD)                                                                         \
    if (causal) {                                                                                  \
        return keep ? launch_tc<DD, true, true>(mq, mk, mv, mo, p, n_ctas, stream)                     \
                    : launch_tc<DD, true, false>(mq, mk, mv, mo, p, n_ctas, stream);                   \
    } else {                                                                                       \
        return keep ? launch_tc<DD, false, true>(mq, mk, mv, mo, p, n_ctas, stream)                    \
                    : launch_tc<DD, false, false>(mq, mk, mv, mo, p, n_ctas, stream);                  \
    }
    if (dim == 128) { RT_TC_DISPATCH(128) }
    if (dim == 64) { RT_TC_DISPATCH(64) }
#undef RT_TC_DISPATCH
    return cudaErrorInvalidValue;
}

}  // namespace rt
