// Flash-attention forward on the Blackwell tensor cores (tcgen05 + TMEM + TMA), bf16.
//
// Replaces rustorch_attention::flash_forward_masked (crates/rustorch-attention/src/cpu_forward.rs:193-425)
// for bf16 device tensors of head dim 64 or 128.  The recurrence is the reference's online
// softmax (cpu_forward.rs:355-386) evaluated in the log2 domain; unlike the reference, KV tiles
// that a causal mask or a per-batch kv_len hides completely are never visited.
//
// Work item = 256 query rows of one (batch, head) = two 128-row Q tiles that share the K/V tiles
// in shared memory and ping-pong on the tensor pipe.  The kernel is persistent: one CTA per SM
// walks a static list of items (see tc_item), and every barrier runs on phase counters that
// carry over from item to item, so the next item's loads and first score MMAs overlap the
// previous item's last steps and write-back.  384 threads = 3 warpgroups:
//   warps 0-3  : softmax + lazy O rescale + epilogue of Q tile 0 (one thread per query row)
//   warps 4-7  : the same for Q tile 1
//   warp  8    : TMA producer (Q per item, K_j / V_j through their rings)
//   warp  9    : TMEM allocation; issues the tcgen05.mma of Q tile 0
//   warp  10   : issues the tcgen05.mma of Q tile 1 (two issuers, so that the barrier waits and
//                commits of one tile hide behind the queued MMAs of the other, and one tile can
//                move on to the next item while the other finishes)
//   warp  11   : idle (it completes the third warpgroup so that setmaxnreg can move its
//                registers to the softmax warpgroups: 72 vs 216 registers per thread; the split
//                must stay below the 64 K register file or setmaxnreg.inc never returns)
// TMEM (512 columns x 128 lanes, f32): per Q tile two 64-column S buffers (S[w][b] at w*128 + b*64),
// O0 [256,256+D), O1 [256+D,256+2D).  K/V are loaded as 128-key tiles but multiplied in 64-key
// steps; P (bf16) overwrites the first 32 columns of its S buffer and feeds the PV MMA from TMEM.
// S = Q K^T is an SS MMA with both operands K-major in 128-byte-swizzled shared memory; O += P V
// is a TS MMA whose B operand (V) is MN-major, i.e. V is used exactly as TMA lands it.
// The normalised O tile is staged in the tile's own (by then idle) Q buffer and leaves through
// TMA stores.  Every mbarrier wait is bounded; on expiry the kernel records a code in the device
// status word, drains its own copies and MMAs, frees TMEM and returns.
#include <cuda.h>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "kernels.h"
#include "tc_ptx.cuh"
#include "tensor_map.h"

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
    static constexpr int NBARS = 2 + 2 + 3 * KS + 3 * VS + 4 + 4 + 2 + 2 + 2 + 2 + 1 + 1;
    // (batch, query block) pairs the length-sorted schedule can hold (two uint16 per pair); what is left of
    // the 227 KB of shared memory at D = 128 bounds it there
    static constexpr int SCHED_CAP = (D == 128) ? 384 : 2048;
    static constexpr int SMEM_BYTES = (2 + KS + VS) * TILE_BYTES + NBARS * 8 + 16 + 4 * SCHED_CAP + 1024;
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can opt into");
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
    int64_t o_stride_b, o_stride_h, o_stride_row;  // element strides of the output (inner dim contiguous)
    int n_qb;          // 256-row blocks per head
    int slots_per_head, n_slots, paired;  // static schedule, see tc_item
    int sorted;        // length-sorted schedule (launches with per-batch kv_lens), see tc_item
    int stagger_clocks;  // single-tile items: head start of tile 0 over tile 1, in SM clocks
    int direct_out;    // one item per CTA: the epilogue stores its rows straight from registers (no staged tile, no TMA store)
    int single_tile;   // items are 128-row blocks whose 64-key steps alternate between the two tiles (small launches, see tc_item)
};


// Timeout codes written to the device status word (100 + site).
enum { kToQ = 101, kToKFull, kToKEmpty, kToVFull, kToVEmpty, kToSFull, kToPFull, kToOFull, kToDone, kToDrain,
       kToQEmpty, kToOFree, kToStage, kToMerge };

// 2^x for a pair of arguments on the FMA and integer pipes (x <= ~100): round to the nearest
// integer n with the 1.5*2^23 trick, a cubic for 2^r on r = x - n in [-0.5, 0.5] (relative error
// 7.5e-5, far below the bf16 rounding of P), and n added into the exponent field.  Arguments
// below -125 (masked scores are -inf) give 2^-125, not 0: invisible next to any visible score,
// and a row without one is recognised by a flag instead of by a zero sum.
// The MUFU pipe (16 ex2 per clock per SM) is the softmax warps' bottleneck; sending a share of
// the exponentials here balances it against the FMA pipe.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
    x.x = fmaxf(x.x, -125.f);
    x.y = fmaxf(x.y, -125.f);
    const float2 magic = make_float2(12582912.f, 12582912.f), nmagic = make_float2(-12582912.f, -12582912.f);
    const float2 t = __fadd2_rn(x, magic);
    const float2 nf = __fadd2_rn(t, nmagic);
    const float2 r = __fadd2_rn(x, make_float2(-nf.x, -nf.y));
    float2 y = __ffma2_rn(r, make_float2(0.0551716685f, 0.0551716685f), make_float2(0.242611125f, 0.242611125f));
    y = __ffma2_rn(y, r, make_float2(0.693260968f, 0.693260968f));
    y = __ffma2_rn(y, r, make_float2(0.999928057f, 0.999928057f));
    y.x = __int_as_float(__float_as_int(y.x) + (__float_as_int(t.x) << 23));
    y.y = __int_as_float(__float_as_int(y.y) + (__float_as_int(t.y) << 23));
    return y;
}
// Which of the 16 element pairs of a 32-column chunk take the polynomial path.
// Which of the 16 element pairs of a 32-column chunk take the polynomial path (a quarter: more
// than that costs more issue slots on the FMA pipe than it frees on the MUFU pipe).
__host__ __device__ constexpr bool poly_pair(int q) { return (q & 3) == 3; }

__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// One work item of a CTA's static list.
struct TcItem {
    int bh, b, h, h_kv, q0, kv_hi, q_off;  // bh = b * heads + h indexes LSE; h_kv is the KV head h reads
    int U0, U1;    // 64-key steps of each Q tile; scalars, so nothing is indexed dynamically
    int n_tiles;   // 128-key K/V tiles to load
    bool end;      // the list is exhausted
    bool valid;    // false: this position of the list holds no item
    __device__ __forceinline__ int steps(int w) const { return w ? U1 : U0; }
    // first query row of tile w: the tiles are stacked (q0, q0 + 128), or both sit on the item's one block
    __device__ __forceinline__ int qrow(int w, bool single) const { return q0 + ((w || single) ? 128 : 0); }
};

// Static schedule.  The (batch, head)-major slot list is dealt round-robin to the CTAs, so the
// CTAs running at one time work on a few neighbouring heads and share their K/V in L2.  In
// paired mode a slot holds the 256-row blocks r and n_qb-1-r of one head, heavy one first: under
// a causal mask every slot then costs the same, and the CTAs finish together.  A launch with fewer
// 256-row blocks than 3/4 of the SMs uses 128-row items instead (single_tile): twice the CTAs, and inside
// a CTA the item's 64-key steps alternate between the two tiles (tile 0 takes the even steps = the first
// half of every 128-key K/V tile, tile 1 the odd ones), each with its own running max, sum and accumulator;
// the epilogue merges the two partial results straight out of TMEM and stores the rows directly (no staged
// tile: such a CTA has no further item).  Both softmax warpgroups and both MMA issuers then work on the one
// block, which nearly halves the critical path of a small problem.
// Sorted mode (per-batch kv_lens, where an item's cost is only known on the device): every CTA ranks the
// (batch, query block) pairs by their step count at start-up (the same deterministic sort in every CTA, so
// no queue, no atomics and no scratch memory are needed), the item list is that order with all heads of a
// pair side by side, and it is dealt to the CTAs boustrophedon (0..G-1, G-1..0, ...), heaviest first: the
// persistent kernel's overlap of one item's set-up with the previous item's tail, and a balanced finish.
template <bool kCausal, bool kSingle>
__device__ __forceinline__ void tc_steps(const TcParams& p, int b, int q0, int& kv_hi, int& q_off, int& U0, int& U1) {
    kv_hi = p.seq_kv;
    if (p.kv_lens) {
        const int l = p.kv_lens[b];
        kv_hi = l < 0 ? 0 : (l < p.seq_kv ? l : p.seq_kv);
    }
    q_off = p.q_offsets ? p.q_offsets[b] : 0;   // query row i sits at key position i + q_off
    const int n_steps = (kv_hi + 63) / 64;      // 64-key steps that hold a visible key
    const int last0 = q0 + 127 + q_off, last1 = last0 + 128;  // last key each tile's last row may see
    U0 = !kCausal ? n_steps : (last0 < 0 ? 0 : min(n_steps, last0 / 64 + 1));
    U1 = !kCausal ? n_steps : (last1 < 0 ? 0 : min(n_steps, last1 / 64 + 1));
    if (kSingle) {  // the block's U1 steps are dealt alternately: even ones to tile 0, odd ones to tile 1
        U0 = (U1 + 1) >> 1;
        U1 = U1 >> 1;
    }
}

template <bool kCausal, bool kSingle>
__device__ __forceinline__ TcItem tc_item(int j, const TcParams& p, const uint16_t* sched) {
    TcItem it;
    it.valid = false;
    int qb;
    if (p.sorted) {
        const int G = (int)gridDim.x;
        it.end = (int64_t)j * G >= (int64_t)p.n_slots;
        if (it.end) return it;
        const int pos = j * G + ((j & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x);
        if (pos >= p.n_slots) return it;
        const int pair = sched[pos / p.heads];
        qb = pair % p.n_qb;
        it.b = pair / p.n_qb;
        it.h = pos % p.heads;
        it.bh = it.b * p.heads + it.h;
    } else {
        const int slot = (int)blockIdx.x + (p.paired ? (j >> 1) : j) * (int)gridDim.x;
        it.end = slot >= p.n_slots;
        if (it.end) return it;
        it.bh = slot / p.slots_per_head;
        const int r = slot % p.slots_per_head;
        qb = p.n_qb - 1 - r;
        if (p.paired && (j & 1)) {
            if (r == qb) return it;  // the middle block of an odd count has no partner
            qb = r;
        }
        it.b = it.bh / p.heads;
        it.h = it.bh % p.heads;
    }
    it.valid = true;
    it.h_kv = it.h / (p.heads / p.heads_kv);
    // Single-tile items: block qb covers rows [128 qb, 128 qb + 128); the item's origin is kept 128 rows
    // earlier so that the block sits where tile 1 sits in a two-tile item (TcItem::qrow).
    it.q0 = kSingle ? qb * 128 - 128 : qb * 256;
    tc_steps<kCausal, kSingle>(p, it.b, it.q0, it.kv_hi, it.q_off, it.U0, it.U1);
    it.n_tiles = kSingle ? it.U0 : (it.U1 + 1) / 2;
    return it;
}

// Pipeline, per Q tile w and 64-key step u (buffer b = u & 1):
//   MMA:     S_w(u) -> TMEM S[w][b]            (SS, N = 64, D/16 k-steps)       commit s_full[w][b]
//   softmax: S[w][b] -> registers -> P (bf16) over the first 32 columns of S[w][b]   arrive p_full[w][b]
//   MMA:     O_w += P V(u)                      (TS, N = D, 4 k-steps)           commit o_full[w]
//            then S_w(u+2) into the same buffer (in-order after the PV that read P from it)
// S is double-buffered, so the softmax of step u+1 never waits for the PV of step u.
// Per item and tile: q_full (Q landed) -> ... -> o_done (last PV retired) -> epilogue reads O
// (o_free: the next item's first PV may overwrite it), stages it in the Q buffer (stage_full),
// one thread stores it (q_empty: the next item's Q may land).  A tile that sees no key in an
// item takes no part in these (its rows are written as NaN directly).
template <int D, bool kCausal, bool kKeep, bool kSingle>
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
    uint64_t* q_empty = q_full + 2;       // [2]  the O tile staged in the Q buffer has been read out
    uint64_t* k_full = q_empty + 2;       // [KS]
    uint64_t* k_empty = k_full + KS;      // [2 tiles][KS]: the issuer of tile w is done with the slot
    uint64_t* v_full = k_empty + 2 * KS;  // [VS]
    uint64_t* v_empty = v_full + VS;      // [2 tiles][VS]
    uint64_t* s_full = v_empty + 2 * VS;  // [2 tiles][2 buffers]
    uint64_t* p_full = s_full + 4;        // [2 tiles][2 buffers]
    uint64_t* o_full = p_full + 4;        // [2]  one phase per PV step (O at rest for a rescale)
    uint64_t* o_done = o_full + 2;        // [2]  one phase per item: the last PV of the tile has retired
    uint64_t* o_free = o_done + 2;        // [2]  one phase per item: the epilogue has read O out of TMEM
    uint64_t* stage_full = o_free + 2;    // [2]  one phase per item: the O tile is staged in shared memory
    uint64_t* done_bar = stage_full + 2;  // [1]
    uint64_t* merge_bar = done_bar + 1;   // [1]  single-tile items: both tiles have published their (max, sum)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(merge_bar + 1);
    uint16_t* sched = reinterpret_cast<uint16_t*>(tmem_slot + 4);  // [SCHED_CAP] pair order, then [SCHED_CAP] step counts

    // Broadcasting the warp index makes it provably warp-uniform, so role dispatch and the MMA
    // operands stay on the uniform datapath.
    const int warp = __shfl_sync(kFullMask, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int N = p.seq;
    const int Nkv = p.seq_kv;

    // ------------------------------------------------------------------ setup
    // Launched with programmatic stream serialization, the CTA may start while the previous kernel of
    // the stream is still running: barrier set-up and the TMEM allocation then overlap that kernel's tail.
    // grid_dep_wait returns once the previous kernel has completed and its writes are visible (at once under
    // a normal launch); every global access of this kernel comes after one.
    if (p.sorted) {
        grid_dep_wait();  // kv_lens may be the previous kernel's output
        // Rank sort of the (batch, query block) pairs by their step count, descending, ties by index:
        // every CTA computes the same table.
        uint16_t* cost = sched + C::SCHED_CAP;
        const int n_pairs = p.n_slots / p.heads;
        for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
            int kv_hi, q_off, U0, U1;
            tc_steps<kCausal, kSingle>(p, i / p.n_qb, (i % p.n_qb) * 256, kv_hi, q_off, U0, U1);
            cost[i] = (uint16_t)min(U0 + U1, 65535);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
            const int ci = cost[i];
            int rank = 0;
            for (int k2 = 0; k2 < n_pairs; ++k2) {
                const int ck = cost[k2];
                rank += (ck > ci || (ck == ci && k2 < i)) ? 1 : 0;
            }
            sched[rank] = (uint16_t)i;
        }
        __syncthreads();
    }
    bool first_preloaded = false;  // meaningful in the producer thread only
    if (warp == 8) {
        // The barriers are initialised by the 32 lanes side by side (one thread doing all of them costs
        // ~0.4 us at the head of every CTA's critical path); all counts are 1 except the ones named here.
        for (int i = lane; i < C::NBARS; i += 32) {
            uint64_t* bar = bars + i;
            uint32_t count = 1;
            if (bar >= p_full && bar < p_full + 4) count = 128;
            else if (bar >= o_free && bar < o_free + 2) count = 128;
            else if (bar >= stage_full && bar < stage_full + 2) count = 128;
            else if (bar == done_bar) count = 2;
            else if (bar == merge_bar) count = 256;
            mbar_init(bar, count);
        }
        fence_barrier_init();
        __syncwarp();
    }
    if (warp == 8 && lane == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_o);
        fence_barrier_init();
        fence_proxy_async();
        grid_dep_wait();
        // Q and the first K tile of the first item are requested right away, so their latency
        // overlaps the TMEM allocation and the CTA-wide barrier below.
        const TcItem it = tc_item<kCausal, kSingle>(0, p, sched);
        if (!it.end && it.valid && it.n_tiles > 0) {
            first_preloaded = true;
            if constexpr (kSingle) {
                // one Q tile serves both issuers (buffer 1, which also stages the output); K tile 0 follows
                mbar_arrive_expect_tx(&q_full[1], TILE);
#pragma unroll
                for (int s = 0; s < C::NSUB; ++s)
                    tma_load_4d(sQ + TILE + s * SUB, &tm_q, &q_full[1], s * 64, it.qrow(1, true), it.h, it.b);
                mbar_arrive_expect_tx(&k_full[0], TILE);
#pragma unroll
                for (int s = 0; s < C::NSUB; ++s)
                    tma_load_4d(sK + s * SUB, &tm_k, &k_full[0], s * 64, 0, it.h_kv, it.b);
            }
            for (int w = 0; w < 2 && !kSingle; ++w) {
                if (it.steps(w) == 0) continue;
                mbar_arrive_expect_tx(&q_full[w], TILE);
#pragma unroll
                for (int s = 0; s < C::NSUB; ++s)
                    tma_load_4d(sQ + w * TILE + s * SUB, &tm_q, &q_full[w], s * 64, it.qrow(w, kSingle), it.h, it.b);
                if (w == 0 || it.U0 == 0) {
                    mbar_arrive_expect_tx(&k_full[0], TILE);
#pragma unroll
                    for (int s = 0; s < C::NSUB; ++s)
                        tma_load_4d(sK + s * SUB, &tm_k, &k_full[0], s * 64, 0, it.h_kv, it.b);
                }
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
    grid_dep_wait();
    // The next kernel of the stream may be scheduled as SMs fall free (it waits as above before it reads or
    // writes anything): its launch latency and set-up hide behind the tail of this grid.
    grid_dep_launch();

    // The register hand-over sits inside each role's own branch: the compiler budgets the code
    // that follows a setmaxnreg only when no path with a different budget merges into it.
    if (warp >= 8) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
      if (warp == 8) {
        // ============================================================== TMA producer
        if (lane == 0 && kSingle) {
            // A single-tile item is its CTA's only item; Q and K tile 0 were requested during setup.  Each
            // issuer reads every tile once and asks for K tile u + 2 right after the PV of step u, so K runs
            // two tiles ahead of V in the request order: K1 | K2 V0 | K3 V1 | ...
            const TcItem it = tc_item<kCausal, kSingle>(0, p, sched);
            if (first_preloaded) {
                bool ok = true;
                int kg = 1, vg = 0;
                auto load_k = [&](int t) {
                    const int ks = t % KS;
                    const uint32_t par = ((uint32_t)(t / KS) & 1u) ^ 1u;
                    if (!mbar_wait(&k_empty[ks], par, p.status, kToKEmpty) ||
                        !mbar_wait(&k_empty[KS + ks], par, p.status, kToKEmpty))
                        return false;
                    mbar_arrive_expect_tx(&k_full[ks], TILE);
#pragma unroll
                    for (int s = 0; s < C::NSUB; ++s)
                        tma_load_4d(sK + ks * TILE + s * SUB, &tm_k, &k_full[ks], s * 64, t * 128, it.h_kv, it.b);
                    ++kg;
                    return true;
                };
                if (it.n_tiles > 1) ok = load_k(1);
                for (int t = 0; t < it.n_tiles && ok; ++t) {
                    if (t + 2 < it.n_tiles && !load_k(t + 2)) break;
                    const int vs = t % VS;
                    const uint32_t par = ((uint32_t)(t / VS) & 1u) ^ 1u;
                    if (!mbar_wait(&v_empty[vs], par, p.status, kToVEmpty) ||
                        !mbar_wait(&v_empty[VS + vs], par, p.status, kToVEmpty))
                        break;
                    mbar_arrive_expect_tx(&v_full[vs], TILE);
#pragma unroll
                    for (int s = 0; s < C::NSUB; ++s)
                        tma_load_4d(sV + vs * TILE + s * SUB, &tm_v, &v_full[vs], s * 64, t * 128, it.h_kv, it.b);
                    ++vg;
                }
                // Drain: every copy this thread issued must have landed before the CTA may exit.
                mbar_wait(&q_full[1], 0u, p.status, kToDrain);
                for (int t = max(0, kg - KS); t < kg; ++t)
                    mbar_wait(&k_full[t % KS], (uint32_t)(t / KS) & 1u, p.status, kToDrain);
                for (int t = max(0, vg - VS); t < vg; ++t)
                    mbar_wait(&v_full[t % VS], (uint32_t)(t / VS) & 1u, p.status, kToDrain);
            }
        } else if (lane == 0) {
            int kg = 0, vg = 0;    // K / V tiles requested so far (ring position and phase)
            int na0 = 0, na1 = 0;  // items so far in which tile w took part (phase of its per-item barriers)
            bool ok = true;
            for (int j = 0; ok; ++j) {
                const TcItem it = tc_item<kCausal, kSingle>(j, p, sched);
                if (it.end) break;
                if (!it.valid || it.n_tiles == 0) continue;  // nothing to load
                auto load_q = [&](int w, int na) {
                    // the previous item's O tile must have left the buffer
                    if (!mbar_wait(&q_empty[w], ((uint32_t)na & 1u) ^ 1u, p.status, kToQEmpty)) return false;
                    mbar_arrive_expect_tx(&q_full[w], TILE);
#pragma unroll
                    for (int s = 0; s < C::NSUB; ++s)
                        tma_load_4d(sQ + w * TILE + s * SUB, &tm_q, &q_full[w], s * 64, it.qrow(w, kSingle), it.h, it.b);
                    return true;
                };
                const bool pre = first_preloaded && j == 0;  // Q and K tile 0 were requested during setup
                if (it.U0 > 0) {
                    if (!pre && !load_q(0, na0)) break;
                    ++na0;
                }
                for (int t = 0; t < it.n_tiles && ok; ++t) {
                    // A slot is free once both issuers have released the tile it held.
                    const int ks = kg % KS, vs = vg % VS;
                    const uint32_t kpar = ((uint32_t)(kg / KS) & 1u) ^ 1u, vpar = ((uint32_t)(vg / VS) & 1u) ^ 1u;
                    if (!(pre && t == 0)) {
                        if (!mbar_wait(&k_empty[ks], kpar, p.status, kToKEmpty) ||
                            !mbar_wait(&k_empty[KS + ks], kpar, p.status, kToKEmpty)) {
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(&k_full[ks], TILE);
#pragma unroll
                        for (int s = 0; s < C::NSUB; ++s)
                            tma_load_4d(sK + ks * TILE + s * SUB, &tm_k, &k_full[ks], s * 64, t * 128, it.h_kv, it.b);
                    }
                    ++kg;
                    if (t == 0 && it.U1 > 0) {  // tile 1 usually still works on the previous item: its Q comes second
                        if (!pre && !load_q(1, na1)) {
                            ok = false;
                            break;
                        }
                        ++na1;
                    }
                    if (!mbar_wait(&v_empty[vs], vpar, p.status, kToVEmpty) ||
                        !mbar_wait(&v_empty[VS + vs], vpar, p.status, kToVEmpty)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&v_full[vs], TILE);
#pragma unroll
                    for (int s = 0; s < C::NSUB; ++s)
                        tma_load_4d(sV + vs * TILE + s * SUB, &tm_v, &v_full[vs], s * 64, t * 128, it.h_kv, it.b);
                    ++vg;
                }
            }
            // Drain: every copy this thread issued must have landed before the CTA may exit.
            if (na0 > 0) mbar_wait(&q_full[0], (uint32_t)(na0 - 1) & 1u, p.status, kToDrain);
            if (na1 > 0) mbar_wait(&q_full[1], (uint32_t)(na1 - 1) & 1u, p.status, kToDrain);
            for (int t = max(0, kg - KS); t < kg; ++t)
                mbar_wait(&k_full[t % KS], (uint32_t)(t / KS) & 1u, p.status, kToDrain);
            for (int t = max(0, vg - VS); t < vg; ++t)
                mbar_wait(&v_full[t % VS], (uint32_t)(t / VS) & 1u, p.status, kToDrain);
        }
      } else if (warp == 9 || warp == 10) {
        // ============================================================== MMA issuer of Q tile w
        // The whole warp runs this loop with uniform control flow and only the elected lane
        // executes the tcgen05 instructions: descriptors, addresses and loop state then live in
        // uniform registers, which is what the MMA instruction takes its operands from.
        {
            const int w = warp - 9;
            const bool leader = elect_one();
            constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);
            constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
            // Descriptors are built once; each MMA only adds an offset (in 16-byte units) to the
            // start-address field, so the issuing thread keeps ahead of the tensor pipe.
            const uint64_t dq = make_smem_desc_sw128(smem_u32(sQ + (kSingle ? 1 : w) * TILE), 16, 1024);
            const uint64_t dk = make_smem_desc_sw128(smem_u32(sK), 16, 1024);
            const uint64_t dv = make_smem_desc_sw128(smem_u32(sV), SUB, 1024);
            const uint32_t tS = tmem_base + C::COL_S + w * 128, tO = tmem_base + C::COL_O + w * D;
            uint64_t* const ke = k_empty + w * KS;
            uint64_t* const ve = v_empty + w * VS;
            int kg = 0, vg = 0;    // ring index of the item's first K / V tile
            int na = 0;            // items so far in which this tile took part
            int cp0 = 0, cp1 = 0;  // p_full phases of each S buffer consumed before the item
            auto commit = [&](uint64_t* bar) {
                if (leader) mma_commit(bar);
            };
            auto wait = [&](uint64_t* bar, uint32_t parity, int code) {
                return __all_sync(kFullMask, mbar_wait(bar, parity, p.status, code));
            };
            bool ok = true;
            for (int j = 0; ok; ++j) {
                const TcItem it = tc_item<kCausal, kSingle>(j, p, sched);
                if (it.end) break;
                if (!it.valid || it.n_tiles == 0) continue;
                const int n_u = it.steps(w);
                // Step u of this tile reads half half_of(u) (64 rows) of the item's K/V tile tile_of(u): the
                // tile's own steps are consecutive 64-key steps, or (single-tile items) every second one.
                constexpr bool il = kSingle;
                auto tile_of = [&](int u) { return il ? u : (u >> 1); };
                auto half_of = [&](int u) { return il ? w : (u & 1); };
                auto issue_S = [&](int u) {
                    const uint64_t bk = dk + (uint64_t)((((kg + tile_of(u)) % KS) * TILE + half_of(u) * HALF) >> 4);
                    const uint32_t d = tS + (u & 1) * 64;
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t off = (uint32_t)(((kk / 4) * SUB + (kk % 4) * 32) >> 4);
                        if (leader) mma_ss(d, dq + off, bk + off, idesc_s, kk > 0);
                    }
                };
                // O_w += P V(u): P (bf16) sits in the first 32 columns of S[w][u&1]
                auto issue_PV = [&](int u) {
                    const uint64_t bv = dv + (uint64_t)((((vg + tile_of(u)) % VS) * TILE + half_of(u) * HALF) >> 4);
                    const uint32_t a = tS + (u & 1) * 64;
                    const uint32_t acc0 = u > 0 ? 1u : 0u;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        if (leader)
                            mma_ts(tO, a + kk * 8, bv + (uint64_t)((kk * 2048) >> 4), idesc_o, kk > 0 ? 1u : acc0);
                };
                auto last_use = [&](int u) { return il || (u & 1) || u == n_u - 1; };  // of a 128-key tile, by this Q tile

                if (n_u > 0) {
                    ok = wait(&k_full[kg % KS], (uint32_t)(kg / KS) & 1u, kToKFull) &&
                         wait(&q_full[il ? 1 : w], (uint32_t)na & 1u, kToQ);
                    if (!ok) break;
                    tc_fence_after();
                    issue_S(0);
                    commit(&s_full[w * 2]);
                    int k_waited = 0, v_waited = -1;  // item-local tile indices already waited for
                    if (il) commit(&ke[kg % KS]);
                    if (n_u > 1) {
                        if (il) {  // the second step reads the next K tile
                            if (!wait(&k_full[(kg + 1) % KS], (uint32_t)((kg + 1) / KS) & 1u, kToKFull)) { ok = false; break; }
                            k_waited = 1;
                            tc_fence_after();
                        }
                        issue_S(1);
                        commit(&s_full[w * 2 + 1]);
                        if (il) commit(&ke[(kg + 1) % KS]);
                    }
                    if (!il) commit(&ke[kg % KS]);
                    for (int u = 0; u < n_u && ok; ++u) {
                        const int vt = tile_of(u);
                        if (vt > v_waited) {
                            if (!wait(&v_full[(vg + vt) % VS], (uint32_t)((vg + vt) / VS) & 1u, kToVFull)) { ok = false; break; }
                            v_waited = vt;
                        }
                        if (!wait(&p_full[w * 2 + (u & 1)], (uint32_t)(((u & 1) ? cp1 : cp0) + (u >> 1)) & 1u, kToPFull)) { ok = false; break; }
                        // the previous item's epilogue must have read O_w before it is overwritten
                        if (u == 0 && na > 0 && !wait(&o_free[w], (uint32_t)(na - 1) & 1u, kToOFree)) { ok = false; break; }
                        tc_fence_after();
                        issue_PV(u);
                        commit(&o_full[w]);
                        if (u == n_u - 1) commit(&o_done[w]);
                        if (last_use(u)) commit(&ve[(vg + vt) % VS]);
                        if (u + 2 < n_u) {
                            const int kt = tile_of(u + 2);
                            if (kt > k_waited) {
                                if (!wait(&k_full[(kg + kt) % KS], (uint32_t)((kg + kt) / KS) & 1u, kToKFull)) { ok = false; break; }
                                k_waited = kt;
                                tc_fence_after();
                            }
                            issue_S(u + 2);
                            commit(&s_full[w * 2 + (u & 1)]);
                            if (last_use(u + 2)) commit(&ke[(kg + kt) % KS]);
                        }
                    }
                    ++na;
                    cp0 += (n_u + 1) / 2;
                    cp1 += n_u / 2;
                }
                // Tiles this Q tile does not read (it sees fewer keys than the other one) are passed on
                // once they have landed, which keeps this issuer inside the ring window.
                for (int t = il ? n_u : (n_u + 1) / 2; t < it.n_tiles && ok; ++t) {
                    ok = wait(&k_full[(kg + t) % KS], (uint32_t)((kg + t) / KS) & 1u, kToKFull);
                    if (ok) commit(&ke[(kg + t) % KS]);
                    ok = ok && wait(&v_full[(vg + t) % VS], (uint32_t)((vg + t) / VS) & 1u, kToVFull);
                    if (ok) commit(&ve[(vg + t) % VS]);
                }
                kg += it.n_tiles;
                vg += it.n_tiles;
            }
            // All MMAs of both issuers must retire before TMEM is freed.
            commit(done_bar);
            wait(done_bar, 0, kToDone);
        }
      }  // warp 11 idle: it only completes the warpgroup for setmaxnreg
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        // ============================================================== softmax / epilogue warps
        const int w = warp >> 2;                       // Q tile
        const int row_in_tile = (warp & 3) * 32 + lane;
        const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tS = tmem_base + lane_sel + C::COL_S + w * 128;
        const uint32_t tO = tmem_base + lane_sel + C::COL_O + w * D;
        const float c = p.scale_log2;
        int na = 0;            // items so far in which this tile took part
        int cs0 = 0, cs1 = 0;  // s_full phases of each S buffer consumed before the item
        int co = 0;            // PV steps of this tile before the item (phase of o_full)
        bool ok = true;

        for (int j = 0; ok; ++j) {
            const TcItem it = tc_item<kCausal, kSingle>(j, p, sched);
            if (it.end) break;
            if (!it.valid) continue;
            const int n_iter = it.steps(w);
            constexpr bool il = kSingle;  // this tile's steps are every second 64-key step of the block
            const int bh = it.bh, kv_hi = it.kv_hi, q_off = it.q_off;
            const int row = it.qrow(w, il) + row_in_tile;  // query index within the sequence
            const uint8_t* keep = kKeep ? p.key_keep + (int64_t)it.b * p.keep_batch_stride : nullptr;

            // The tile sees no key: NaN rows, LSE = -inf (cpu_forward.rs:411-420).  A single-tile item whose
            // other tile has a step still goes through the merge below with an empty partial result.
            if (n_iter == 0 && !(il && it.n_tiles > 0)) {
                if (row < N && !(il && w == 0)) {
                    uint4* dst = reinterpret_cast<uint4*>(p.out + it.b * p.o_stride_b + it.h * p.o_stride_h +
                                                          (int64_t)row * p.o_stride_row);
#pragma unroll
                    for (int i = 0; i < D / 8; ++i) dst[i] = make_uint4(0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u);
                    if (p.lse) p.lse[(int64_t)bh * N + row] = -INFINITY;
                }
                continue;
            }

            float m_ref = -INFINITY;  // reference max (raw score units) the running sums are relative to
            float l = 0.f;
            bool seen = false;  // the row has met a score that no mask hides
            for (int u = 0; u < n_iter; ++u) {
                const int buf = u & 1;
                if (!__all_sync(kFullMask, mbar_wait(&s_full[w * 2 + buf], (uint32_t)((buf ? cs1 : cs0) + (u >> 1)) & 1u,
                                                     p.status, kToSFull))) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (il && w == 1 && u == 0 && p.stagger_clocks > 0) {
                    // The two tiles of a single-tile item start together and would stay in step: both
                    // warps of a scheduler would then wait for TMEM at the same moments.  Half a step of
                    // offset lets one tile's loads and stores hide behind the other's arithmetic
                    // (measured: 0.5-1 us of 21 on B=1 H=8 N=2048 D=64; RT_ATTN_PREFILL_STAGGER sets the clocks).
                    const long long t0 = clock64();
                    while (clock64() - t0 < p.stagger_clocks) {}
                }

                uint32_t s[64];
                {
                    uint32_t(&s0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[0]);
                    uint32_t(&s1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[32]);
                    tmem_ld32(tS + buf * 64, s0);
                    tmem_ld32(tS + buf * 64 + 32, s1);
                    tc_wait_ld();
                }

                // ---- masks: keys beyond kv_hi, causal diagonal, keep flags
                const int col0 = (il ? 2 * u + w : u) * 64;
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
                seen = seen || (mx > -INFINITY);

                // ---- lazy rescale: move the reference max only when it would grow by > 2^8
                if (u == 0) {
                    m_ref = mx;
                } else {
                    const bool need = (mx > m_ref) && ((mx - m_ref) * c > 8.0f || m_ref == -INFINITY);
                    if (__any_sync(kFullMask, need)) {
                        // O must be at rest: the PV of the previous step has to be complete.  (The score
                        // MMA just waited for was issued after the PV before that one, so the barrier is
                        // at most one phase behind and the parity wait is unambiguous.)
                        if (!__all_sync(kFullMask, mbar_wait(&o_full[w], (uint32_t)(co + u - 1) & 1u, p.status, kToOFull))) {
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
                            make_float2(__uint_as_float(s[ch * 32 + 2 * i]), __uint_as_float(s[ch * 32 + 2 * i + 1])), c2,
                            nmc2);
                        const float2 xb = __ffma2_rn(
                            make_float2(__uint_as_float(s[ch * 32 + 2 * i + 2]), __uint_as_float(s[ch * 32 + 2 * i + 3])),
                            c2, nmc2);
                        // a quarter of the exponentials go to the polynomial (see exp2_poly2)
                        const float2 pa = poly_pair(i) ? exp2_poly2(xa) : make_float2(fast_exp2(xa.x), fast_exp2(xa.y));
                        const float2 pb = poly_pair(i + 1) ? exp2_poly2(xb) : make_float2(fast_exp2(xb.x), fast_exp2(xb.y));
                        sum_a = __fadd2_rn(sum_a, pa);
                        sum_b = __fadd2_rn(sum_b, pb);
                        pk[i] = float2_to_bf16x2(pa.x, pa.y);
                        pk[i + 1] = float2_to_bf16x2(pb.x, pb.y);
                    }
                    tmem_st16(tS + buf * 64 + ch * 16, pk);
                }
                l += (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
                tc_wait_st();  // warp-wide: every lane's part of the store has completed
                tc_fence_before();
                mbar_arrive(&p_full[w * 2 + buf]);
            }
            if (!ok) break;

            // ---- epilogue: O / l -> bf16 into the (now idle) shared-memory tile of Q_w in the swizzled
            // layout of the output tensor map, then one TMA store per 64-column half: 16-byte shared
            // stores instead of row-strided global stores, and rows past N are clipped by the hardware.
            if (n_iter > 0 && !__all_sync(kFullMask, mbar_wait(&o_done[w], (uint32_t)na & 1u, p.status, kToOFull))) {
                ok = false;
                break;
            }
            tc_fence_after();
            if (il) {
                // ---- single-tile item: the two tiles hold partial results of the same 128 rows (even and odd
                // 64-key steps).  Each thread publishes its (max, sum, seen) in the first columns of its tile's
                // idle score buffer, TMEM being readable by the other warpgroup's warp of the same lane
                // quarter; after the barrier every thread knows both partials of its row.  The merged row is
                //   O = (f0 O_0 + f1 O_1) / (f0 l_0 + f1 l_1),  f_w = 2^((m_w - max(m_0, m_1)) c),
                // and warpgroup w produces columns [w D/2, (w+1) D/2) of it from both accumulators.
                {
                    uint32_t ex[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) ex[i] = 0u;
                    ex[0] = __float_as_uint(m_ref);
                    ex[1] = __float_as_uint(l);
                    ex[2] = seen ? 1u : 0u;
                    tmem_st16(tS, ex);
                    tc_wait_st();
                    tc_fence_before();
                    mbar_arrive(merge_bar);
                }
                if (!__all_sync(kFullMask, mbar_wait(merge_bar, (uint32_t)na & 1u, p.status, kToMerge))) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t tS_other = tmem_base + lane_sel + C::COL_S + (1 - w) * 128;
                const uint32_t tO_other = tmem_base + lane_sel + C::COL_O + (1 - w) * D;
                uint32_t exo[16];
                tmem_ld16(tS_other, exo);
                tc_wait_ld();
                const float m_o = __uint_as_float(exo[0]), l_o = __uint_as_float(exo[1]);
                const bool seen_any = seen || (exo[2] != 0u);
                const float m_all = fmaxf(m_ref, m_o);
                const float f_own = (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - m_all) * c);
                const float f_oth = (m_o == -INFINITY) ? 0.f : fast_exp2((m_o - m_all) * c);
                const float l_all = f_own * l + f_oth * l_o;
                const bool valid = seen_any && (l_all > 0.f);
                const float inv = valid ? 1.f / l_all : 0.f;
                const float a_own = f_own * inv, a_oth = f_oth * inv;
                const bool has_own = n_iter > 0, has_oth = it.steps(1 - w) > 0;  // an idle tile's accumulator was never written
                // The merged half rows go straight to global memory (64 or 128 contiguous bytes per thread): the CTA
                // has no further item, and a staged tile, its barrier and a TMA store would only lengthen the
                // tail of a launch whose time is its longest CTA.
                __nv_bfloat16* dst = p.out + it.b * p.o_stride_b + it.h * p.o_stride_h + (int64_t)row * p.o_stride_row;
#pragma unroll
                for (int cq = 0; cq < D / 64; ++cq) {
                    const int ch = w * (D / 64) + cq;
                    uint32_t oa[32], ob[32];
                    if (has_own) tmem_ld32(tO + ch * 32, oa);
                    if (has_oth) tmem_ld32(tO_other + ch * 32, ob);
                    tc_wait_ld();
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4) {
                        uint4 pack;
                        uint32_t* pw = reinterpret_cast<uint32_t*>(&pack);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int e = v4 * 8 + 2 * i;
                            const float x0 = (has_own ? __uint_as_float(oa[e]) * a_own : 0.f) +
                                             (has_oth ? __uint_as_float(ob[e]) * a_oth : 0.f);
                            const float x1 = (has_own ? __uint_as_float(oa[e + 1]) * a_own : 0.f) +
                                             (has_oth ? __uint_as_float(ob[e + 1]) * a_oth : 0.f);
                            pw[i] = valid ? float2_to_bf16x2(x0, x1) : 0x7fc07fc0u;
                        }
                        if (row < N) *reinterpret_cast<uint4*>(dst + ch * 32 + v4 * 8) = pack;
                    }
                }
                if (w == 1 && p.lse && row < N)
                    p.lse[(int64_t)bh * N + row] =
                        valid ? (m_all * c + fast_log2(l_all)) * kLn2 : (seen_any ? NAN : -INFINITY);
            } else {
                // A masked score costs the polynomial path 2^-125 instead of 0, so a row counts as
                // empty when it never saw a visible score, not when its sum is exactly 0.
                const bool valid = seen && (l > 0.f);
                const float inv = valid ? 1.f / l : 0.f;
                uint8_t* stage = sQ + w * TILE + row_in_tile * 128;  // every score MMA that read Q_w has retired
                __nv_bfloat16* dst = p.out + it.b * p.o_stride_b + it.h * p.o_stride_h + (int64_t)row * p.o_stride_row;
#pragma unroll
                for (int ch = 0; ch < D / 32; ++ch) {
                    uint32_t o[32];
                    tmem_ld32(tO + ch * 32, o);
                    tc_wait_ld();
                    if (ch == D / 32 - 1) {  // O_w is in registers: the next item's first PV may overwrite it
                        tc_fence_before();
                        mbar_arrive(&o_free[w]);
                    }
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
                        if (p.direct_out) {  // the CTA's only item: no overlap to win, the staged store would just add to the tail
                            if (row < N) *reinterpret_cast<uint4*>(dst + cc * 8) = pack;
                        } else {
                            *reinterpret_cast<uint4*>(stage + (cc / 8) * SUB + (((cc % 8) ^ (row_in_tile & 7)) << 4)) = pack;
                        }
                    }
                }
                if (p.lse && row < N)
                    p.lse[(int64_t)bh * N + row] =
                        valid ? (m_ref * c + fast_log2(l)) * kLn2 : (seen ? NAN : -INFINITY);
                if (!p.direct_out) {
                    fence_proxy_async();  // generic-proxy writes above -> visible to the TMA (async proxy) read
                    mbar_arrive(&stage_full[w]);
                }
            }
            if (row_in_tile == 0 && !il && !p.direct_out) {
                if (!mbar_wait(&stage_full[w], (uint32_t)na & 1u, p.status, kToStage)) {
                    ok = false;
                } else {
#pragma unroll
                    for (int s = 0; s < C::NSUB; ++s)
                        tma_store_4d(&tm_o, sQ + w * TILE + s * SUB, s * 64, it.qrow(w, il), it.h, it.b);
                    tma_store_commit_and_wait_read();  // the staged tile has been read: the next Q may land
                    mbar_arrive(&q_empty[w]);
                }
            }
            ok = __all_sync(kFullMask, ok);
            ++na;
            cs0 += (n_iter + 1) / 2;
            cs1 += n_iter / 2;
            co += n_iter;
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

bool encode_bf16_map_cached(CUtensorMap* out, int rank, const void* base, const uint64_t* dims,
                            const uint64_t* strides_bytes, const uint32_t* box) {
    struct Key {
        const void* base;
        uint64_t dims[4], strides[3];
        uint32_t box[4];
        int rank;
    };
    constexpr int kEntries = 32;
    struct Cache {
        Key key[kEntries];
        CUtensorMap map[kEntries];
        int used = 0, next = 0;
    };
    thread_local Cache cache;
    if (rank < 1 || rank > 4) return false;
    Key k;
    memset(&k, 0, sizeof(k));
    k.base = base;
    k.rank = rank;
    for (int i = 0; i < rank; ++i) {
        k.dims[i] = dims[i];
        k.box[i] = box[i];
        if (i + 1 < rank) k.strides[i] = strides_bytes[i];
    }
    for (int i = 0; i < cache.used; ++i)
        if (memcmp(&cache.key[i], &k, sizeof(Key)) == 0) {
            *out = cache.map[i];
            return true;
        }
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return false;
    cuuint64_t d[4], st[3];
    cuuint32_t bx[4], estr[4] = {1, 1, 1, 1};
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        bx[i] = box[i];
        if (i + 1 < rank) st[i] = strides_bytes[i];
    }
    if (enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), d, st, bx, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    const int slot = cache.used < kEntries ? cache.used++ : (cache.next = (cache.next + 1) % kEntries);
    cache.key[slot] = k;
    cache.map[slot] = *out;
    return true;
}

bool make_tensor_map_bf16_4d(CUtensorMap* map, const void* base, int64_t batch, int64_t heads, int64_t seq, int dim,
                             int64_t stride_b, int64_t stride_h, int64_t stride_row, int box_rows = 128);

// View of a [B, H, N, D] bf16 tensor with arbitrary batch / head / row strides (inner dim contiguous)
// as a 4-D TMA tensor (d, row, head, batch); box = 64 columns x box_rows (128, or 64) rows of one (b,h), 128-byte
// swizzle.  Rows past N are zero-filled on loads and clipped on stores, so tiles never touch a
// neighbouring head.  Strides are in elements and must be multiples of 8 (16 bytes).
bool make_tensor_map_bf16_4d(CUtensorMap* map, const void* base, int64_t batch, int64_t heads, int64_t seq, int dim,
                             int64_t stride_b, int64_t stride_h, int64_t stride_row, int box_rows) {
    const uint64_t dims[4] = {(uint64_t)dim, (uint64_t)seq, (uint64_t)heads, (uint64_t)batch};
    const uint64_t strides[3] = {(uint64_t)stride_row * 2, (uint64_t)stride_h * 2, (uint64_t)stride_b * 2};
    const uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
    return encode_bf16_map_cached(map, 4, base, dims, strides, box);
}

// The contiguous [B*H, N, D] view used by the self-test kernel.
bool make_tensor_map_bf16_3d(CUtensorMap* map, const void* base, int64_t bh, int64_t seq, int dim) {
    const uint64_t dims[3] = {(uint64_t)dim, (uint64_t)seq, (uint64_t)bh};
    const uint64_t strides[2] = {(uint64_t)dim * 2, (uint64_t)seq * dim * 2};
    const uint32_t box[3] = {64, 128, 1};
    return encode_bf16_map_cached(map, 3, base, dims, strides, box);
}

template <int D, bool kCausal, bool kKeep, bool kSingle>
static cudaError_t launch_tc_s(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                             const TcParams& p, int64_t n_ctas, cudaStream_t stream) {
    auto kern = prefill_tc_kernel<D, kCausal, kKeep, kSingle>;
    cudaError_t e = set_max_dynamic_smem_once<prefill_tc_kernel<D, kCausal, kKeep, kSingle>>(TcCfg<D>::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    // RT_ATTN_PREFILL_PDL=0|1 forces programmatic stream serialization off or on.
    static const int env_pdl = [] {
        const char* s = getenv("RT_ATTN_PREFILL_PDL");
        return s ? (s[0] == '0' ? 0 : 1) : -1;
    }();
    // Measured: the overlap pays for short single-tile launches (up to 1 us of 9-16 us); for long ones the
    // dependency wait costs as much as the launch gap it hides.
    const bool pdl = env_pdl >= 0 ? env_pdl == 1 : (kSingle && p.seq_kv <= 1024);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)n_ctas);
    cfg.blockDim = dim3(384);
    cfg.dynamicSmemBytes = TcCfg<D>::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, mo, p);
}

template <int D, bool kCausal, bool kKeep>
static cudaError_t launch_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                             const TcParams& p, int64_t n_ctas, cudaStream_t stream) {
    return p.single_tile ? launch_tc_s<D, kCausal, kKeep, true>(mq, mk, mv, mo, p, n_ctas, stream)
                         : launch_tc_s<D, kCausal, kKeep, false>(mq, mk, mv, mo, p, n_ctas, stream);
}

cudaError_t launch_prefill_tc(const void* q, const void* k, const void* v, void* out, float* lse, int64_t batch,
                              int64_t heads, int64_t heads_kv, int64_t seq, int64_t seq_kv, int dim,
                              const TensorStrides& sq, const TensorStrides& sk, const TensorStrides& sv,
                              const TensorStrides& so, int causal, const int32_t* kv_lens, const int32_t* q_offsets,
                              const uint8_t* key_keep, int64_t keep_batch_stride, float scale, cudaStream_t stream) {
    const int64_t bh = batch * heads;
    if (bh == 0 || seq == 0) return cudaSuccess;
    CUtensorMap mq, mk, mv, mo;
    // With no key at all nothing is loaded through the K/V maps; they still have to be valid.
    const void* kk = seq_kv > 0 ? k : q;
    const void* vv = seq_kv > 0 ? v : q;
    const int64_t skv = seq_kv > 0 ? seq_kv : 1;
    if (!make_tensor_map_bf16_4d(&mq, q, batch, heads, seq, dim, sq.batch, sq.head, sq.row) ||
        !make_tensor_map_bf16_4d(&mo, out, batch, heads, seq, dim, so.batch, so.head, so.row) ||
        !make_tensor_map_bf16_4d(&mk, kk, batch, heads_kv, skv, dim, sk.batch, sk.head, sk.row) ||
        !make_tensor_map_bf16_4d(&mv, vv, batch, heads_kv, skv, dim, sv.batch, sv.head, sv.row))
        return cudaErrorInvalidValue;
    TcParams p;
    p.o_stride_b = so.batch;
    p.o_stride_h = so.head;
    p.o_stride_row = so.row;
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
    // Schedule (tc_item).  A causal launch without per-batch lengths has a known cost per item, so
    // it runs one CTA per SM over a static list in which the 256-row blocks of a head are paired
    // heavy + light: every CTA gets the same work and the per-item set-up overlaps the previous
    // item.  Other launches (uniform items, or lengths only the device knows) use one CTA per item
    // and leave the balancing to the hardware scheduler.  RT_ATTN_PREFILL_SCHED=persistent|percta
    // overrides the choice.
    const int n_sm = sm_count();
    // RT_ATTN_PREFILL_TILES=1|2 and RT_ATTN_PREFILL_SCHED=persistent|percta override the choices below
    // (read once per process).
    static const int env_tiles = [] {
        const char* s = getenv("RT_ATTN_PREFILL_TILES");
        return (s && s[0] == '1') ? 1 : (s && s[0] == '2') ? 2 : 0;
    }();
    static const int env_sched = [] {
        const char* s = getenv("RT_ATTN_PREFILL_SCHED");
        return (s && !strcmp(s, "persistent")) ? 1 : (s && !strcmp(s, "percta")) ? 2 : 0;
    }();
    // 128-row items (key split inside the CTA) for launches of fewer 256-row blocks than 3/4 of the SMs, and for
    // long sequences up to the point where the persistent schedule takes over: with 64 and more key steps per
    // block the finer items pack the causal imbalance better than they lose per step (measured on B=1 H=8 / 16,
    // N=4096, D=128: 58.6 / 93.7 us against 62.4 / 98.4; at N=2048 the two are level or 256-row items win).
    const int64_t n_blocks256 = bh * ((seq + 255) / 256);
    p.single_tile = (seq > 128 && (n_blocks256 * 4 < 3 * (int64_t)n_sm ||
                                   (n_blocks256 < 2 * (int64_t)n_sm && seq_kv >= 4096 && causal && kv_lens == nullptr)))
                        ? 1 : 0;
    static const int env_stagger = [] {
        const char* s = getenv("RT_ATTN_PREFILL_STAGGER");
        return s ? atoi(s) : 900;
    }();
    p.stagger_clocks = env_stagger;
    if (env_tiles == 1) p.single_tile = 1;
    if (env_tiles == 2) p.single_tile = 0;
    const int64_t n_qb = p.single_tile ? (seq + 127) / 128 : (seq + 255) / 256;
    const int64_t n_items = bh * n_qb;
    if (n_items > 0x3fffffff) return cudaErrorInvalidValue;
    p.n_qb = (int)n_qb;
    bool persistent = causal && kv_lens == nullptr && n_items >= 2 * (int64_t)n_sm && !p.single_tile;
    if (env_sched == 1 && !p.single_tile) persistent = true;  // a single-tile item is its CTA's only item (the merge reuses barriers)
    if (env_sched == 2) persistent = false;
    p.paired = (persistent && n_items >= 2 * (int64_t)n_sm) ? 1 : 0;
    // Per-batch lengths: the length-sorted persistent schedule, if its table fits (tc_item).
    p.sorted = 0;
    if (kv_lens != nullptr && !p.single_tile && env_sched != 2 && n_items >= 2 * (int64_t)n_sm &&
        batch * n_qb <= (dim == 128 ? TcCfg<128>::SCHED_CAP : TcCfg<64>::SCHED_CAP) && batch * n_qb <= 65535) {
        p.sorted = 1;
        p.paired = 0;
        persistent = true;
    }
    p.slots_per_head = p.paired ? (int)((n_qb + 1) / 2) : (int)n_qb;
    p.n_slots = (int)(bh * p.slots_per_head);
    const int64_t n_ctas = (persistent && p.n_slots > n_sm) ? n_sm : p.n_slots;
    p.direct_out = (n_ctas == p.n_slots && !p.paired && !p.sorted) ? 1 : 0;  // every CTA has exactly one item
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
