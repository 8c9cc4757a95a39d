// Device self-test of the tensor-core building blocks the prefill kernel is made of.
//
// One CTA runs the two MMA shapes of the attention kernel on a single 128-row tile and dumps
// the raw accumulators, so the descriptor encodings can be checked against a plain matmul:
//   S = A * B^T        SS MMA, A and B K-major in 128-byte-swizzled shared memory (as Q, K)
//   O = bf16(S/16) * V  TS MMA, A from TMEM (as P), B MN-major shared memory (as V)
// Exposed through rt_debug_tc_selftest() in the C ABI.
#include <cuda.h>

#include "../../include/rustorch_attn.h"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace rt {

using namespace ptx;

template <int D>
__global__ void __launch_bounds__(128, 1)
tc_selftest_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                   const __grid_constant__ CUtensorMap tm_v, float* s_out, float* o_out, int* status) {
    constexpr int TILE = 128 * D * 2, SUB = 128 * 64 * 2, NSUB = D / 64;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = sA + TILE;
    uint8_t* sV = sB + TILE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + TILE);  // [0] loads, [1] S done, [2] O done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_init(&bars[2], 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t lane_sel = (uint32_t)(warp * 32) << 16;
    bool ok = true;

    if (threadIdx.x == 0) {
        mbar_arrive_expect_tx(&bars[0], 3 * TILE);
        for (int s = 0; s < NSUB; ++s) {
            tma_load_3d(sA + s * SUB, &tm_a, &bars[0], s * 64, 0, 0);
            tma_load_3d(sB + s * SUB, &tm_b, &bars[0], s * 64, 0, 0);
            tma_load_3d(sV + s * SUB, &tm_v, &bars[0], s * 64, 0, 0);
        }
        if (mbar_wait(&bars[0], 0, status, 201)) {
            tc_fence_after();
            constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t off = (kk / 4) * SUB + (kk % 4) * 32;
                mma_ss(tmem_base, make_smem_desc_sw128(smem_u32(sA) + off, 16, 1024),
                       make_smem_desc_sw128(smem_u32(sB) + off, 16, 1024), idesc_s, kk > 0);
            }
        }
        mma_commit(&bars[1]);
    }
    ok = __all_sync(kFullMask, mbar_wait(&bars[1], 0, status, 202));
    if (ok) {
        tc_fence_after();
        const int row = warp * 32 + lane;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            uint32_t s[32];
            tmem_ld32(tmem_base + lane_sel + ch * 32, s);
            tc_wait_ld();
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; ++i) s_out[row * 128 + ch * 32 + i] = __uint_as_float(s[i]);
#pragma unroll
            for (int i = 0; i < 16; ++i)
                pk[i] = float2_to_bf16x2(__uint_as_float(s[2 * i]) * 0.0625f, __uint_as_float(s[2 * i + 1]) * 0.0625f);
            tmem_st16(tmem_base + lane_sel + 128 + ch * 16, pk);  // P at columns [128,192)
        }
        tc_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
        tc_fence_after();
        if (ok) {
            constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
                mma_ts(tmem_base + 256, tmem_base + 128 + kk * 8,
                       make_smem_desc_sw128(smem_u32(sV) + kk * 2048, SUB, 1024), idesc_o, kk > 0);
        }
        mma_commit(&bars[2]);
    }
    if (__all_sync(kFullMask, mbar_wait(&bars[2], 0, status, 203)) && ok) {
        tc_fence_after();
        const int row = warp * 32 + lane;
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
            uint32_t o[32];
            tmem_ld32(tmem_base + lane_sel + 256 + ch * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o_out[row * D + ch * 32 + i] = __uint_as_float(o[i]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

bool make_tensor_map_bf16_3d(CUtensorMap* map, const void* base, int64_t bh, int64_t seq, int dim);

template <int D>
static cudaError_t run_selftest(const void* a, const void* b, const void* v, float* s_out, float* o_out,
                                cudaStream_t stream) {
    CUtensorMap ma, mb, mv;
    if (!make_tensor_map_bf16_3d(&ma, a, 1, 128, D) || !make_tensor_map_bf16_3d(&mb, b, 1, 128, D) ||
        !make_tensor_map_bf16_3d(&mv, v, 1, 128, D))
        return cudaErrorInvalidValue;
    int* status = device_status_ptr();
    if (!status) return cudaErrorInvalidSymbol;
    constexpr int smem = 3 * 128 * D * 2 + 64 + 1024;
    auto kern = tc_selftest_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kern<<<1, 128, smem, stream>>>(ma, mb, mv, s_out, o_out, status);
    return cudaGetLastError();
}

}  // namespace rt

extern "C" int rt_debug_tc_selftest(const void* a, const void* b, const void* v, float* s_out, float* o_out, int dim,
                                    void* stream) {
    if (!a || !b || !v || !s_out || !o_out) return RT_ERR_NULL_POINTER;
    cudaError_t e;
    if (dim == 128)
        e = rt::run_selftest<128>(a, b, v, s_out, o_out, reinterpret_cast<cudaStream_t>(stream));
    else if (dim == 64)
        e = rt::run_selftest<64>(a, b, v, s_out, o_out, reinterpret_cast<cudaStream_t>(stream));
    else
        return RT_ERR_UNSUPPORTED;
    return (int)e;
}
