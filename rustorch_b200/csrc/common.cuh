// Shared device helpers for the sm_100a attention kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rt {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr unsigned kFullMask = 0xffffffffu;

// Device status word: 0 = clean; kernels record here which bounded wait gave up.  The word
// lives in api.cu; kernels receive its device address as a parameter.  Read (and cleared)
// by rt_attn_device_status().
__device__ __forceinline__ void report_timeout(int* status, int code) { atomicCAS(status, 0, code); }

// 16-byte streaming load that bypasses L1 allocation (KV cache is read exactly once).
__device__ __forceinline__ uint4 ld_stream_16B(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// Two bf16 packed in a 32-bit word -> (low element, high element) as f32.
__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

__device__ __forceinline__ uint32_t float2_to_bf16x2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);  // .x = lo (low half), RNE
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// max(a, b, c) in one instruction (three-input max exists from sm_100 on).
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ float fast_log2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace rt
