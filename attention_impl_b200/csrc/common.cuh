// Shared device helpers for libattn_b200 (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/attn_b200.h"

namespace attn {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------------------------
// element conversion
// ---------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_fp8_e4m3>(__nv_fp8_e4m3 x) { return float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Unpack one 32-bit word of packed elements into floats.
__device__ __forceinline__ void unpack2(uint32_t w, __half, float& a, float& b) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    a = f.x; b = f.y;
}
__device__ __forceinline__ void unpack2(uint32_t w, __nv_bfloat16, float& a, float& b) {
    // bf16 -> f32 is a 16-bit left shift
    a = __uint_as_float(w << 16);
    b = __uint_as_float(w & 0xffff0000u);
}
// Four e4m3 bytes -> four floats (via the hardware e4m3x2 -> f16x2 conversion).
__device__ __forceinline__ void unpack4_e4m3(uint32_t w, float& a, float& b, float& c, float& d) {
    uint32_t lo, hi;
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
        : "=r"(lo), "=r"(hi) : "r"(w));
    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    a = f0.x; b = f0.y; c = f1.x; d = f1.y;
}

// Four e4m3 bytes -> two packed fp16 pairs (elements 0,1 and 2,3).
__device__ __forceinline__ void e4m3x4_to_half2x2(uint32_t w, __half2& lo, __half2& hi) {
    uint32_t a, b;
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
        : "=r"(a), "=r"(b) : "r"(w));
    lo = *reinterpret_cast<__half2*>(&a);
    hi = *reinterpret_cast<__half2*>(&b);
}

// ---------------------------------------------------------------------------------------------
// memory
// ---------------------------------------------------------------------------------------------
// 128-bit read-only load that does not allocate in L1 (streamed KV rows are used once).
__device__ __forceinline__ uint4 ldg_stream128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// ---------------------------------------------------------------------------------------------
// warp reductions (xor butterflies)
// ---------------------------------------------------------------------------------------------
template <int WIDTH> __device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int m = WIDTH / 2; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}
template <int WIDTH> __device__ __forceinline__ float group_max(float v) {
#pragma unroll
    for (int m = WIDTH / 2; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace attn
