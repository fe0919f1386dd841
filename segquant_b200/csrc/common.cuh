// Shared host/device helpers of the segquant_b200 native library (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/segquant_b200.h"

namespace sq {

// ---- host-side error reporting (thread local message, C status codes) ---------------------
void set_error(const char* fmt, ...);
void clear_error();

#define SQ_REQUIRE(cond, code, ...)      \
    do {                                 \
        if (!(cond)) {                   \
            ::sq::set_error(__VA_ARGS__);\
            return (code);               \
        }                                \
    } while (0)

#define SQ_CUDA_OK(expr)                                                               \
    do {                                                                               \
        cudaError_t _e = (expr);                                                       \
        if (_e != cudaSuccess) {                                                       \
            ::sq::set_error("%s failed: %s", #expr, cudaGetErrorString(_e));           \
            return SQ_ERR_CUDA;                                                        \
        }                                                                              \
    } while (0)

constexpr int kNumSMs = 148;  // B200

// ---- device helpers -----------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// The reference's int8 rule: clamp to [-128, 127] first, then round to nearest even
// (segquant/src/real_quant/quantizer.cuh:32-35).  Returns the byte.
__device__ __forceinline__ uint32_t quant_int8(float scaled) {
    float clipped = fminf(fmaxf(scaled, -128.0f), 127.0f);
    return static_cast<uint32_t>(__float2int_rn(clipped)) & 0xFFu;
}
// The reference's int4 rule (quantizer.cuh:37-39): clamp to [-8, 7], RN-even, low 4 bits.
__device__ __forceinline__ uint32_t quant_int4(float scaled) {
    float clipped = fminf(fmaxf(scaled, -8.0f), 7.0f);
    return static_cast<uint32_t>(__float2int_rn(clipped)) & 0xFu;
}
// The reference's fp8 rule: static_cast<__nv_fp8_e4m3>(float) = saturating RN-even
// (quantizer.cuh:21-29).
__device__ __forceinline__ uint32_t quant_e4m3(float scaled) {
    return static_cast<uint32_t>(__nv_cvt_float_to_fp8(scaled, __NV_SATFINITE, __NV_E4M3));
}
// Two at once: low byte = a, high byte = b.
__device__ __forceinline__ uint32_t quant_e4m3x2(float a, float b) {
    return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3));
}

// 16 consecutive elements of T as floats, through 128-bit loads.  p must be 16-byte aligned.
template <typename T>
__device__ __forceinline__ void load16(const T* __restrict__ p, float (&v)[16]);
template <>
__device__ __forceinline__ void load16<float>(const float* __restrict__ p, float (&v)[16]) {
    const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float4 t = __ldg(q + i);
        v[4 * i + 0] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
}
template <>
__device__ __forceinline__ void load16<__half>(const __half* __restrict__ p, float (&v)[16]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 t = __ldg(q + i);
        const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 f = __half22float2(h[j]);
            v[8 * i + 2 * j] = f.x; v[8 * i + 2 * j + 1] = f.y;
        }
    }
}
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* __restrict__ p, float (&v)[16]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 t = __ldg(q + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(h[j]);
            v[8 * i + 2 * j] = f.x; v[8 * i + 2 * j + 1] = f.y;
        }
    }
}

}  // namespace sq
