// Shared device helpers for the sm_100a FP8 decode kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#define RV_FP8_MAX 448.0f

namespace rv {

// ---- 16-bit activation types ------------------------------------------------------
template <typename T> struct T16;
template <> struct T16<__half> {
    static __device__ __forceinline__ float to_f32(__half h) { return __half2float(h); }
    static __device__ __forceinline__ __half from_f32(float f) { return __float2half(f); }
    // f16 results are clamped to the largest finite value before narrowing so that an
    // overflowing accumulator cannot inject inf into the residual stream.
    static __device__ __forceinline__ __half from_f32_sat(float f) {
        return __float2half(fminf(fmaxf(f, -65504.0f), 65504.0f));
    }
    static __device__ __forceinline__ float2 to_f32x2(uint32_t u) {
        return __half22float2(*reinterpret_cast<const __half2*>(&u));
    }
};
template <> struct T16<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f32(__nv_bfloat16 h) { return __bfloat162float(h); }
    static __device__ __forceinline__ __nv_bfloat16 from_f32(float f) { return __float2bfloat16(f); }
    static __device__ __forceinline__ __nv_bfloat16 from_f32_sat(float f) { return __float2bfloat16(f); }
    static __device__ __forceinline__ float2 to_f32x2(uint32_t u) {
        return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
    }
};

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b) {
    T lo = T16<T>::from_f32(a), hi = T16<T>::from_f32(b);
    return (uint32_t)(*reinterpret_cast<unsigned short*>(&lo)) |
           ((uint32_t)(*reinterpret_cast<unsigned short*>(&hi)) << 16);
}
template <typename T> __device__ __forceinline__ uint32_t pack2_sat(float a, float b) {
    T lo = T16<T>::from_f32_sat(a), hi = T16<T>::from_f32_sat(b);
    return (uint32_t)(*reinterpret_cast<unsigned short*>(&lo)) |
           ((uint32_t)(*reinterpret_cast<unsigned short*>(&hi)) << 16);
}

// ---- FP8 E4M3 -----------------------------------------------------------------------
// Round-to-nearest-even, saturate to +-448, NaN -> 0x7f.
__device__ __forceinline__ uint8_t f32_to_e4m3(float x) {
    return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
// Four values -> four bytes packed little-endian (value 0 in the low byte).
__device__ __forceinline__ uint32_t f32x4_to_e4m3x4(float a, float b, float c, float d) {
    uint32_t lo = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    uint32_t hi = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}
// Two E4M3 bytes -> two f32.  E4M3 -> f16 is an exact widening.
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint32_t pair16) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((unsigned short)pair16));
    return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t pair16) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((unsigned short)pair16));
    return h2;
}
__device__ __forceinline__ void e4m3x4_to_f32x4(uint32_t u, float* f) {
    float2 lo = e4m3x2_to_f32x2(u & 0xffffu), hi = e4m3x2_to_f32x2(u >> 16);
    f[0] = lo.x; f[1] = lo.y; f[2] = hi.x; f[3] = hi.y;
}

// ---- warp / block reductions ---------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block-wide sum / max broadcast to every thread.  `red` holds >= 33 floats.  The sum
// uses a fixed order (lane butterfly, then a butterfly over the per-warp totals) so a
// given block size always rounds the same way.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (l == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = l < nw ? red[l] : 0.0f;
        t = warp_sum(t);
        if (l == 0) red[32] = t;
    }
    __syncthreads();
    float r = red[32];
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    if (l == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = l < nw ? red[l] : 0.0f;
        t = warp_max(t);
        if (l == 0) red[32] = t;
    }
    __syncthreads();
    float r = red[32];
    __syncthreads();
    return r;
}

// Per-row scale and its reciprocal: scale = max(absmax / 448, 1e-12).
__device__ __forceinline__ float row_scale(float absmax) { return fmaxf(absmax / RV_FP8_MAX, 1e-12f); }

__device__ __forceinline__ uint4 ldg128(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
// Streaming 128-bit load that does not pollute L1 (weights and KV rows are read once).
__device__ __forceinline__ uint4 ld_stream128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Programmatic dependent launch.  Every kernel of the decode chain calls pdl_launch() first
// (lets the next kernel of the stream start its prologue and weight prefetch while this one
// runs) and pdl_wait() before it touches anything a predecessor wrote or may still read.
// Both are no-ops when the kernel was launched without the programmatic-serialization
// attribute (e.g. by a caller that uses plain launches).
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

}  // namespace rv
