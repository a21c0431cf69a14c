// FP8 weights with 128 x 128 block scales times 16-bit activations, one warp per output row (PTX module
// `fp8_gemv`): the alternative scale layout of the Gemma-4 path,
//   out[m, n] = f16( sum_k dec(W[n, k]) * scale[n / 128, k / 128] * x[m, k] ).
// Entry point, argument list and geometry of the reference's fp8_gemv_blockwise_wpr_native_f16in_kernel
// (kernels/fp8_gemv.cu:811-891; launcher Fp8GemvF16InLaunch, v3/crates/rvllm-fused/src/gemma4_launcher.rs:839-886):
// grid (ceil(N / 8), M), block 256, W [N, K] E4M3 row-major, scale f32 [ceil(N/128), num_col_blocks], x and out
// 16-bit.  Arithmetic order as the reference, so that results are bit-equal at that geometry: lane l takes the
// eight values at k = 8 l + 256 i; (w * s) * x accumulated into two chains (first four, last four), chains added,
// shuffle-down tree over the lanes.  What differs is the memory side: four iterations of loads (weights, activations,
// scales) are in flight before the first multiply, instead of one dependent 8-byte load at a time.
#include "common.cuh"

namespace rvbs {

__device__ __forceinline__ void dec2(unsigned short packed, float& f0, float& f1) {
    const float2 f = rv::e4m3x2_to_f32x2(packed);
    f0 = f.x;
    f1 = f.y;
}
// bit-level decode of one code (the tail path of the reference; equals the hardware convert for every non-NaN code)
__device__ __forceinline__ float dec1(unsigned char v) {
    const unsigned s = (v >> 7) & 1u, e = (v >> 3) & 0xFu, m = v & 0x7u;
    if (e == 0u) {
        if (m == 0u) return __uint_as_float(s << 31);
        const float sub = ldexpf((float)m, -9);
        return s ? -sub : sub;
    }
    if (e == 0xFu && m == 0x7u) return __uint_as_float((s << 31) | 0x7fc00000u);
    return __uint_as_float((s << 31) | ((e + 120u) << 23) | (m << 20));
}

template <typename T>
__device__ __forceinline__ void gemv_blockscale_body(T* __restrict__ output, const unsigned char* __restrict__ weight,
                                                     const float* __restrict__ scale, const T* __restrict__ input, int M,
                                                     int N, int K, int num_col_blocks) {
    rv::pdl_launch();
    rv::pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp, m = blockIdx.y;
    if (n >= N || m >= M) return;
    const float* srow = scale + (size_t)(n >> 7) * num_col_blocks;
    const unsigned char* w_row = weight + (long long)n * K;
    const T* x_row = input + (long long)m * K;
    float acc0 = 0.0f, acc1 = 0.0f;
    constexpr int UN = 4;
    auto mac = [&](unsigned long long w8, uint4 xv, float s0, float s4) {
        float w0, w1, w2, w3, w4, w5, w6, w7;
        dec2((unsigned short)(w8), w0, w1);
        dec2((unsigned short)(w8 >> 16), w2, w3);
        dec2((unsigned short)(w8 >> 32), w4, w5);
        dec2((unsigned short)(w8 >> 48), w6, w7);
        const float2 x01 = rv::T16<T>::to_f32x2(xv.x), x23 = rv::T16<T>::to_f32x2(xv.y), x45 = rv::T16<T>::to_f32x2(xv.z),
                     x67 = rv::T16<T>::to_f32x2(xv.w);
        acc0 += w0 * s0 * x01.x;
        acc0 += w1 * s0 * x01.y;
        acc0 += w2 * s0 * x23.x;
        acc0 += w3 * s0 * x23.y;
        acc1 += w4 * s4 * x45.x;
        acc1 += w5 * s4 * x45.y;
        acc1 += w6 * s4 * x67.x;
        acc1 += w7 * s4 * x67.y;
    };
    const bool vec_x = (reinterpret_cast<uintptr_t>(x_row) & 15) == 0 && (K & 7) == 0;
    auto load_x = [&](int k) -> uint4 {
        if (vec_x) return rv::ldg128(x_row + k);
        const uint2 lo = __ldg(reinterpret_cast<const uint2*>(x_row + k)), hi = __ldg(reinterpret_cast<const uint2*>(x_row + k + 4));
        return make_uint4(lo.x, lo.y, hi.x, hi.y);
    };
    int k = lane * 8;
    for (; k + 7 + 256 * (UN - 1) < K; k += 256 * UN) {
        unsigned long long w8[UN];
        uint4 xv[UN];
        float s0[UN], s4[UN];
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const int ku = k + 256 * u;
            w8[u] = __ldg(reinterpret_cast<const unsigned long long*>(w_row + ku));
            xv[u] = load_x(ku);
            s0[u] = __ldg(srow + (ku >> 7));
            s4[u] = __ldg(srow + ((ku + 4) >> 7));
        }
#pragma unroll
        for (int u = 0; u < UN; u++) mac(w8[u], xv[u], s0[u], s4[u]);
    }
    for (; k + 7 < K; k += 256)
        mac(__ldg(reinterpret_cast<const unsigned long long*>(w_row + k)), load_x(k), __ldg(srow + (k >> 7)),
            __ldg(srow + ((k + 4) >> 7)));
    float acc = acc0 + acc1;
    for (int kr = (K / 8) * 8 + lane; kr < K; kr += 32)
        acc += dec1(__ldg(w_row + kr)) * __ldg(srow + (kr >> 7)) * rv::T16<T>::to_f32(x_row[kr]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if (lane == 0) output[(long long)m * N + n] = rv::T16<T>::from_f32(acc);
}

}  // namespace rvbs

extern "C" __global__ void __launch_bounds__(256)
fp8_gemv_blockwise_wpr_native_f16in_kernel(__half* output, const unsigned char* weight, const float* scale,
                                           const __half* input, int M, int N, int K, int num_col_blocks) {
    rvbs::gemv_blockscale_body<__half>(output, weight, scale, input, M, N, K, num_col_blocks);
}
extern "C" __global__ void __launch_bounds__(256)
fp8_gemv_blockwise_wpr_native_bf16in_kernel(__nv_bfloat16* output, const unsigned char* weight, const float* scale,
                                            const __nv_bfloat16* input, int M, int N, int K, int num_col_blocks) {
    rvbs::gemv_blockscale_body<__nv_bfloat16>(output, weight, scale, input, M, N, K, num_col_blocks);
}
