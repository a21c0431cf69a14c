// act(gate) * up + per-token FP8 E4M3 quantisation over rows laid out [gate(0..I) | up(I..2I)].
//
// Shared body of the PTX modules `fused_silu_fp8_quant` (reference:
// kernels/fused_silu_fp8_quant.cu:42-120) and `fused_gelu_mul_fp8_quant` (reference:
// v3/kernels/fused_gelu_mul_fp8_quant.cu:53-129).  Caller geometry: grid =
// (num_tokens), block = (min(I, 1024)) (v3/crates/rvllm-fused/src/launcher.rs:318-321).
//
// One CTA per row.  Gate and up are read once with 128-bit loads; the products stay in
// registers (up to 4 vectors of 8 per thread) across the absmax reduction, and rows
// too long for that are recomputed from L2 instead of being refused.  A non-finite
// product makes the row's scale NaN, as in the reference.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace rvact {

constexpr int ACT_SILU = 0;
constexpr int ACT_GELU = 1;

template <int ACT> __device__ __forceinline__ float act(float g) {
    if (ACT == ACT_SILU) return g / (1.0f + expf(-g));
    float g3 = g * g * g;
    float inner = 0.7978845608f * (g + 0.044715f * g3);
    return 0.5f * g * (1.0f + tanhf(inner));
}

template <int ACT, typename T>
__device__ __forceinline__ void mul8(const uint4& gv, const uint4& uv, float* y) {
    const uint32_t* gp = &gv.x;
    const uint32_t* up = &uv.x;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float2 g = rv::T16<T>::to_f32x2(gp[j]), u = rv::T16<T>::to_f32x2(up[j]);
        y[2 * j] = act<ACT>(g.x) * u.x;
        y[2 * j + 1] = act<ACT>(g.y) * u.y;
    }
}

template <int ACT, typename T>
__device__ __forceinline__ void act_mul_quant_row(uint8_t* __restrict__ out, float* __restrict__ scales,
                                                  const T* __restrict__ gate_up, int inter) {
    constexpr int CACHE_VECS = 4;
    __shared__ float red[33];
    __shared__ int bad;
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    rv::pdl_launch();
    rv::pdl_wait();
    if (out == nullptr || scales == nullptr || gate_up == nullptr || inter <= 0 || (inter & 7) != 0) return;
    const T* g = gate_up + (size_t)row * 2 * inter;
    const T* u = g + inter;
    uint8_t* o = out + (size_t)row * inter;
    if (((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(u)) & 15) != 0 ||
        (reinterpret_cast<uintptr_t>(o) & 7) != 0)
        return;
    if (tid == 0) bad = 0;
    __syncthreads();
    const int nvec = inter >> 3;
    float cache[CACHE_VECS * 8];
    float amax = 0.0f;
    bool nonfinite = false;
    int c = 0;
    for (int v = tid; v < nvec; v += nt, c++) {
        float y[8];
        mul8<ACT, T>(rv::ldg128(reinterpret_cast<const uint4*>(g) + v),
                     rv::ldg128(reinterpret_cast<const uint4*>(u) + v), y);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            nonfinite |= !isfinite(y[j]);
            amax = fmaxf(amax, fabsf(y[j]));
        }
        if (c < CACHE_VECS) {
#pragma unroll
            for (int k = 0; k < CACHE_VECS; k++)
                if (k == c) {
#pragma unroll
                    for (int j = 0; j < 8; j++) cache[k * 8 + j] = y[j];
                }
        }
    }
    if (nonfinite) atomicExch(&bad, 1);
    amax = rv::block_max(amax, red);  // barriers inside order the flag as well
    const float scale = bad ? CUDART_NAN_F : rv::row_scale(amax);
    if (tid == 0) scales[row] = scale;
    const float inv = 1.0f / scale;
    c = 0;
    for (int v = tid; v < nvec; v += nt, c++) {
        float y[8];
        if (c < CACHE_VECS) {
#pragma unroll
            for (int k = 0; k < CACHE_VECS; k++)
                if (k == c) {
#pragma unroll
                    for (int j = 0; j < 8; j++) y[j] = cache[k * 8 + j];
                }
        } else {
            mul8<ACT, T>(rv::ldg128(reinterpret_cast<const uint4*>(g) + v),
                         rv::ldg128(reinterpret_cast<const uint4*>(u) + v), y);
        }
        uint2 w;
        w.x = rv::f32x4_to_e4m3x4(y[0] * inv, y[1] * inv, y[2] * inv, y[3] * inv);
        w.y = rv::f32x4_to_e4m3x4(y[4] * inv, y[5] * inv, y[6] * inv, y[7] * inv);
        reinterpret_cast<uint2*>(o)[v] = w;
    }
}

// The same row operation spread over a thread-block cluster: CL CTAs share one row, each owns a
// contiguous slice of it, and the row's absmax / non-finite flag are combined through distributed
// shared memory.  A decode batch has only a few dozen rows, so one CTA per row leaves most SMs idle
// and the row's 2 * I values crawl through a single SM; with eight CTAs per row the kernel is a
// short HBM/L2 burst instead.  max() is order-independent and the per-element arithmetic is the
// one above, so bytes and scales are identical to the one-CTA-per-row kernel.
// Geometry: grid = (CL, num_tokens), cluster = (CL, 1, 1), block = CLUSTER_THREADS.
constexpr int CLUSTER_THREADS = 256;
// CLUSTER_CACHE_VECS 16-byte pieces of the slice stay in registers between the two passes (the rest is
// read again); MINB CTAs per SM are asked of the compiler.  Two forms are launched: (4, 3) when the
// whole grid is resident anyway (at most 3 CTAs per SM), (3, 4) when a fourth CTA per SM lets a larger
// grid run as one wave -- the kernel is one latency chain per CTA, so a second wave doubles its time.
template <int ACT, typename T, int CLUSTER_CACHE_VECS, int MINB>
__global__ void __launch_bounds__(CLUSTER_THREADS, MINB)
act_mul_quant_cluster_kernel(uint8_t* __restrict__ out, float* __restrict__ scales, const T* __restrict__ gate_up, int inter) {
    namespace cg = cooperative_groups;
    __shared__ float red[33];
    __shared__ int bad;
    __shared__ float share[16];  // {absmax, non-finite flag} of each of the (at most 8) CTAs of the cluster
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank(), cl = (int)cluster.num_blocks();
    const int row = blockIdx.y, tid = threadIdx.x;
    rv::pdl_launch();
    cluster.barrier_arrive();  // "this CTA runs": awaited (long since complete) before the first store into a peer
    rv::pdl_wait();
    const T* g = gate_up + (size_t)row * 2 * inter;
    const T* u = g + inter;
    uint8_t* o = out + (size_t)row * inter;
    if (tid == 0) bad = 0;
    __syncthreads();
    const int nvec = inter >> 3;
    const int v_lo = (int)((long long)nvec * rank / cl), v_hi = (int)((long long)nvec * (rank + 1) / cl);
    float cache[CLUSTER_CACHE_VECS * 8];
    float amax = 0.0f;
    bool nonfinite = false;
    int c = 0;
    for (int v = v_lo + tid; v < v_hi; v += CLUSTER_THREADS, c++) {
        float y[8];
        mul8<ACT, T>(rv::ldg128(reinterpret_cast<const uint4*>(g) + v),
                     rv::ldg128(reinterpret_cast<const uint4*>(u) + v), y);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            nonfinite |= !isfinite(y[j]);
            amax = fmaxf(amax, fabsf(y[j]));
        }
        if (c < CLUSTER_CACHE_VECS) {
#pragma unroll
            for (int k = 0; k < CLUSTER_CACHE_VECS; k++)
                if (k == c) {
#pragma unroll
                    for (int j = 0; j < 8; j++) cache[k * 8 + j] = y[j];
                }
        }
    }
    if (nonfinite) atomicExch(&bad, 1);
    amax = rv::block_max(amax, red);  // barriers inside order the flag as well
    // Every CTA stores its {absmax, flag} into slot `rank` of every peer's table and the cluster meets
    // once (one barrier round trip instead of meet, read remotely, meet again before leaving).
    cluster.barrier_wait();
    if (tid < cl) {
        float* peer = cluster.map_shared_rank(share, tid);
        peer[2 * rank] = amax;
        peer[2 * rank + 1] = bad ? 1.0f : 0.0f;
    }
    cluster.sync();
    float row_max = 0.0f, row_bad = 0.0f;
    for (int r = 0; r < cl; r++) {
        row_max = fmaxf(row_max, share[2 * r]);
        row_bad = fmaxf(row_bad, share[2 * r + 1]);
    }
    const float scale = row_bad != 0.0f ? CUDART_NAN_F : rv::row_scale(row_max);
    if (rank == 0 && tid == 0) scales[row] = scale;
    const float inv = 1.0f / scale;
    c = 0;
    for (int v = v_lo + tid; v < v_hi; v += CLUSTER_THREADS, c++) {
        float y[8];
        if (c < CLUSTER_CACHE_VECS) {
#pragma unroll
            for (int k = 0; k < CLUSTER_CACHE_VECS; k++)
                if (k == c) {
#pragma unroll
                    for (int j = 0; j < 8; j++) y[j] = cache[k * 8 + j];
                }
        } else {
            mul8<ACT, T>(rv::ldg128(reinterpret_cast<const uint4*>(g) + v),
                         rv::ldg128(reinterpret_cast<const uint4*>(u) + v), y);
        }
        uint2 w;
        w.x = rv::f32x4_to_e4m3x4(y[0] * inv, y[1] * inv, y[2] * inv, y[3] * inv);
        w.y = rv::f32x4_to_e4m3x4(y[4] * inv, y[5] * inv, y[6] * inv, y[7] * inv);
        reinterpret_cast<uint2*>(o)[v] = w;
    }
}

}  // namespace rvact
