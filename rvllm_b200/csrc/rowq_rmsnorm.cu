// RMSNorm + per-token FP8 E4M3 quantisation (and the plain per-token quantiser).
//
// Drop-in entry points for the PTX module `fused_rmsnorm_fp8_quant`
// (reference: kernels/fused_rmsnorm_fp8_quant.cu:52,108,166), called with the
// geometry the reference launcher fixes: grid = (num_tokens), block =
// (min(hidden, 1024)) or (max(256, min(dim, 1024))), 128 B dynamic shared memory
// (v3/crates/rvllm-fused/src/launcher.rs:218-221,269-272).  Any block size that is a
// multiple of 32 works.
//
// One CTA owns one token row.  The row is pulled from global memory once with 128-bit
// loads into shared memory; the three passes (sum of squares, absmax, encode) then run
// out of shared memory, so HBM sees one read and one write of the row.  The sum of
// squares walks the staged row in thread-strided order (i = tid, tid + blockDim, ...)
// and reduces lane-butterfly then warp-butterfly, which is the order the reference
// kernel rounds in — the scale and every FP8 byte therefore match it bit for bit at
// the same block size.  `*_bf16` twins take bfloat16 rows.
#include "common.cuh"

namespace {

constexpr int STAGE_ELEMS = 16384;  // 32 KB of 16-bit values; longer rows stream from L2

template <typename T>
__device__ __forceinline__ void rmsnorm_quant_row(uint8_t* __restrict__ out, float* __restrict__ scales,
                                                  T* __restrict__ residual_out, const T* __restrict__ in,
                                                  const T* __restrict__ residual, const T* __restrict__ gamma,
                                                  float eps, int hidden) {
    __shared__ __align__(16) T srow[STAGE_ELEMS];
    rv::pdl_launch();
    __shared__ float red[33];
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const size_t base = (size_t)row * hidden;
    const T* x = in + base;
    const bool vec_ok = (hidden % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                        (residual == nullptr || (((reinterpret_cast<uintptr_t>(residual + base) |
                                                   reinterpret_cast<uintptr_t>(residual_out + base)) & 15) == 0));
    const bool staged = hidden <= STAGE_ELEMS && vec_ok;
    // Rows of at most 8 * blockDim values (every decode shape): a thread's one vector of the row and
    // of gamma stays in registers across the absmax and the encode pass.  gamma is a weight: its vector is
    // fetched before the wait for the kernel ahead in the stream (under programmatic dependent launch; a
    // plain launch starts behind that kernel anyway), not behind the sum-of-squares reduction.
    const bool one_vec = vec_ok && (hidden >> 3) <= nt && ((reinterpret_cast<uintptr_t>(out + base) & 7) == 0);
    uint4 keep_x = make_uint4(0, 0, 0, 0), keep_g = make_uint4(0, 0, 0, 0);
    if (one_vec && tid < (hidden >> 3)) keep_g = rv::ldg128(reinterpret_cast<const uint4*>(gamma) + tid);
    rv::pdl_wait();

    float ss = 0.0f;
    if (residual != nullptr) {
        // sum of squares of the unrounded sum, in thread-strided order; the rounded sum is
        // what the later passes normalise (reference :129-131,143).
        const T* r = residual + base;
        for (int i = tid; i < hidden; i += nt) {
            float v = rv::T16<T>::to_f32(x[i]) + rv::T16<T>::to_f32(r[i]);
            T h = rv::T16<T>::from_f32(v);
            residual_out[base + i] = h;
            if (staged) srow[i] = h;
            ss += v * v;
        }
    } else if (staged) {
        const int nvec = hidden >> 3;
        for (int v = tid; v < nvec; v += nt)
            reinterpret_cast<uint4*>(srow)[v] = rv::ldg128(reinterpret_cast<const uint4*>(x) + v);
        __syncthreads();
        for (int i = tid; i < hidden; i += nt) {
            float v = rv::T16<T>::to_f32(srow[i]);
            ss += v * v;
        }
    } else {
        for (int i = tid; i < hidden; i += nt) {
            float v = rv::T16<T>::to_f32(x[i]);
            ss += v * v;
        }
    }
    const float sum_sq = rv::block_sum(ss, red);  // barrier inside also publishes srow
    const float rms = rsqrtf(sum_sq / (float)hidden + eps);
    const T* src = staged ? srow : (residual != nullptr ? residual_out + base : x);

    float amax = 0.0f;
    if (one_vec) {
        if (tid < (hidden >> 3)) {
            keep_x = reinterpret_cast<const uint4*>(src)[tid];
            const uint32_t* xp = &keep_x.x;
            const uint32_t* gp = &keep_g.x;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 a = rv::T16<T>::to_f32x2(xp[j]), g = rv::T16<T>::to_f32x2(gp[j]);
                amax = fmaxf(amax, fmaxf(fabsf(a.x * rms * g.x), fabsf(a.y * rms * g.y)));
            }
        }
    } else if (vec_ok) {
        const int nvec = hidden >> 3;
        for (int v = tid; v < nvec; v += nt) {
            uint4 xv = reinterpret_cast<const uint4*>(src)[v];
            uint4 gv = rv::ldg128(reinterpret_cast<const uint4*>(gamma) + v);
            const uint32_t* xp = &xv.x;
            const uint32_t* gp = &gv.x;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 a = rv::T16<T>::to_f32x2(xp[j]), g = rv::T16<T>::to_f32x2(gp[j]);
                amax = fmaxf(amax, fmaxf(fabsf(a.x * rms * g.x), fabsf(a.y * rms * g.y)));
            }
        }
    } else {
        for (int i = tid; i < hidden; i += nt)
            amax = fmaxf(amax, fabsf(rv::T16<T>::to_f32(src[i]) * rms * rv::T16<T>::to_f32(gamma[i])));
    }
    amax = rv::block_max(amax, red);
    const float scale = rv::row_scale(amax);
    if (tid == 0) scales[row] = scale;
    const float inv = 1.0f / scale;

    if (one_vec) {
        if (tid < (hidden >> 3)) {
            const uint32_t* xp = &keep_x.x;
            const uint32_t* gp = &keep_g.x;
            float f[8];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 a = rv::T16<T>::to_f32x2(xp[j]), g = rv::T16<T>::to_f32x2(gp[j]);
                f[2 * j] = a.x * rms * g.x * inv;
                f[2 * j + 1] = a.y * rms * g.y * inv;
            }
            uint2 o;
            o.x = rv::f32x4_to_e4m3x4(f[0], f[1], f[2], f[3]);
            o.y = rv::f32x4_to_e4m3x4(f[4], f[5], f[6], f[7]);
            reinterpret_cast<uint2*>(out + base)[tid] = o;
        }
    } else if (vec_ok && ((reinterpret_cast<uintptr_t>(out + base) & 7) == 0)) {
        const int nvec = hidden >> 3;
        for (int v = tid; v < nvec; v += nt) {
            uint4 xv = reinterpret_cast<const uint4*>(src)[v];
            uint4 gv = rv::ldg128(reinterpret_cast<const uint4*>(gamma) + v);
            const uint32_t* xp = &xv.x;
            const uint32_t* gp = &gv.x;
            float f[8];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 a = rv::T16<T>::to_f32x2(xp[j]), g = rv::T16<T>::to_f32x2(gp[j]);
                f[2 * j] = a.x * rms * g.x * inv;
                f[2 * j + 1] = a.y * rms * g.y * inv;
            }
            uint2 o;
            o.x = rv::f32x4_to_e4m3x4(f[0], f[1], f[2], f[3]);
            o.y = rv::f32x4_to_e4m3x4(f[4], f[5], f[6], f[7]);
            reinterpret_cast<uint2*>(out + base)[v] = o;
        }
    } else {
        for (int i = tid; i < hidden; i += nt)
            out[base + i] = rv::f32_to_e4m3(rv::T16<T>::to_f32(src[i]) * rms * rv::T16<T>::to_f32(gamma[i]) * inv);
    }
}

template <typename T>
__device__ __forceinline__ void quant_row(uint8_t* __restrict__ out, float* __restrict__ scales,
                                          const T* __restrict__ in, int dim) {
    __shared__ float red[33];
    rv::pdl_launch();
    rv::pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const size_t base = (size_t)row * dim;
    const T* x = in + base;
    const bool vec_ok = (dim % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                        ((reinterpret_cast<uintptr_t>(out + base) & 7) == 0);
    const int nvec = dim >> 3;
    // First vector of each thread stays in registers; rows of <= 8 * blockDim values
    // (every decode shape) are therefore read from memory once.
    uint4 keep = make_uint4(0, 0, 0, 0);
    float amax = 0.0f;
    if (vec_ok) {
        for (int v = tid; v < nvec; v += nt) {
            uint4 xv = rv::ldg128(reinterpret_cast<const uint4*>(x) + v);
            if (v == tid) keep = xv;
            const uint32_t* xp = &xv.x;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 a = rv::T16<T>::to_f32x2(xp[j]);
                amax = fmaxf(amax, fmaxf(fabsf(a.x), fabsf(a.y)));
            }
        }
    } else {
        for (int i = tid; i < dim; i += nt) amax = fmaxf(amax, fabsf(rv::T16<T>::to_f32(x[i])));
    }
    amax = rv::block_max(amax, red);
    const float scale = rv::row_scale(amax);
    if (tid == 0) scales[row] = scale;
    const float inv = 1.0f / scale;
    if (vec_ok) {
        for (int v = tid; v < nvec; v += nt) {
            uint4 xv = (v == tid) ? keep : rv::ldg128(reinterpret_cast<const uint4*>(x) + v);
            const uint32_t* xp = &xv.x;
            float f[8];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 a = rv::T16<T>::to_f32x2(xp[j]);
                f[2 * j] = a.x * inv;
                f[2 * j + 1] = a.y * inv;
            }
            uint2 o;
            o.x = rv::f32x4_to_e4m3x4(f[0], f[1], f[2], f[3]);
            o.y = rv::f32x4_to_e4m3x4(f[4], f[5], f[6], f[7]);
            reinterpret_cast<uint2*>(out + base)[v] = o;
        }
    } else {
        for (int i = tid; i < dim; i += nt) out[base + i] = rv::f32_to_e4m3(rv::T16<T>::to_f32(x[i]) * inv);
    }
}

}  // namespace

extern "C" __global__ void __launch_bounds__(1024)
fused_rmsnorm_fp8_quant_kernel(uint8_t* out, float* scales, const __half* in, const __half* gamma, float eps,
                               int hidden) {
    rmsnorm_quant_row<__half>(out, scales, nullptr, in, nullptr, gamma, eps, hidden);
}
extern "C" __global__ void __launch_bounds__(1024)
fused_add_rmsnorm_fp8_quant_kernel(uint8_t* out, float* scales, __half* residual_out, const __half* in,
                                   const __half* residual, const __half* gamma, float eps, int hidden) {
    rmsnorm_quant_row<__half>(out, scales, residual_out, in, residual, gamma, eps, hidden);
}
extern "C" __global__ void __launch_bounds__(1024)
quantize_fp8_per_token_kernel(uint8_t* out, float* scales, const __half* in, int dim) {
    quant_row<__half>(out, scales, in, dim);
}
extern "C" __global__ void __launch_bounds__(1024)
fused_rmsnorm_fp8_quant_bf16_kernel(uint8_t* out, float* scales, const __nv_bfloat16* in,
                                    const __nv_bfloat16* gamma, float eps, int hidden) {
    rmsnorm_quant_row<__nv_bfloat16>(out, scales, nullptr, in, nullptr, gamma, eps, hidden);
}
extern "C" __global__ void __launch_bounds__(1024)
fused_add_rmsnorm_fp8_quant_bf16_kernel(uint8_t* out, float* scales, __nv_bfloat16* residual_out,
                                        const __nv_bfloat16* in, const __nv_bfloat16* residual,
                                        const __nv_bfloat16* gamma, float eps, int hidden) {
    rmsnorm_quant_row<__nv_bfloat16>(out, scales, residual_out, in, residual, gamma, eps, hidden);
}
extern "C" __global__ void __launch_bounds__(1024)
quantize_fp8_per_token_bf16_kernel(uint8_t* out, float* scales, const __nv_bfloat16* in, int dim) {
    quant_row<__nv_bfloat16>(out, scales, in, dim);
}
