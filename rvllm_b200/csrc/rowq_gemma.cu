// Row kernels of the Gemma-4 layer decorations and of the greedy tail, under the reference's entry-point
// names and argument lists (PTX modules fused_qkv_rmsnorm, fused_norm_add_residual_f16,
// residual_scale_f16, logit_softcap, fused_rope_cache_fp8kv):
//
//   fused_qkv_rmsnorm_kernel             per-head RMSNorm of Q and K (learned gain) and V (no gain)
//                                        (v3/kernels/fused_qkv_rmsnorm.cu:28-130)
//   fused_norm_add_residual_f16_kernel   residual = (residual + rmsnorm(gemm_out * channelscale) * gamma) * layer_scalar
//   fused_norm_add_residual_f16in_kernel the same from a 16-bit GEMM output without channel scales
//                                        (v3/kernels/fused_norm_add_residual_f16.cu:8-116)
//   residual_scale_f16_kernel            residual *= scalar (v3/kernels/residual_scale_f16.cu:13-27)
//   logit_softcap_kernel                 logits = cap * tanh(logits / cap) (v3/kernels/logit_softcap.cu:12-31)
//   fused_rope_cache_fp8kv_kernel        interleaved-pair RoPE + static-scale FP8 Q / paged K,V write
//                                        (v3/kernels/fused_rope_cache_fp8kv.cu:20-101)
//
// The caller chooses the geometry (grid = tokens [x heads], block = min(width, 1024)), so every kernel
// works for any block that is a whole number of warps.  Results equal the reference kernels bit for bit
// at the same geometry: a thread accumulates the elements i = tid, tid + blockDim, ... in that order, a
// warp reduces with the same shuffle tree, and the per-warp totals are combined as the reference does
// (a second tree for the QKV norm, a running sum in warp order for the post-norm).  What differs is the
// memory traffic: each element is read from global memory once and kept in registers across the
// reduction instead of being read again for the second pass.
#include "common.cuh"

namespace rvgemma {

constexpr int MAX_KEEP = 8;  // elements a thread keeps in registers (covers widths up to 8 * blockDim)

// sum over lanes with the shuffle-down tree: lane 0 holds the total
__device__ __forceinline__ float warp_sum_down(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}

template <typename T>
__device__ __forceinline__ void qkv_rmsnorm_body(const T* q_in, const T* k_in, const T* v_in, T* q_out, T* k_out,
                                                 T* v_out, const T* q_gamma, const T* k_gamma, int num_tokens,
                                                 int num_heads, int num_kv_heads, int head_dim, float eps,
                                                 int src_row_stride) {
    __shared__ float smem[32];
    rv::pdl_launch();
    rv::pdl_wait();
    const int token = blockIdx.x, head_global = blockIdx.y, tid = threadIdx.x;
    const long long total_width = ((long long)num_heads + 2LL * num_kv_heads) * head_dim;
    if (!q_in || !q_out || !q_gamma || num_tokens <= 0 || num_heads <= 0 || num_kv_heads < 0 || head_dim <= 0 ||
        (num_kv_heads > 0 && (!k_in || !v_in || !k_out || !v_out || !k_gamma)) || token >= num_tokens ||
        total_width > 2147483647LL || (long long)head_global >= (long long)num_heads + 2LL * num_kv_heads ||
        src_row_stride < total_width || !isfinite(eps) || eps <= 0.0f || blockDim.x < 32 || blockDim.x > 1024 ||
        blockDim.x % 32 != 0 || blockDim.y != 1 || blockDim.z != 1 || gridDim.z != 1 || q_out == q_in ||
        (num_kv_heads > 0 && (k_out == k_in || v_out == v_in)))
        return;
    const T* src;
    T* dst;
    const T* gamma = nullptr;
    int heads_this, head_local;
    if (head_global < num_heads) {
        head_local = head_global, heads_this = num_heads, src = q_in, dst = q_out, gamma = q_gamma;
    } else if (head_global < num_heads + num_kv_heads) {
        head_local = head_global - num_heads, heads_this = num_kv_heads, src = k_in, dst = k_out, gamma = k_gamma;
    } else {
        head_local = head_global - num_heads - num_kv_heads, heads_this = num_kv_heads, src = v_in, dst = v_out;
    }
    src += (long long)token * src_row_stride + (long long)head_local * head_dim;  // rows of the packed QKV output
    dst += ((long long)token * heads_this + head_local) * head_dim;               // compact per-component scratch
    float keep[MAX_KEEP];
    float ss = 0.0f;
    int n = 0;
    for (int i = tid; i < head_dim; i += blockDim.x, n++) {
        const float v = rv::T16<T>::to_f32(src[i]);
        if (n < MAX_KEEP) keep[n] = v;
        ss += v * v;
    }
    ss = warp_sum_down(ss);
    const int warp = tid >> 5, lane = tid & 31, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) smem[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float v = lane < nw ? smem[lane] : 0.0f;
        v = warp_sum_down(v);
        if (lane == 0) smem[0] = rsqrtf(v / (float)head_dim + eps);
    }
    __syncthreads();
    const float rms_inv = smem[0];
    n = 0;
    for (int i = tid; i < head_dim; i += blockDim.x, n++) {
        float v = (n < MAX_KEEP ? keep[n] : rv::T16<T>::to_f32(src[i])) * rms_inv;
        if (gamma) v *= rv::T16<T>::to_f32(gamma[i]);
        dst[i] = rv::T16<T>::from_f32(v);
    }
}

// IN = float with channel scales, or the 16-bit type without.
template <typename T, typename IN>
__device__ __forceinline__ void norm_add_residual_body(const IN* gemm_out, const float* channelscale, const T* gamma,
                                                       T* residual, const T* layer_scalar, int hidden, float eps) {
    __shared__ float warp_ss[32];
    rv::pdl_launch();
    rv::pdl_wait();
    constexpr bool F32IN = sizeof(IN) == 4;
    const int token = blockIdx.x, tid = threadIdx.x, stride = blockDim.x;
    if (!gemm_out || (F32IN && !channelscale) || !gamma || !residual || hidden <= 0 || !isfinite(eps) || eps <= 0.0f ||
        blockDim.x < 32 || blockDim.x > 1024 || blockDim.x % 32 != 0 || blockDim.y != 1 || blockDim.z != 1 ||
        gridDim.y != 1 || gridDim.z != 1)
        return;
    const IN* row = gemm_out + (size_t)token * hidden;
    T* res = residual + (size_t)token * hidden;
    auto load = [&](int i) -> float {
        if constexpr (F32IN) return (float)row[i] * channelscale[i];
        else return rv::T16<T>::to_f32(row[i]);
    };
    float keep[MAX_KEEP];
    float ss = 0.0f;
    int n = 0;
    for (int i = tid; i < hidden; i += stride, n++) {
        const float v = load(i);
        if (n < MAX_KEEP) keep[n] = v;
        ss += v * v;
    }
    ss = rv::warp_sum(ss);  // xor butterfly, as the reference
    const int warp = tid >> 5, lane = tid & 31;
    if (lane == 0) warp_ss[warp] = ss;
    __syncthreads();
    if (tid == 0) {
        const int nw = (stride + 31) >> 5;
        float total = 0.0f;
        for (int w = 0; w < nw; w++) total += warp_ss[w];  // running sum in warp order
        warp_ss[0] = total;
    }
    __syncthreads();
    const float rms_inv = rsqrtf(warp_ss[0] / (float)hidden + eps);
    const float ls = layer_scalar ? rv::T16<T>::to_f32(*layer_scalar) : 1.0f;
    n = 0;
    for (int i = tid; i < hidden; i += stride, n++) {
        const float v = n < MAX_KEEP ? keep[n] : load(i);
        const float normed = v * rms_inv * rv::T16<T>::to_f32(gamma[i]);
        const float r = rv::T16<T>::to_f32(res[i]) + normed;
        res[i] = rv::T16<T>::from_f32(r * ls);
    }
}

template <typename T>
__device__ __forceinline__ void residual_scale_body(T* residual, const T* scalar, int hidden) {
    rv::pdl_launch();
    rv::pdl_wait();
    const float s = rv::T16<T>::to_f32(scalar[0]);
    T* row = residual + (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) row[i] = rv::T16<T>::from_f32(rv::T16<T>::to_f32(row[i]) * s);
}

template <typename T>
__device__ __forceinline__ void logit_softcap_body(T* logits, int vocab, float cap) {
    rv::pdl_launch();
    rv::pdl_wait();
    if (!logits || vocab <= 0 || !isfinite(cap) || cap <= 0.0f || blockDim.x == 0 || blockDim.x > 1024 ||
        blockDim.y != 1 || blockDim.z != 1 || gridDim.y != 1 || gridDim.z != 1)
        return;
    const float inv_cap = 1.0f / cap;
    T* row = logits + (long long)blockIdx.x * vocab;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x)
        row[i] = rv::T16<T>::from_f32(cap * tanhf(rv::T16<T>::to_f32(row[i]) * inv_cap));
}

// Interleaved-pair RoPE (elements 2t, 2t + 1 rotate together) with static per-tensor scales: Q is
// written as FP8 with 1 / *q_scale, K (rotated) and V into the paged cache with 1 / *kv_scale.  Inputs
// may be rows of a packed QKV buffer: q_stride / kv_stride are the element strides between tokens
// (heads * head_dim and kv_heads * head_dim for the reference's compact buffers).
template <typename T>
__device__ __forceinline__ void rope_cache_fp8kv_body(const T* q_in, const T* k_in, const T* v_in, long long q_stride,
                                                      long long kv_stride, uint8_t* q_fp8, uint8_t* key_cache,
                                                      uint8_t* value_cache, const T* cos_t, const T* sin_t,
                                                      const int* positions, const int* slot_mapping,
                                                      const float* q_scale_ptr, const float* kv_scale_ptr,
                                                      int num_tokens, int num_heads, int num_kv_heads, int head_dim,
                                                      int max_positions, int num_cache_slots) {
    rv::pdl_launch();
    rv::pdl_wait();
    const int token = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    if (!q_in || !q_fp8 || !positions || !q_scale_ptr || num_tokens <= 0 || num_heads <= 0 || num_kv_heads < 0 ||
        head_dim <= 0 || head_dim % 2 != 0 || max_positions <= 0 || !cos_t || !sin_t ||
        (num_kv_heads > 0 && (!k_in || !v_in || !key_cache || !value_cache || !slot_mapping || !kv_scale_ptr ||
                              num_cache_slots <= 0)) ||
        (long long)num_heads * head_dim > 2147483647LL || (long long)num_kv_heads * head_dim > 2147483647LL ||
        token >= num_tokens || head >= (num_heads > num_kv_heads ? num_heads : num_kv_heads) ||
        blockDim.x < (unsigned)(head_dim / 2) || blockDim.x > 1024 || blockDim.y != 1 || blockDim.z != 1 || gridDim.z != 1)
        return;
    const int half_dim = head_dim / 2;
    if (tid >= half_dim) return;
    const float q_scale = *q_scale_ptr;
    if (!isfinite(q_scale) || q_scale <= 0.0f) return;
    const float q_inv = 1.0f / q_scale;
    float kv_inv = 0.0f;
    if (num_kv_heads > 0) {
        const float kv_scale = *kv_scale_ptr;
        if (!isfinite(kv_scale) || kv_scale <= 0.0f) return;
        kv_inv = 1.0f / kv_scale;
    }
    const int pos = positions[token];
    if (pos < 0 || pos >= max_positions) return;
    const float c = rv::T16<T>::to_f32(cos_t[(long long)pos * half_dim + tid]);
    const float s = rv::T16<T>::to_f32(sin_t[(long long)pos * half_dim + tid]);
    // a pair is one aligned 32-bit word on both sides
    auto pair_in = [](const T* p) { return rv::T16<T>::to_f32x2(*reinterpret_cast<const uint32_t*>(p)); };
    auto pair_out = [](uint8_t* p, float a, float b) {
        *reinterpret_cast<uint16_t*>(p) = (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    };
    if (head < num_heads) {
        const float2 q = pair_in(q_in + (long long)token * q_stride + (long long)head * head_dim + 2 * tid);
        pair_out(q_fp8 + ((long long)token * num_heads + head) * head_dim + 2 * tid, (q.x * c - q.y * s) * q_inv,
                 (q.x * s + q.y * c) * q_inv);
    }
    if (head < num_kv_heads) {
        const int slot = slot_mapping[token];
        if (slot >= 0 && slot < num_cache_slots) {
            const long long in_off = (long long)token * kv_stride + (long long)head * head_dim + 2 * tid;
            const float2 k = pair_in(k_in + in_off), v = pair_in(v_in + in_off);
            const long long off = ((long long)slot * num_kv_heads + head) * head_dim + 2 * tid;
            pair_out(key_cache + off, (k.x * c - k.y * s) * kv_inv, (k.x * s + k.y * c) * kv_inv);
            pair_out(value_cache + off, v.x * kv_inv, v.y * kv_inv);
        }
    }
}

}  // namespace rvgemma

#define RV_GEMMA_ENTRIES(SUFFIX, T)                                                                                     \
    extern "C" __global__ void __launch_bounds__(1024) fused_qkv_rmsnorm##SUFFIX##_kernel(                              \
        const T* q_in, const T* k_in, const T* v_in, T* q_out, T* k_out, T* v_out, const T* q_gamma, const T* k_gamma,  \
        int num_tokens, int num_heads, int num_kv_heads, int head_dim, float eps, int src_row_stride) {                 \
        rvgemma::qkv_rmsnorm_body<T>(q_in, k_in, v_in, q_out, k_out, v_out, q_gamma, k_gamma, num_tokens, num_heads,    \
                                     num_kv_heads, head_dim, eps, src_row_stride);                                      \
    }                                                                                                                   \
    extern "C" __global__ void __launch_bounds__(1024) fused_norm_add_residual_f16##SUFFIX##_kernel(                    \
        const float* gemm_out, const float* channelscale, const T* gamma, T* residual, const T* layer_scalar,           \
        int hidden, float eps) {                                                                                        \
        rvgemma::norm_add_residual_body<T, float>(gemm_out, channelscale, gamma, residual, layer_scalar, hidden, eps);  \
    }                                                                                                                   \
    extern "C" __global__ void __launch_bounds__(1024) fused_norm_add_residual_f16in##SUFFIX##_kernel(                  \
        const T* gemm_out, const T* gamma, T* residual, const T* layer_scalar, int hidden, float eps) {                 \
        rvgemma::norm_add_residual_body<T, T>(gemm_out, nullptr, gamma, residual, layer_scalar, hidden, eps);           \
    }                                                                                                                   \
    extern "C" __global__ void __launch_bounds__(1024) residual_scale_f16##SUFFIX##_kernel(T* residual, const T* scalar, \
                                                                                           int hidden) {                \
        rvgemma::residual_scale_body<T>(residual, scalar, hidden);                                                      \
    }                                                                                                                   \
    extern "C" __global__ void __launch_bounds__(1024) logit_softcap##SUFFIX##_kernel(T* logits, int vocab, float cap) { \
        rvgemma::logit_softcap_body<T>(logits, vocab, cap);                                                             \
    }                                                                                                                   \
    extern "C" __global__ void __launch_bounds__(1024) fused_rope_cache_fp8kv##SUFFIX##_kernel(                         \
        const T* q_in, const T* k_in, const T* v_in, uint8_t* q_fp8_out, uint8_t* key_cache, uint8_t* value_cache,      \
        const T* cos_table, const T* sin_table, const int* positions, const int* slot_mapping,                          \
        const float* q_scale_ptr, const float* kv_scale_ptr, int num_tokens, int num_heads, int num_kv_heads,           \
        int head_dim, int max_positions, int num_cache_slots) {                                                         \
        rvgemma::rope_cache_fp8kv_body<T>(q_in, k_in, v_in, (long long)num_heads * head_dim,                            \
                                          (long long)num_kv_heads * head_dim, q_fp8_out, key_cache, value_cache,        \
                                          cos_table, sin_table, positions, slot_mapping, q_scale_ptr, kv_scale_ptr,     \
                                          num_tokens, num_heads, num_kv_heads, head_dim, max_positions,                 \
                                          num_cache_slots);                                                             \
    }

// f32 logits (this library's LM head writes f32): the same arithmetic without the 16-bit round trip
extern "C" __global__ void __launch_bounds__(1024) logit_softcap_f32_kernel(float* logits, int vocab, float cap) {
    rv::pdl_launch();
    rv::pdl_wait();
    if (!logits || vocab <= 0 || !isfinite(cap) || cap <= 0.0f) return;
    const float inv_cap = 1.0f / cap;
    float* row = logits + (long long)blockIdx.x * vocab;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) row[i] = cap * tanhf(row[i] * inv_cap);
}

RV_GEMMA_ENTRIES(, __half)
RV_GEMMA_ENTRIES(_bf16, __nv_bfloat16)
#undef RV_GEMMA_ENTRIES

// Strided forms for the C launcher (rows of a packed QKV buffer).
extern "C" __global__ void __launch_bounds__(1024)
rvllm_rope_cache_fp8kv_strided_kernel(const __half* q_in, const __half* k_in, const __half* v_in, int in_stride,
                                      uint8_t* q_fp8, uint8_t* key_cache, uint8_t* value_cache, const __half* cos_t,
                                      const __half* sin_t, const int* positions, const int* slot_mapping,
                                      const float* q_scale_ptr, const float* kv_scale_ptr, int num_tokens, int num_heads,
                                      int num_kv_heads, int head_dim, int max_positions, int num_cache_slots) {
    rvgemma::rope_cache_fp8kv_body<__half>(q_in, k_in, v_in, in_stride, in_stride, q_fp8, key_cache, value_cache, cos_t,
                                           sin_t, positions, slot_mapping, q_scale_ptr, kv_scale_ptr, num_tokens,
                                           num_heads, num_kv_heads, head_dim, max_positions, num_cache_slots);
}
extern "C" __global__ void __launch_bounds__(1024)
rvllm_rope_cache_fp8kv_strided_bf16_kernel(const __nv_bfloat16* q_in, const __nv_bfloat16* k_in, const __nv_bfloat16* v_in,
                                           int in_stride, uint8_t* q_fp8, uint8_t* key_cache, uint8_t* value_cache,
                                           const __nv_bfloat16* cos_t, const __nv_bfloat16* sin_t, const int* positions,
                                           const int* slot_mapping, const float* q_scale_ptr, const float* kv_scale_ptr,
                                           int num_tokens, int num_heads, int num_kv_heads, int head_dim,
                                           int max_positions, int num_cache_slots) {
    rvgemma::rope_cache_fp8kv_body<__nv_bfloat16>(q_in, k_in, v_in, in_stride, in_stride, q_fp8, key_cache, value_cache,
                                                  cos_t, sin_t, positions, slot_mapping, q_scale_ptr, kv_scale_ptr,
                                                  num_tokens, num_heads, num_kv_heads, head_dim, max_positions,
                                                  num_cache_slots);
}
