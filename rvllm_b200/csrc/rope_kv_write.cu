// RoPE + FP8 quantisation of Q + write of K/V into the paged FP8 cache with
// per-(slot, kv_head) scales — the producer of the attention kernel's inputs.
//
// Numerics follow the reference's fused_rope_partial_fp8kv_kernel
// (v3/kernels/fused_rope_partial_fp8kv.cu:54-214): half-split rotary pairing (element i
// pairs with i + head_dim/2) over the first rotary_dim/2 pairs, cos/sin tables
// [max_positions, rotary_dim/2] in the activation type, dynamic scale
// max(amax / 448, 1e-12) per (token, head) for Q and per (slot, kv_head) for K and V,
// a non-finite value making that scale NaN; slot < 0 or >= num_cache_slots skips the
// cache write.  Unlike the reference entry point, the Q/K/V inputs carry an explicit row
// stride so the packed [T, q_dim + 2*kv_dim] output of the fused QKV projection can be
// consumed for T > 1 without a split copy.
// grid = (num_tokens, max(heads, kv_heads)), block = head_dim / 2 (32..256 threads).
#include "common.cuh"

namespace {

template <typename T>
__device__ __forceinline__ void rope_pair(const T* row, const T* cos_t, const T* sin_t, int pos, int tid,
                                          int half_head, int half_rot, float& lo, float& hi) {
    const float a = rv::T16<T>::to_f32(row[tid]), b = rv::T16<T>::to_f32(row[tid + half_head]);
    if (tid < half_rot) {
        const float c = rv::T16<T>::to_f32(cos_t[(size_t)pos * half_rot + tid]);
        const float s = rv::T16<T>::to_f32(sin_t[(size_t)pos * half_rot + tid]);
        lo = a * c - b * s;
        hi = a * s + b * c;
    } else {
        lo = a;
        hi = b;
    }
}

// block-wide max of a non-negative value plus an "any non-finite" vote
__device__ __forceinline__ float pair_scale(float lo, float hi, float* red, int* flag) {
    const bool nf = !isfinite(lo) || !isfinite(hi);
    const float pm = nf ? 0.0f : fmaxf(fabsf(lo), fabsf(hi));
    if (threadIdx.x == 0) *flag = 0;
    __syncthreads();
    if (nf) atomicExch(flag, 1);
    const float amax = rv::block_max(pm, red);
    const float sc = *flag ? CUDART_NAN_F : rv::row_scale(amax);
    __syncthreads();
    return sc;
}

template <typename T>
__device__ __forceinline__ void rope_fp8kv_body(const T* q_in, const T* k_in, const T* v_in, int in_stride,
                                                uint8_t* q_fp8, uint8_t* k_cache, uint8_t* v_cache,
                                                float* k_scale_cache, float* v_scale_cache, float* q_scale_cache,
                                                const T* cos_t, const T* sin_t, const int* positions,
                                                const int* slot_mapping, int num_tokens, int heads, int kv_heads,
                                                int head_dim, int rotary_dim, int max_positions,
                                                int num_cache_slots) {
    __shared__ float red[33];
    __shared__ int flag;
    rv::pdl_launch();
    rv::pdl_wait();
    const int tok = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int half_head = head_dim / 2, half_rot = rotary_dim / 2;
    if (tok >= num_tokens || (int)blockDim.x != half_head || rotary_dim > head_dim || (rotary_dim & 1)) return;
    const int pos = positions[tok];
    if (pos < 0 || pos >= max_positions) return;

    if (head < heads) {
        float lo, hi;
        rope_pair<T>(q_in + (size_t)tok * in_stride + (size_t)head * head_dim, cos_t, sin_t, pos, tid, half_head,
                     half_rot, lo, hi);
        const float sc = pair_scale(lo, hi, red, &flag);
        if (tid == 0) q_scale_cache[(size_t)tok * heads + head] = sc;
        const float inv = 1.0f / sc;
        uint8_t* o = q_fp8 + ((size_t)tok * heads + head) * head_dim;
        o[tid] = rv::f32_to_e4m3(lo * inv);
        o[tid + half_head] = rv::f32_to_e4m3(hi * inv);
    }
    if (head < kv_heads) {
        const int slot = slot_mapping[tok];
        if (slot < 0 || slot >= num_cache_slots) return;
        const size_t sidx = (size_t)slot * kv_heads + head;
        float klo, khi;
        rope_pair<T>(k_in + (size_t)tok * in_stride + (size_t)head * head_dim, cos_t, sin_t, pos, tid, half_head,
                     half_rot, klo, khi);
        const float ksc = pair_scale(klo, khi, red, &flag);
        const T* vrow = v_in + (size_t)tok * in_stride + (size_t)head * head_dim;
        const float vlo = rv::T16<T>::to_f32(vrow[tid]), vhi = rv::T16<T>::to_f32(vrow[tid + half_head]);
        const float vsc = pair_scale(vlo, vhi, red, &flag);
        if (tid == 0) {
            k_scale_cache[sidx] = ksc;
            v_scale_cache[sidx] = vsc;
        }
        const float kinv = 1.0f / ksc, vinv = 1.0f / vsc;
        uint8_t* ko = k_cache + sidx * head_dim;
        uint8_t* vo = v_cache + sidx * head_dim;
        ko[tid] = rv::f32_to_e4m3(klo * kinv);
        ko[tid + half_head] = rv::f32_to_e4m3(khi * kinv);
        vo[tid] = rv::f32_to_e4m3(vlo * vinv);
        vo[tid + half_head] = rv::f32_to_e4m3(vhi * vinv);
    }
}

}  // namespace

extern "C" __global__ void __launch_bounds__(256)
rvllm_rope_fp8kv_kernel(const __half* q_in, const __half* k_in, const __half* v_in, int in_stride, uint8_t* q_fp8,
                        uint8_t* k_cache, uint8_t* v_cache, float* k_scale_cache, float* v_scale_cache,
                        float* q_scale_cache, const __half* cos_t, const __half* sin_t, const int* positions,
                        const int* slot_mapping, int num_tokens, int heads, int kv_heads, int head_dim,
                        int rotary_dim, int max_positions, int num_cache_slots) {
    rope_fp8kv_body<__half>(q_in, k_in, v_in, in_stride, q_fp8, k_cache, v_cache, k_scale_cache, v_scale_cache,
                            q_scale_cache, cos_t, sin_t, positions, slot_mapping, num_tokens, heads, kv_heads,
                            head_dim, rotary_dim, max_positions, num_cache_slots);
}
extern "C" __global__ void __launch_bounds__(256)
rvllm_rope_fp8kv_bf16_kernel(const __nv_bfloat16* q_in, const __nv_bfloat16* k_in, const __nv_bfloat16* v_in,
                             int in_stride, uint8_t* q_fp8, uint8_t* k_cache, uint8_t* v_cache,
                             float* k_scale_cache, float* v_scale_cache, float* q_scale_cache,
                             const __nv_bfloat16* cos_t, const __nv_bfloat16* sin_t, const int* positions,
                             const int* slot_mapping, int num_tokens, int heads, int kv_heads, int head_dim,
                             int rotary_dim, int max_positions, int num_cache_slots) {
    rope_fp8kv_body<__nv_bfloat16>(q_in, k_in, v_in, in_stride, q_fp8, k_cache, v_cache, k_scale_cache,
                                   v_scale_cache, q_scale_cache, cos_t, sin_t, positions, slot_mapping, num_tokens,
                                   heads, kv_heads, head_dim, rotary_dim, max_positions, num_cache_slots);
}

// Token embedding gather (reference: kernels/embedding_gather_f16.cu): out[t, :] =
// table[token_ids[t], :]; an id outside [0, vocab) yields a zero row.  16-bit rows of either
// activation type; grid = (num_tokens), any block size.
extern "C" __global__ void embedding_gather_f16_kernel(__half* out, const __half* table, const int* token_ids,
                                                       int hidden, int vocab) {
    rv::pdl_launch();
    rv::pdl_wait();
    const int t = blockIdx.x, id = token_ids[t];
    unsigned short* o = reinterpret_cast<unsigned short*>(out) + (size_t)t * hidden;
    const unsigned short* src = reinterpret_cast<const unsigned short*>(table) + (size_t)id * hidden;
    const bool valid = id >= 0 && id < vocab;
    if ((hidden & 7) == 0 && ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(src)) & 15) == 0) {
        for (int v = threadIdx.x; v < (hidden >> 3); v += blockDim.x)
            reinterpret_cast<uint4*>(o)[v] = valid ? rv::ldg128(reinterpret_cast<const uint4*>(src) + v)
                                                   : make_uint4(0, 0, 0, 0);
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = valid ? src[i] : (unsigned short)0;
    }
}
