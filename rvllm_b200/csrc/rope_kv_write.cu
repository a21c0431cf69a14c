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

// |lo|, |hi| -> their max, or +inf when either is not finite (an absmax of finite values is never
// +inf, so the reduction below carries the "any non-finite" vote in the same number)
__device__ __forceinline__ float pair_amax(float lo, float hi) {
    return (!isfinite(lo) || !isfinite(hi)) ? CUDART_INF_F : fmaxf(fabsf(lo), fabsf(hi));
}
__device__ __forceinline__ float scale_of(float amax) { return isinf(amax) ? CUDART_NAN_F : rv::row_scale(amax); }

// One CTA per (token, head): Q head `head` and, while head < kv_heads, K and V head `head`.  Every
// global load is issued before the first reduction, and the three absmax reductions share one pass
// and one barrier, so a CTA pays two dependent memory round trips (position -> cos/sin) instead of
// one per operand.
template <typename T>
__device__ __forceinline__ void rope_fp8kv_body(const T* q_in, const T* k_in, const T* v_in, long long q_stride,
                                                long long kv_stride, uint8_t* q_fp8, uint8_t* k_cache, uint8_t* v_cache,
                                                float* k_scale_cache, float* v_scale_cache, float* q_scale_cache,
                                                const float* q_scale_ptr, const T* cos_t, const T* sin_t,
                                                const int* positions, const int* slot_mapping, int num_tokens,
                                                int heads, int kv_heads, int head_dim, int rotary_dim,
                                                int max_positions, int num_cache_slots) {
    __shared__ float red[8][3];
    rv::pdl_launch();
    rv::pdl_wait();
    const int tok = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int half_head = head_dim / 2, half_rot = rotary_dim / 2;
    if (tok >= num_tokens || (int)blockDim.x != half_head || rotary_dim > head_dim || (rotary_dim & 1)) return;
    const int pos = positions[tok];
    const int slot = slot_mapping[tok];
    const bool do_q = head < heads;
    const bool do_kv = head < kv_heads && slot >= 0 && slot < num_cache_slots;
    float qa = 0.0f, qb = 0.0f, ka = 0.0f, kb = 0.0f, va = 0.0f, vb = 0.0f;
    if (do_q) {
        const T* row = q_in + (size_t)tok * q_stride + (size_t)head * head_dim;
        qa = rv::T16<T>::to_f32(row[tid]);
        qb = rv::T16<T>::to_f32(row[tid + half_head]);
    }
    if (do_kv) {
        const T* krow = k_in + (size_t)tok * kv_stride + (size_t)head * head_dim;
        const T* vrow = v_in + (size_t)tok * kv_stride + (size_t)head * head_dim;
        ka = rv::T16<T>::to_f32(krow[tid]);
        kb = rv::T16<T>::to_f32(krow[tid + half_head]);
        va = rv::T16<T>::to_f32(vrow[tid]);
        vb = rv::T16<T>::to_f32(vrow[tid + half_head]);
    }
    if (pos < 0 || pos >= max_positions) return;
    float qlo = qa, qhi = qb, klo = ka, khi = kb;
    if (tid < half_rot) {
        const float c = rv::T16<T>::to_f32(cos_t[(size_t)pos * half_rot + tid]);
        const float s = rv::T16<T>::to_f32(sin_t[(size_t)pos * half_rot + tid]);
        qlo = qa * c - qb * s;
        qhi = qa * s + qb * c;
        klo = ka * c - kb * s;
        khi = ka * s + kb * c;
    }
    float mq = rv::warp_max(pair_amax(qlo, qhi)), mk = rv::warp_max(pair_amax(klo, khi)),
          mv = rv::warp_max(pair_amax(va, vb));
    const int warp = tid >> 5, nwarps = ((int)blockDim.x + 31) >> 5;
    if ((tid & 31) == 0) {
        red[warp][0] = mq;
        red[warp][1] = mk;
        red[warp][2] = mv;
    }
    __syncthreads();
    mq = mk = mv = 0.0f;
    for (int w = 0; w < nwarps; w++) {
        mq = fmaxf(mq, red[w][0]);
        mk = fmaxf(mk, red[w][1]);
        mv = fmaxf(mv, red[w][2]);
    }
    if (do_q) {
        // dynamic per-(token, head) scale, or — when the caller keeps no scale cache — the static *q_scale_ptr
        float sc;
        if (q_scale_cache) {
            sc = scale_of(mq);
            if (tid == 0) q_scale_cache[(size_t)tok * heads + head] = sc;
        } else {
            sc = *q_scale_ptr;
            if (!isfinite(sc) || sc <= 0.0f) sc = CUDART_NAN_F;
        }
        const float inv = 1.0f / sc;
        uint8_t* o = q_fp8 + ((size_t)tok * heads + head) * head_dim;
        o[tid] = rv::f32_to_e4m3(qlo * inv);
        o[tid + half_head] = rv::f32_to_e4m3(qhi * inv);
    }
    if (do_kv) {
        const size_t sidx = (size_t)slot * kv_heads + head;
        const float ksc = scale_of(mk), vsc = scale_of(mv);
        if (tid == 0) {
            k_scale_cache[sidx] = ksc;
            v_scale_cache[sidx] = vsc;
        }
        const float kinv = 1.0f / ksc, vinv = 1.0f / vsc;
        uint8_t* ko = k_cache + sidx * head_dim;
        uint8_t* vo = v_cache + sidx * head_dim;
        ko[tid] = rv::f32_to_e4m3(klo * kinv);
        ko[tid + half_head] = rv::f32_to_e4m3(khi * kinv);
        vo[tid] = rv::f32_to_e4m3(va * vinv);
        vo[tid + half_head] = rv::f32_to_e4m3(vb * vinv);
    }
}

}  // namespace

extern "C" __global__ void __launch_bounds__(256)
rvllm_rope_fp8kv_kernel(const __half* q_in, const __half* k_in, const __half* v_in, int in_stride, uint8_t* q_fp8,
                        uint8_t* k_cache, uint8_t* v_cache, float* k_scale_cache, float* v_scale_cache,
                        float* q_scale_cache, const __half* cos_t, const __half* sin_t, const int* positions,
                        const int* slot_mapping, int num_tokens, int heads, int kv_heads, int head_dim,
                        int rotary_dim, int max_positions, int num_cache_slots) {
    rope_fp8kv_body<__half>(q_in, k_in, v_in, in_stride, in_stride, q_fp8, k_cache, v_cache, k_scale_cache,
                            v_scale_cache, q_scale_cache, nullptr, cos_t, sin_t, positions, slot_mapping, num_tokens,
                            heads, kv_heads, head_dim, rotary_dim, max_positions, num_cache_slots);
}
extern "C" __global__ void __launch_bounds__(256)
rvllm_rope_fp8kv_bf16_kernel(const __nv_bfloat16* q_in, const __nv_bfloat16* k_in, const __nv_bfloat16* v_in,
                             int in_stride, uint8_t* q_fp8, uint8_t* k_cache, uint8_t* v_cache,
                             float* k_scale_cache, float* v_scale_cache, float* q_scale_cache,
                             const __nv_bfloat16* cos_t, const __nv_bfloat16* sin_t, const int* positions,
                             const int* slot_mapping, int num_tokens, int heads, int kv_heads, int head_dim,
                             int rotary_dim, int max_positions, int num_cache_slots) {
    rope_fp8kv_body<__nv_bfloat16>(q_in, k_in, v_in, in_stride, in_stride, q_fp8, k_cache, v_cache, k_scale_cache,
                                   v_scale_cache, q_scale_cache, nullptr, cos_t, sin_t, positions, slot_mapping,
                                   num_tokens, heads, kv_heads, head_dim, rotary_dim, max_positions, num_cache_slots);
}

// The reference's own entry point and argument list (v3/kernels/fused_rope_partial_fp8kv.cu:54-76; launcher
// FusedRopePartialFp8KvLaunch, v3/crates/rvllm-fused/src/gemma4_launcher.rs:248-400): compact
// [tokens, heads, head_dim] Q and [tokens, kv_heads, head_dim] K / V inputs, and a static Q scale read from
// q_scale_ptr when q_scale_cache is null.  grid (tokens, max(heads, kv_heads)), block head_dim / 2.
extern "C" __global__ void __launch_bounds__(256)
fused_rope_partial_fp8kv_kernel(const __half* q_in, const __half* k_in, const __half* v_in, uint8_t* q_fp8_out,
                                uint8_t* key_cache, uint8_t* value_cache, float* k_scale_cache, float* v_scale_cache,
                                float* q_scale_cache, const __half* cos_table, const __half* sin_table,
                                const int* positions, const int* slot_mapping, const float* q_scale_ptr, int num_tokens,
                                int num_heads, int num_kv_heads, int head_dim, int rotary_dim, int max_positions,
                                int num_cache_slots) {
    if (!q_in || !q_fp8_out || !positions || num_tokens <= 0 || num_heads <= 0 || num_kv_heads < 0 || head_dim < 64 ||
        head_dim % 64 != 0 || rotary_dim < 0 || max_positions <= 0 || (rotary_dim > 0 && (!cos_table || !sin_table)) ||
        (!q_scale_cache && !q_scale_ptr) ||
        (num_kv_heads > 0 && (!k_in || !v_in || !key_cache || !value_cache || !k_scale_cache || !v_scale_cache ||
                              !slot_mapping || num_cache_slots <= 0)) ||
        (int)blockIdx.y >= (num_heads > num_kv_heads ? num_heads : num_kv_heads) || blockDim.y != 1 || blockDim.z != 1 ||
        gridDim.z != 1)
        return;
    rope_fp8kv_body<__half>(q_in, k_in, v_in, (long long)num_heads * head_dim, (long long)num_kv_heads * head_dim,
                            q_fp8_out, key_cache, value_cache, k_scale_cache, v_scale_cache, q_scale_cache, q_scale_ptr,
                            cos_table, sin_table, positions, num_kv_heads > 0 ? slot_mapping : positions, num_tokens,
                            num_heads, num_kv_heads, head_dim, rotary_dim, max_positions,
                            num_kv_heads > 0 ? num_cache_slots : 0);
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
