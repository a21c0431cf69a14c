// PTX module `flash_attention`: the FP8-KV paged decode entry point that the reference's Gemma
// bring-up selects by name on sm_100 (symbol flash_attention_2_decode_fp8kv_kernel,
// kernels/flash_attention.cu:987-1216; launch geometry fixed by the caller,
// v3/crates/rvllm-attention/src/decode.rs:572-630: grid = (num_seqs, num_heads), block = 128,
// dynamic shared memory sized by the caller's formula, which this kernel does not use).
//
// Contract kept from the reference entry point:
//   * 20-argument list, f16 output [num_seqs, num_heads, head_dim];
//   * block_tables are indexed linearly (page = position / block_size; no ring), every page of
//     [0, context_len) must name a block inside the cache;
//   * nothing is written for: a null pointer, geometry that does not match the launch,
//     context_len <= 0, a context longer than the table, a table entry outside the cache, a
//     non-finite or non-positive scalar scale;
//   * a non-finite / non-positive per-slot scale, or a non-finite score, makes the row NaN;
//   * positions before context_len - 1 - window_size_left do not attend.
// Difference, stated: masked positions are not read at all (the reference decodes them and
// multiplies by zero, so a NaN code in a masked V row reaches its output; here it cannot).
//
// Work decomposition: one CTA per (sequence, query head) as the caller's grid dictates; a warp
// owns every fourth attended token, its lanes cover the head dims in 8-byte pieces, each warp
// keeps its own online-softmax state, and the four states are merged once at the end.  This is
// the compatibility path: the split-KV tcgen05 kernel behind the shared-object ABI is the fast one.
#include <cfloat>

#include "common.cuh"

namespace {

constexpr int FA2_THREADS = 128;
constexpr int FA2_WARPS = FA2_THREADS / 32;
constexpr int MAX_PIECES = 2;  // 8-byte pieces per lane: head_dim <= 512

__device__ __forceinline__ bool good_scale(float s) { return isfinite(s) && s > 0.0f; }

}  // namespace

extern "C" __global__ void __launch_bounds__(FA2_THREADS)
flash_attention_2_decode_fp8kv_kernel(__half* __restrict__ output, const unsigned char* __restrict__ query,
                                      const unsigned char* __restrict__ key_cache,
                                      const unsigned char* __restrict__ value_cache,
                                      const float* __restrict__ k_scale_cache, const float* __restrict__ v_scale_cache,
                                      const float* __restrict__ q_scale_cache,
                                      const float* __restrict__ k_descale_fallback,
                                      const float* __restrict__ v_descale_fallback, const int* __restrict__ block_tables,
                                      const int* __restrict__ context_lens, const float* __restrict__ q_descale,
                                      float scale, int num_heads, int num_kv_heads, int head_dim, int block_size,
                                      int max_blocks_per_seq, int window_size_left, int num_blocks_total) {
    __shared__ int invalid_table;
    __shared__ float merge[FA2_WARPS][512 + 2];
    rv::pdl_launch();
    rv::pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool k_perslot = k_scale_cache != nullptr, v_perslot = v_scale_cache != nullptr;
    if (output == nullptr || query == nullptr || key_cache == nullptr || value_cache == nullptr ||
        block_tables == nullptr || context_lens == nullptr || (q_scale_cache == nullptr && q_descale == nullptr) ||
        (!k_perslot && k_descale_fallback == nullptr) || (!v_perslot && v_descale_fallback == nullptr))
        return;
    if (!(isfinite(scale) && scale > 0.0f) || num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0 ||
        head_dim <= 0 || head_dim > 512 || head_dim % 8 != 0 || block_size <= 0 || max_blocks_per_seq <= 0 ||
        num_blocks_total <= 0 || head >= num_heads || blockDim.x != FA2_THREADS || blockDim.y != 1 || blockDim.z != 1 ||
        gridDim.y != (unsigned)num_heads || gridDim.z != 1 || window_size_left < -1 ||
        (reinterpret_cast<uintptr_t>(key_cache) & 7) != 0 || (reinterpret_cast<uintptr_t>(value_cache) & 7) != 0)
        return;
    const int ctx = context_lens[seq];
    if (ctx <= 0 || (long long)ctx > (long long)max_blocks_per_seq * block_size) return;
    const int* table = block_tables + (long long)seq * max_blocks_per_seq;
    if (tid == 0) invalid_table = 0;
    __syncthreads();
    const int pages = (int)(((long long)ctx + block_size - 1) / block_size);
    for (int page = tid; page < pages; page += FA2_THREADS) {
        const int physical = table[page];
        if (physical < 0 || physical >= num_blocks_total) atomicExch(&invalid_table, 1);
    }
    __syncthreads();
    if (invalid_table) return;

    const int kvh = num_kv_heads == num_heads ? head : head / (num_heads / num_kv_heads);
    const float q_scale = q_scale_cache ? __ldg(q_scale_cache + (long long)seq * num_heads + head) : *q_descale;
    const float k_scalar = k_perslot ? 0.0f : __ldg(k_descale_fallback);
    const float v_scalar = v_perslot ? 0.0f : __ldg(v_descale_fallback);
    if (!good_scale(q_scale) || (!k_perslot && !good_scale(k_scalar)) || (!v_perslot && !good_scale(v_scalar))) return;
    const int start = window_size_left < 0 ? 0 : max(0, ctx - 1 - window_size_left);

    // this lane's query values (already times q_scale * softmax scale), 8 dims per piece
    const int pieces = (head_dim / 8 + 31) / 32;
    float q[MAX_PIECES][8];
#pragma unroll
    for (int pc = 0; pc < MAX_PIECES; pc++) {
        const int d0 = (pc * 32 + lane) * 8;
#pragma unroll
        for (int j = 0; j < 8; j++) q[pc][j] = 0.0f;
        if (pc < pieces && d0 < head_dim) {
            const unsigned char* qb = query + ((long long)seq * num_heads + head) * head_dim + d0;  // no alignment promised
            uint2 raw = make_uint2(0u, 0u);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                raw.x |= (unsigned)qb[j] << (8 * j);
                raw.y |= (unsigned)qb[4 + j] << (8 * j);
            }
            float f[8];
            rv::e4m3x4_to_f32x4(raw.x, f);
            rv::e4m3x4_to_f32x4(raw.y, f + 4);
#pragma unroll
            for (int j = 0; j < 8; j++) q[pc][j] = f[j] * q_scale * scale;
        }
    }
    float m = -FLT_MAX, l = 0.0f;
    float acc[MAX_PIECES][8];
#pragma unroll
    for (int pc = 0; pc < MAX_PIECES; pc++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[pc][j] = 0.0f;
    bool poisoned = false;

    for (int pos = start + warp; pos < ctx; pos += FA2_WARPS) {
        const int page = pos / block_size;
        const long long slot = (long long)table[page] * block_size + (pos - page * block_size);
        const long long row = slot * num_kv_heads + kvh;
        const float ks = k_perslot ? __ldg(k_scale_cache + row) : k_scalar;
        const float vs = v_perslot ? __ldg(v_scale_cache + row) : v_scalar;
        if (!good_scale(ks) || !good_scale(vs)) poisoned = true;
        float dot = 0.0f;
        float vf[MAX_PIECES][8];
#pragma unroll
        for (int pc = 0; pc < MAX_PIECES; pc++) {
            const int d0 = (pc * 32 + lane) * 8;
#pragma unroll
            for (int j = 0; j < 8; j++) vf[pc][j] = 0.0f;
            if (pc < pieces && d0 < head_dim) {
                const uint2 kr = __ldg(reinterpret_cast<const uint2*>(key_cache + row * head_dim + d0));
                const uint2 vr = __ldg(reinterpret_cast<const uint2*>(value_cache + row * head_dim + d0));
                float kf[8];
                rv::e4m3x4_to_f32x4(kr.x, kf);
                rv::e4m3x4_to_f32x4(kr.y, kf + 4);
                rv::e4m3x4_to_f32x4(vr.x, vf[pc]);
                rv::e4m3x4_to_f32x4(vr.y, vf[pc] + 4);
#pragma unroll
                for (int j = 0; j < 8; j++) dot = fmaf(q[pc][j], kf[j], dot);
            }
        }
        const float s = rv::warp_sum(dot) * ks;
        if (!isfinite(s)) {
            poisoned = true;
            continue;
        }
        const float m_new = fmaxf(m, s);
        const float corr = __expf(m - m_new), pr = __expf(s - m_new);
        l = l * corr + pr;
        const float w = pr * vs;
#pragma unroll
        for (int pc = 0; pc < MAX_PIECES; pc++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[pc][j] = fmaf(w, vf[pc][j], acc[pc][j] * corr);
        m = m_new;
    }

    // merge the four warps' states
#pragma unroll
    for (int pc = 0; pc < MAX_PIECES; pc++) {
        const int d0 = (pc * 32 + lane) * 8;
        if (pc < pieces && d0 < head_dim)
#pragma unroll
            for (int j = 0; j < 8; j++) merge[warp][d0 + j] = acc[pc][j];
    }
    if (lane == 0) {
        merge[warp][512] = m;
        merge[warp][513] = poisoned ? CUDART_NAN_F : l;
    }
    __syncthreads();
    for (int d = tid; d < head_dim; d += FA2_THREADS) {
        float M = -FLT_MAX, L = 0.0f, A = 0.0f;
#pragma unroll
        for (int w = 0; w < FA2_WARPS; w++) {
            const float mw = merge[w][512], lw = merge[w][513];
            const float Mn = fmaxf(M, mw);
            const float ea = __expf(M - Mn), eb = __expf(mw - Mn);
            A = A * ea + merge[w][d] * eb;
            L = L * ea + lw * eb;  // a poisoned warp carries NaN here
            M = Mn;
        }
        const float inv = isfinite(L) && L > 0.0f ? 1.0f / L : CUDART_NAN_F;
        output[((long long)seq * num_heads + head) * head_dim + d] = __float2half(A * inv);
    }
}
