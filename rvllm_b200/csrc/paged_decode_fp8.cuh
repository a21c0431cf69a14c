// FP8-KV paged GQA decode attention: split-KV partials + log-sum-exp combine.
//
// Semantics follow the reference's split-KV decode (v3/kernels/fp8_decode_v2.cu:339-671)
// and its scalar definition (:199-325):
//   * Q [batch, heads, HD] fp8 with a per-(seq, head) scale (or one scalar), K/V caches
//     [num_blocks, block_size, kv_heads, HD] fp8 with per-(slot, kv_head) scales (or scalars);
//   * attended interval = last (window_size_left + 1) tokens of the context when a window is
//     set; sliding layers index the block table as a ring (page % max_blocks_per_seq);
//   * ctx == 0 -> zeros; ctx < 0, a context longer than the table (no window), a physical
//     block outside [0, num_blocks_total) or a non-finite / non-positive scale -> NaN row;
//     never a fault;
//   * f32 online softmax started at m = -1e20 with __expf; partials (acc[HD], m, l) per
//     chunk in workspace [batch][heads][max_chunks][HD + 2]; combine walks chunks in order.
//
// What is different from the reference kernel is the work decomposition: the number of
// chunks a sequence is cut into depends on its own attended length (one chunk per
// MIN_CHUNK_TOKENS, at most max_chunks), so a 32k-token row spreads over many CTAs while
// a 512-token row does not pay for empty ones, and max_chunks is sized from the SM count.
// grid = (kv_heads, max_chunks, batch), 256 threads.  All q-heads of a KV head share every
// K/V row fetched (16-byte streaming loads, HD/16 lanes per row, several rows in flight
// per warp); lanes of a row reduce q.k with shuffles; row groups of a warp, then warps,
// merge their online-softmax states once at the end.
#pragma once
#include "common.cuh"

namespace rvattn {

constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;
constexpr int MIN_CHUNK_TOKENS = 256;
constexpr int MAX_CHUNKS = 32;
constexpr int TARGET_CTAS = 148 * 2;  // measured: more, smaller CTAs only add merge work
constexpr int DEPTH = 8;            // cp.async rounds in flight per warp
constexpr int STAGE_BYTES = 1088;   // 32 lanes x 16 B of K, the same of V, 8 + 8 row scales
constexpr int TBL_MAX = 2048;       // block-table entries staged in shared memory per CTA

__host__ __device__ constexpr size_t smem_bytes(int hd, int gt) {
    return (size_t)WARPS * DEPTH * STAGE_BYTES + TBL_MAX * sizeof(int) >
                   (size_t)WARPS * gt * (hd + 2) * sizeof(float)
               ? (size_t)WARPS * DEPTH * STAGE_BYTES + TBL_MAX * sizeof(int)
               : (size_t)WARPS * gt * (hd + 2) * sizeof(float);
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem)
                 : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

struct Params {
    const uint8_t* q;
    const uint8_t* k_cache;
    const uint8_t* v_cache;
    void* out;
    float* workspace;
    const int* block_tables;
    const int* context_lens;
    const float* k_scale_cache;
    const float* v_scale_cache;
    const float* q_scale_cache;
    const float* q_descale;
    const float* k_descale;
    const float* v_descale;
    float scale;
    int batch, heads, kv_heads;
    int block_size, bs_shift;  // bs_shift = log2(block_size) or -1
    int max_blocks_per_seq, num_blocks_total, window_size_left;
    int max_chunks;
    int min_chunk_tokens;  // a sequence is cut into ceil(attended / this) chunks, at most max_chunks
    int force_partial;     // always leave partials in the workspace (the fused combine+quant pass reads them)
    float* amax_out;       // tcgen05 kernel, 16-bit output: max |rounded output| per (sequence, kv_head), or null
    int early_meta;        // tcgen05 kernel: context lengths and block tables were written before the preceding kernel
                           // started (only the newest token's K/V, its scales and Q come from it): geometry, table
                           // look-ups and the loads of every tile but the last do not wait for that kernel
    int cluster_combine;   // tcgen05 kernel: the chunks of a (sequence, kv_head) are one thread-block cluster and the
                           // chunk-0 CTA merges their partials out of its own shared memory (no workspace, no combine launch)
};

// Upper bound on chunks per sequence for a launch shape; the workspace-size query and the
// launch both use it, so they always agree.
inline int pick_max_chunks(int batch, int kv_heads, int target_ctas = TARGET_CTAS) {
    long long d = (long long)batch * kv_heads;
    if (d <= 0) return 0;
    long long c = (target_ctas + d - 1) / d;
    if (c < 1) c = 1;
    if (c > MAX_CHUNKS) c = MAX_CHUNKS;
    return (int)c;
}

__device__ __forceinline__ void attend_interval(int ctx, int window, int& start, int& len) {
    start = 0;
    len = ctx;
    if (window >= 0 && len > window + 1) {
        len = window + 1;
        start = ctx - len;
    }
}
__device__ __forceinline__ int chunks_for(int attend_len, int max_chunks, int min_tokens) {
    int c = (attend_len + min_tokens - 1) / min_tokens;
    c = c < 1 ? 1 : c;
    return c < max_chunks ? c : max_chunks;
}
__device__ __forceinline__ bool bad_scale(float s) { return !isfinite(s) || s <= 0.0f; }

__device__ __forceinline__ void dequant16(const uint4& v, float* f) {
    rv::e4m3x4_to_f32x4(v.x, f);
    rv::e4m3x4_to_f32x4(v.y, f + 4);
    rv::e4m3x4_to_f32x4(v.z, f + 8);
    rv::e4m3x4_to_f32x4(v.w, f + 12);
}

template <int HD, int GT, typename OutT>
__global__ void __launch_bounds__(THREADS) paged_decode_fp8_kernel(Params p) {
    constexpr int LPR = HD / 16;    // lanes per K/V row
    constexpr int RPW = 32 / LPR;   // rows a warp covers per step
    constexpr int STEP = WARPS * RPW;
    constexpr int PSTRIDE = HD + 2;
    // dynamic shared memory: per-warp cp.async ring [WARPS][DEPTH][STAGE_BYTES], then the staged
    // block table [TBL_MAX]; after the stream the ring is reused as the merge buffer
    // [WARPS][GT][HD + 2] f32.
    extern __shared__ __align__(16) uint8_t sm_raw[];
    float* sm = reinterpret_cast<float*>(sm_raw);
    uint8_t* ring = sm_raw + (size_t)(threadIdx.x >> 5) * DEPTH * STAGE_BYTES;
    int* tbl = reinterpret_cast<int*>(sm_raw + (size_t)WARPS * DEPTH * STAGE_BYTES);
    __shared__ unsigned s_bad;  // bit j: q-head j of the tile is invalid; all ones: the whole KV head is

    rv::pdl_launch();
    rv::pdl_wait();
    const int kvh = blockIdx.x, chunk = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int unit = lane / LPR, sub = lane % LPR;
    const int group = p.heads / p.kv_heads;
    OutT* out = reinterpret_cast<OutT*>(p.out);

    const int ctx = p.context_lens[b];
    const long long capacity = (long long)p.block_size * p.max_blocks_per_seq;
    if (ctx <= 0 || (p.window_size_left < 0 && (long long)ctx > capacity)) {
        if (chunk != 0) return;
        const float fill = ctx == 0 ? 0.0f : CUDART_NAN_F;
        if (p.force_partial) {
            for (int i = tid; i < group * PSTRIDE; i += THREADS) {
                const int hh = i / PSTRIDE, d = i % PSTRIDE;
                float* ws = p.workspace + (((size_t)b * p.heads + (size_t)kvh * group + hh) * p.max_chunks) * PSTRIDE;
                ws[d] = d < HD ? fill : (d == HD ? -1e20f : 0.0f);
            }
            return;
        }
        for (int i = tid; i < group * HD; i += THREADS)
            out[((size_t)b * p.heads + (size_t)kvh * group) * HD + i] = rv::T16<OutT>::from_f32(fill);
        return;
    }
    int start, len;
    attend_interval(ctx, p.window_size_left, start, len);
    const int nchunks = chunks_for(len, p.max_chunks, p.min_chunk_tokens);
    if (chunk >= nchunks) return;
    const int chunk_size = (len + nchunks - 1) / nchunks;
    const int t_begin = start + chunk * chunk_size;
    const int t_end = min(t_begin + chunk_size, start + len);
    const bool k_perslot = p.k_scale_cache != nullptr, v_perslot = p.v_scale_cache != nullptr;
    const float k_ds_scalar = k_perslot ? 0.0f : *p.k_descale;
    const float v_ds_scalar = v_perslot ? 0.0f : *p.v_descale;
    const int* table = p.block_tables + (size_t)b * p.max_blocks_per_seq;
    // stage this chunk's slice of the block table (ring-mapped for sliding layers)
    const int first_page = p.bs_shift >= 0 ? (t_begin >> p.bs_shift) : (t_begin / p.block_size);
    const int last_page = p.bs_shift >= 0 ? ((t_end - 1) >> p.bs_shift) : ((t_end - 1) / p.block_size);
    const bool tbl_in_smem = last_page - first_page + 1 <= TBL_MAX;
    if (tbl_in_smem)
        for (int i = tid; i <= last_page - first_page; i += THREADS) {
            const int page = first_page + i;
            tbl[i] = __ldg(table + (p.window_size_left >= 0 ? page % p.max_blocks_per_seq : page));
        }
    __syncthreads();

    for (int h0 = 0; h0 < group; h0 += GT) {
        const int nh = min(GT, group - h0);
        if (tid == 0) s_bad = 0;
        __syncthreads();
        float q[GT][16];
        unsigned bad = 0;
#pragma unroll
        for (int j = 0; j < GT; j++) {
            const int head = kvh * group + h0 + (j < nh ? j : 0);
            const float q_ds = p.q_scale_cache ? p.q_scale_cache[(size_t)b * p.heads + head] : *p.q_descale;
            if (bad_scale(q_ds)) bad |= 1u << j;
            const uint4 qv = rv::ldg128(p.q + ((size_t)b * p.heads + head) * HD + 16 * sub);
            dequant16(qv, q[j]);
#pragma unroll
            for (int d = 0; d < 16; d++) q[j][d] *= q_ds;
        }
        float m[GT], l[GT], acc[GT][16];
#pragma unroll
        for (int j = 0; j < GT; j++) {
            m[j] = -1e20f;
            l[j] = 0.0f;
#pragma unroll
            for (int d = 0; d < 16; d++) acc[j][d] = 0.0f;
        }

        // ---- pipelined K/V stream: DEPTH rounds of cp.async in flight per warp -------------
        auto issue = [&](int round) {
            const int tok = t_begin + (round * WARPS + warp) * RPW + unit;
            uint8_t* st = ring + (size_t)(round % DEPTH) * STAGE_BYTES;
            if (tok < t_end) {
                const int page = p.bs_shift >= 0 ? (tok >> p.bs_shift) : (tok / p.block_size);
                const int off = tok - page * p.block_size;
                int phys;
                if (tbl_in_smem) {
                    phys = tbl[page - first_page];
                } else {
                    const int tpage = p.window_size_left >= 0 ? page % p.max_blocks_per_seq : page;
                    phys = __ldg(table + tpage);
                }
                if (phys < 0 || phys >= p.num_blocks_total) {
                    bad = 0xffffffffu;
                } else {
                    const size_t sidx = ((size_t)phys * p.block_size + off) * p.kv_heads + kvh;
                    cp_async16(st + lane * 16, p.k_cache + sidx * HD + 16 * sub);
                    cp_async16(st + 512 + lane * 16, p.v_cache + sidx * HD + 16 * sub);
                    if (k_perslot && sub == 0) cp_async4(st + 1024 + unit * 4, p.k_scale_cache + sidx);
                    if (v_perslot && sub == 1) cp_async4(st + 1024 + 32 + unit * 4, p.v_scale_cache + sidx);
                }
            }
            cp_async_commit();
        };
        const int rounds = (t_end - t_begin + STEP - 1) / STEP;
#pragma unroll 1
        for (int r = 0; r < DEPTH; r++) issue(r);
#pragma unroll 1
        for (int r = 0; r < rounds; r++) {
            cp_async_wait<DEPTH - 1>();
            __syncwarp();
            const uint8_t* st = ring + (size_t)(r % DEPTH) * STAGE_BYTES;
            const int tok = t_begin + (r * WARPS + warp) * RPW + unit;
            const bool ok = tok < t_end;
            const uint4 kv = *reinterpret_cast<const uint4*>(st + lane * 16);
            const uint4 vv = *reinterpret_cast<const uint4*>(st + 512 + lane * 16);
            const float ks = k_perslot ? *reinterpret_cast<const float*>(st + 1024 + unit * 4) : k_ds_scalar;
            const float vs = v_perslot ? *reinterpret_cast<const float*>(st + 1024 + 32 + unit * 4) : v_ds_scalar;
            __syncwarp();
            issue(r + DEPTH);  // refill the stage just read
            float kf[16];
            dequant16(kv, kf);
            float dot[GT];
#pragma unroll
            for (int j = 0; j < GT; j++) {
                float acc_s = 0.0f;
#pragma unroll
                for (int d = 0; d < 16; d++) acc_s = fmaf(q[j][d], kf[d], acc_s);
                dot[j] = acc_s;
            }
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1)
#pragma unroll
                for (int j = 0; j < GT; j++) dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], o);
            if (ok && bad != 0xffffffffu) {
                if (bad_scale(ks) || bad_scale(vs)) bad = 0xffffffffu;
                float vf[16];
                dequant16(vv, vf);
                const float kscale = ks * p.scale;
#pragma unroll
                for (int j = 0; j < GT; j++) {
                    const float qk = dot[j] * kscale;
                    if (!isfinite(qk)) bad |= 1u << j;
                    const float m_new = fmaxf(m[j], qk);
                    const float e0 = __expf(m[j] - m_new);
                    const float e1 = __expf(qk - m_new);
                    const float ev = e1 * vs;
#pragma unroll
                    for (int d = 0; d < 16; d++) acc[j][d] = fmaf(ev, vf[d], acc[j][d] * e0);
                    l[j] = l[j] * e0 + e1;
                    m[j] = m_new;
                }
            }
        }
        cp_async_wait<0>();
        __syncthreads();  // every warp is done with its ring before the merge buffer overlays it

        // merge the row groups of this warp (same sub-lane, different unit)
#pragma unroll
        for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
            for (int j = 0; j < GT; j++) {
                const float mo = __shfl_xor_sync(0xffffffffu, m[j], o);
                const float lo = __shfl_xor_sync(0xffffffffu, l[j], o);
                const float M = fmaxf(m[j], mo);
                const float ea = __expf(m[j] - M), eb = __expf(mo - M);
#pragma unroll
                for (int d = 0; d < 16; d++) {
                    const float ao = __shfl_xor_sync(0xffffffffu, acc[j][d], o);
                    acc[j][d] = acc[j][d] * ea + ao * eb;
                }
                l[j] = l[j] * ea + lo * eb;
                m[j] = M;
            }
        }
        if (bad) atomicOr(&s_bad, bad);
        if (unit == 0) {
#pragma unroll
            for (int j = 0; j < GT; j++) {
                float* dst = sm + ((size_t)warp * GT + j) * PSTRIDE;
#pragma unroll
                for (int d = 0; d < 16; d++) dst[16 * sub + d] = acc[j][d];
                if (sub == 0) {
                    dst[HD] = m[j];
                    dst[HD + 1] = l[j];
                }
            }
        }
        __syncthreads();
        const unsigned bad_mask = s_bad;
        // merge warps in order; thread (j, d) pairs are dealt round-robin
        for (int e = tid; e < nh * HD; e += THREADS) {
            const int j = e / HD, d = e % HD;
            const bool any_bad = (bad_mask >> j) & 1u;
            float M = -1e20f, L = 0.0f, A = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; w++) {
                const float* src = sm + ((size_t)w * GT + j) * PSTRIDE;
                const float mw = src[HD], lw = src[HD + 1];
                const float Mn = fmaxf(M, mw);
                const float ea = __expf(M - Mn), eb = __expf(mw - Mn);
                A = A * ea + src[d] * eb;
                L = L * ea + lw * eb;
                M = Mn;
            }
            const int head = kvh * group + h0 + j;
            if (nchunks == 1 && !p.force_partial) {
                float v = L > 0.0f ? A / L : A;
                if (any_bad) v = CUDART_NAN_F;
                out[((size_t)b * p.heads + head) * HD + d] = rv::T16<OutT>::from_f32(v);
            } else {
                float* ws = p.workspace + (((size_t)b * p.heads + head) * p.max_chunks + chunk) * PSTRIDE;
                ws[d] = any_bad ? CUDART_NAN_F : A;
                if (d == 0) {
                    ws[HD] = M;
                    ws[HD + 1] = any_bad ? CUDART_NAN_F : L;
                }
            }
        }
        __syncthreads();
    }
}

// grid = (batch * heads), block = min(HD, 256): LSE merge of a sequence's chunks.
template <int HD, typename OutT>
__global__ void paged_decode_fp8_combine_kernel(const float* __restrict__ workspace, OutT* __restrict__ out,
                                                const int* __restrict__ context_lens, int heads, int block_size,
                                                int max_blocks_per_seq, int window_size_left, int max_chunks,
                                                int min_chunk_tokens) {
    constexpr int PSTRIDE = HD + 2;
    rv::pdl_launch();
    rv::pdl_wait();
    const int bh = blockIdx.x, b = bh / heads;
    const int ctx = context_lens[b];
    if (ctx <= 0 || (window_size_left < 0 && (long long)ctx > (long long)block_size * max_blocks_per_seq)) return;
    int start, len;
    attend_interval(ctx, window_size_left, start, len);
    const int nchunks = chunks_for(len, max_chunks, min_chunk_tokens);
    if (nchunks <= 1) return;  // the main kernel already wrote the row
    const float* ws = workspace + (size_t)bh * max_chunks * PSTRIDE;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float M = -1e20f, L = 0.0f, A = 0.0f;
        for (int c = 0; c < nchunks; c++) {
            const float* src = ws + (size_t)c * PSTRIDE;
            const float mc = src[HD], lc = src[HD + 1];
            const float Mn = fmaxf(M, mc);
            const float ea = __expf(M - Mn), eb = __expf(mc - Mn);
            A = A * ea + src[d] * eb;
            L = L * ea + lc * eb;
            M = Mn;
        }
        out[(size_t)bh * HD + d] = rv::T16<OutT>::from_f32(L > 0.0f ? A / L : A);
    }
}

// Fused epilogue of a decode-attention call: LSE-combine every head of one token, round to the
// 16-bit activation type (so the bytes equal those of combine -> store -> quantize), then the
// per-token FP8 quantisation of the whole [heads * HD] row (reference: QuantizeFp8PerTokenLaunch
// after the attention launch, v3/crates/rvllm-runtime/src/layer_exec.rs:425).  grid = (batch),
// 512 threads, heads * HD floats of dynamic shared memory.  The main kernel ran with
// force_partial, so every (head, chunk) partial is in the workspace.
template <int HD, typename OutT>
__global__ void __launch_bounds__(512)
paged_decode_fp8_combine_quant_kernel(const float* __restrict__ workspace, uint8_t* __restrict__ out_fp8,
                                      float* __restrict__ out_scale, const int* __restrict__ context_lens, int heads,
                                      int block_size, int max_blocks_per_seq, int window_size_left, int max_chunks,
                                      int min_chunk_tokens) {
    constexpr int PSTRIDE = HD + 2;
    extern __shared__ __align__(16) float row[];  // [heads * HD]
    __shared__ float red[33];
    rv::pdl_launch();
    rv::pdl_wait();
    const int b = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const int ctx = context_lens[b];
    int nchunks = 1;
    if (!(ctx <= 0 || (window_size_left < 0 && (long long)ctx > (long long)block_size * max_blocks_per_seq))) {
        int start, len;
        attend_interval(ctx, window_size_left, start, len);
        nchunks = chunks_for(len, max_chunks, min_chunk_tokens);
    }
    const int dim = heads * HD;
    float amax = 0.0f;
    for (int e = tid; e < dim; e += nt) {
        const int h = e / HD, d = e % HD;
        const float* ws = workspace + ((size_t)b * heads + h) * max_chunks * PSTRIDE;
        float M = -1e20f, L = 0.0f, A = 0.0f;
        for (int c = 0; c < nchunks; c++) {
            const float* src = ws + (size_t)c * PSTRIDE;
            const float mc = src[HD], lc = src[HD + 1];
            const float Mn = fmaxf(M, mc);
            const float ea = __expf(M - Mn), eb = __expf(mc - Mn);
            A = A * ea + src[d] * eb;
            L = L * ea + lc * eb;
            M = Mn;
        }
        const float v = rv::T16<OutT>::to_f32(rv::T16<OutT>::from_f32(L > 0.0f ? A / L : A));
        row[e] = v;
        amax = fmaxf(amax, fabsf(v));
    }
    amax = rv::block_max(amax, red);
    const float scale = rv::row_scale(amax);
    if (tid == 0) out_scale[b] = scale;
    const float inv = 1.0f / scale;
    uint8_t* o = out_fp8 + (size_t)b * dim;
    for (int v4 = tid; v4 < dim / 4; v4 += nt) {
        const float4 f = reinterpret_cast<const float4*>(row)[v4];
        reinterpret_cast<uint32_t*>(o)[v4] = rv::f32x4_to_e4m3x4(f.x * inv, f.y * inv, f.z * inv, f.w * inv);
    }
}

}  // namespace rvattn
