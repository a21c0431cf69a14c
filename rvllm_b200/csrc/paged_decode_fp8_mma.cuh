// FP8-KV paged GQA decode attention, tensor-core variant of the split-KV main kernel.
//
// Same contract, grid and partial layout as paged_decode_fp8_kernel (paged_decode_fp8.cuh; the
// reference semantics are those of v3/kernels/fp8_decode_v2.cu:199-325,339-624).  What changes is
// where the instructions go.  Streaming 256-512 bytes per token and KV head at HBM speed leaves
// about 45 warp-instructions per token on a B200; dequantising K and forming q.k with FMAs spends
// that whole budget.  Here q.k runs on the FP8 tensor cores directly on the cache bytes:
//
//   * a warp owns tiles of 16 tokens.  K rows are the 16-row operand of mma.sync.m16n8k32.e4m3,
//     the (up to 8) query heads that share the KV head are the 8-column operand, raw E4M3 codes on
//     both sides, f32 accumulation; the per-row scales (q, k, softmax scale) multiply the 16 x 8
//     score tile afterwards.  The K index inside each 64-byte chunk is permuted the same way for
//     both operands (lane t of a quad owns bytes 16t..16t+15), which a dot product does not see.
//   * softmax state (running max per head) is uniform across the warp, updated once per 16-token
//     tile, so the accumulator is rescaled once per tile and only when the max moved.
//   * P.V stays on the FP32 pipes: each lane owns 16 output dims, V is dequantised once per row,
//     and the probability (already multiplied by the row's V scale) arrives by shuffle.
//   * K/V/scales of DEPTH tiles per warp are in flight as cp.async copies into a per-warp ring;
//     every lane reads back exactly the bytes it copied, so the ring needs no barriers.
#pragma once
#include "paged_decode_fp8.cuh"

namespace rvattn {

constexpr int MMA_WARPS = 4;
constexpr int MMA_THREADS = MMA_WARPS * 32;
constexpr int TILE_TOK = 16;

// tiles in flight per warp: shallow on purpose — shared memory per CTA decides how many warps an SM
// holds, and the per-tile dependency chain (MMA -> max -> exp -> P.V) needs many warps to hide
__host__ __device__ constexpr int mma_depth(int hd) { return hd <= 64 ? 4 : 2; }
constexpr int MMA_TBL_MAX = 512;  // staged block-table entries per CTA (longer chunks look the table up in L2)
__host__ __device__ constexpr int mma_stage_bytes(int hd) { return 2 * TILE_TOK * hd + 128; }
__host__ __device__ constexpr size_t mma_smem_bytes(int hd, int gt) {
    return (size_t)MMA_WARPS * mma_depth(hd) * mma_stage_bytes(hd) + MMA_TBL_MAX * sizeof(int) >
                   (size_t)MMA_WARPS * gt * (hd + 2) * sizeof(float)
               ? (size_t)MMA_WARPS * mma_depth(hd) * mma_stage_bytes(hd) + MMA_TBL_MAX * sizeof(int)
               : (size_t)MMA_WARPS * gt * (hd + 2) * sizeof(float);
}

__device__ __forceinline__ void mma_e4m3_16x8x32(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void st_zero16(void* smem) {
    *reinterpret_cast<uint4*>(smem) = make_uint4(0, 0, 0, 0);
}

template <int HD, int GT, typename OutT>
__global__ void __launch_bounds__(MMA_THREADS, (GT <= 2 ? 4 : 3)) paged_decode_fp8_mma_kernel(Params p) {
    static_assert(GT <= 8, "at most 8 query heads per tile (the MMA's column count)");
    constexpr int CH = HD / 64;          // 64-byte chunks per K row
    constexpr int LPR = HD / 16;         // lanes per V row
    constexpr int RPW = 32 / LPR;        // V rows a warp covers per pass
    constexpr int PASSES = TILE_TOK / RPW;
    constexpr int KPIECES = 2 * CH;      // 16-byte K pieces per lane per tile (== PASSES)
    constexpr int DEPTH = mma_depth(HD);
    constexpr int STAGE = mma_stage_bytes(HD);
    constexpr int STEP = MMA_WARPS * TILE_TOK;
    constexpr int PSTRIDE = HD + 2;
    constexpr int NHL = (GT + 1) / 2;    // quad lanes (t) that hold real heads

    extern __shared__ __align__(16) uint8_t sm_raw[];
    float* sm = reinterpret_cast<float*>(sm_raw);
    __shared__ unsigned s_bad;
    rv::pdl_launch();
    rv::pdl_wait();
    const int kvh = blockIdx.x, chunk = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;        // MMA fragment coordinates
    const int unit = lane / LPR, sub = lane % LPR; // P.V coordinates
    const int group = p.heads / p.kv_heads;
    OutT* out = reinterpret_cast<OutT*>(p.out);
    uint8_t* ring = sm_raw + (size_t)warp * DEPTH * STAGE;
    int* tbl = reinterpret_cast<int*>(sm_raw + (size_t)MMA_WARPS * DEPTH * STAGE);

    const int ctx = p.context_lens[b];
    const long long capacity = (long long)p.block_size * p.max_blocks_per_seq;
    if (ctx <= 0 || (p.window_size_left < 0 && (long long)ctx > capacity)) {
        if (chunk != 0) return;
        const float fill = ctx == 0 ? 0.0f : CUDART_NAN_F;
        if (p.force_partial) {
            for (int i = tid; i < group * PSTRIDE; i += MMA_THREADS) {
                const int hh = i / PSTRIDE, d = i % PSTRIDE;
                float* ws = p.workspace + (((size_t)b * p.heads + (size_t)kvh * group + hh) * p.max_chunks) * PSTRIDE;
                ws[d] = d < HD ? fill : (d == HD ? -1e20f : 0.0f);
            }
            return;
        }
        for (int i = tid; i < group * HD; i += MMA_THREADS)
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
    const int first_page = p.bs_shift >= 0 ? (t_begin >> p.bs_shift) : (t_begin / p.block_size);
    const int last_page = p.bs_shift >= 0 ? ((t_end - 1) >> p.bs_shift) : ((t_end - 1) / p.block_size);
    const bool tbl_in_smem = last_page - first_page + 1 <= MMA_TBL_MAX;
    if (tbl_in_smem)
        for (int i = tid; i <= last_page - first_page; i += MMA_THREADS) {
            const int page = first_page + i;
            tbl[i] = __ldg(table + (p.window_size_left >= 0 ? page % p.max_blocks_per_seq : page));
        }
    __syncthreads();

    unsigned bad = 0;
    // cache slot index ((phys * block_size + off) * kv_heads + kvh) of a token, or -1
    auto slot_of = [&](int tok) -> long long {
        const int page = p.bs_shift >= 0 ? (tok >> p.bs_shift) : (tok / p.block_size);
        const int off = tok - page * p.block_size;
        int phys;
        if (tbl_in_smem) {
            phys = tbl[page - first_page];
        } else {
            phys = __ldg(table + (p.window_size_left >= 0 ? page % p.max_blocks_per_seq : page));
        }
        if (phys < 0 || phys >= p.num_blocks_total) {
            bad = 0xffffffffu;
            return -1;
        }
        return ((long long)phys * p.block_size + off) * p.kv_heads + kvh;
    };
    // one tile (16 tokens) of K, V and scales into ring stage (round % DEPTH)
    auto issue = [&](int round) {
        const int tok0 = t_begin + (round * MMA_WARPS + warp) * TILE_TOK;
        uint8_t* st = ring + (size_t)(round % DEPTH) * STAGE;
        if (tok0 < t_end) {
#pragma unroll
            for (int half = 0; half < 2; half++) {  // K rows g and g + 8
                const int tok = tok0 + g + 8 * half;
                const long long sidx = tok < t_end ? slot_of(tok) : -1;
#pragma unroll
                for (int c = 0; c < CH; c++) {
                    uint8_t* dst = st + ((2 * c + half) * 32 + lane) * 16;
                    if (sidx >= 0) cp_async16(dst, p.k_cache + (size_t)sidx * HD + c * 64 + 16 * t);
                    else st_zero16(dst);
                }
                if (t == 0) {
                    float* sc = reinterpret_cast<float*>(st + 2 * TILE_TOK * HD);
                    if (sidx >= 0 && k_perslot) cp_async4(sc + g + 8 * half, p.k_scale_cache + sidx);
                    else sc[g + 8 * half] = k_ds_scalar;
                    if (sidx >= 0 && v_perslot) cp_async4(sc + 16 + g + 8 * half, p.v_scale_cache + sidx);
                    else sc[16 + g + 8 * half] = v_ds_scalar;
                }
            }
#pragma unroll
            for (int ps = 0; ps < PASSES; ps++) {  // V rows
                const int tok = tok0 + ps * RPW + unit;
                const long long sidx = tok < t_end ? slot_of(tok) : -1;
                uint8_t* dst = st + TILE_TOK * HD + (ps * 32 + lane) * 16;
                if (sidx >= 0) cp_async16(dst, p.v_cache + (size_t)sidx * HD + 16 * sub);
                else st_zero16(dst);
            }
        }
        cp_async_commit();
    };
    (void)KPIECES;

    for (int h0 = 0; h0 < group; h0 += GT) {
        const int nh = min(GT, group - h0);
        if (tid == 0) s_bad = 0;
        __syncthreads();
        bad = 0;
        // B operand: raw Q codes of head column g (zero beyond the tile's heads), per 64-byte chunk
        uint4 qf[CH];
        {
            const int head = kvh * group + h0 + (g < nh ? g : 0);
            const uint8_t* qrow = p.q + ((size_t)b * p.heads + head) * HD;
#pragma unroll
            for (int c = 0; c < CH; c++)
                qf[c] = g < nh ? rv::ldg128(qrow + c * 64 + 16 * t) : make_uint4(0, 0, 0, 0);
        }
        // this lane's score columns are heads 2t and 2t+1 of the tile: q scale * softmax scale
        float qsc[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int j = 2 * t + k;
            float v = 0.0f;
            if (j < nh) {
                const int head = kvh * group + h0 + j;
                const float q_ds = p.q_scale_cache ? p.q_scale_cache[(size_t)b * p.heads + head] : *p.q_descale;
                if (bad_scale(q_ds)) bad |= 1u << j;
                v = q_ds * p.scale;
            }
            qsc[k] = v;
        }
        float m[2] = {-1e20f, -1e20f};  // running max of heads 2t, 2t+1 (uniform over g)
        float l[2] = {0.0f, 0.0f};      // this lane's share of the softmax denominators
        float acc[GT][16];
#pragma unroll
        for (int j = 0; j < GT; j++)
#pragma unroll
            for (int d = 0; d < 16; d++) acc[j][d] = 0.0f;

        const int rounds = (t_end - t_begin + STEP - 1) / STEP;
#pragma unroll 1
        for (int r = 0; r < DEPTH; r++) issue(r);
#pragma unroll 1
        for (int r = 0; r < rounds; r++) {
            cp_async_wait<DEPTH - 1>();
            __syncwarp();  // row scales are copied by one lane of a quad and read by its neighbours
            const uint8_t* st = ring + (size_t)(r % DEPTH) * STAGE;
            const int tok0 = t_begin + (r * MMA_WARPS + warp) * TILE_TOK;
            if (tok0 < t_end) {  // warp-uniform: this warp's tile lies inside the chunk
            // ---- scores: 16 tokens x 8 head columns on the tensor cores ----
            float S[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < CH; c++) {
                const uint4 ka = *reinterpret_cast<const uint4*>(st + ((2 * c) * 32 + lane) * 16);
                const uint4 kb = *reinterpret_cast<const uint4*>(st + ((2 * c + 1) * 32 + lane) * 16);
                mma_e4m3_16x8x32(S, ka.x, kb.x, ka.y, kb.y, qf[c].x, qf[c].y);
                mma_e4m3_16x8x32(S, ka.z, kb.z, ka.w, kb.w, qf[c].z, qf[c].w);
            }
            const float* sc = reinterpret_cast<const float*>(st + 2 * TILE_TOK * HD);
            float pv[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // p * v_scale for (token g | g+8, head 2t | 2t+1)
            float e0[2] = {1.0f, 1.0f};
            if (t < NHL) {  // quad lanes that carry real heads
                const bool tv0 = tok0 + g < t_end, tv1 = tok0 + g + 8 < t_end;
                const float kd0 = sc[g], kd1 = sc[g + 8], vd0 = sc[16 + g], vd1 = sc[16 + g + 8];
                if ((tv0 && (bad_scale(kd0) || bad_scale(vd0))) || (tv1 && (bad_scale(kd1) || bad_scale(vd1))))
                    bad = 0xffffffffu;
                float s[4];
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    s[k] = tv0 ? S[k] * qsc[k] * kd0 : -1e30f;
                    s[2 + k] = tv1 ? S[2 + k] * qsc[k] * kd1 : -1e30f;
                    if ((tv0 && !isfinite(s[k])) || (tv1 && !isfinite(s[2 + k]))) bad |= 1u << (2 * t + k);
                }
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    float tm = fmaxf(s[k], s[2 + k]);
                    tm = fmaxf(tm, __shfl_xor_sync(NHL == 4 ? 0xffffffffu : (NHL == 2 ? 0x33333333u : 0x11111111u), tm, 4));
                    tm = fmaxf(tm, __shfl_xor_sync(NHL == 4 ? 0xffffffffu : (NHL == 2 ? 0x33333333u : 0x11111111u), tm, 8));
                    tm = fmaxf(tm, __shfl_xor_sync(NHL == 4 ? 0xffffffffu : (NHL == 2 ? 0x33333333u : 0x11111111u), tm, 16));
                    const float m_new = fmaxf(m[k], tm);
                    e0[k] = __expf(m[k] - m_new);
                    const float p0 = __expf(s[k] - m_new), p1 = __expf(s[2 + k] - m_new);
                    l[k] = l[k] * e0[k] + (p0 + p1);
                    pv[k] = tv0 ? p0 * vd0 : 0.0f;
                    pv[2 + k] = tv1 ? p1 * vd1 : 0.0f;
                    m[k] = m_new;
                }
            }
            __syncwarp();
            // ---- P.V on the FP32 pipes: rescale (only when a max moved), then 16 rows ----
#pragma unroll
            for (int j = 0; j < GT; j++) {
                const float e = __shfl_sync(0xffffffffu, e0[j & 1], j >> 1);
                if (e != 1.0f) {
#pragma unroll
                    for (int d = 0; d < 16; d++) acc[j][d] *= e;
                }
            }
#pragma unroll
            for (int ps = 0; ps < PASSES; ps++) {
                const uint4 vv = *reinterpret_cast<const uint4*>(st + TILE_TOK * HD + (ps * 32 + lane) * 16);
                float vf[16];
                dequant16(vv, vf);
                const int row = ps * RPW + unit;      // token of the tile this lane's V piece belongs to
#pragma unroll
                for (int j = 0; j < GT; j++) {
                    const int src = (row & 7) * 4 + (j >> 1);
                    const bool hi = (ps * RPW) >= 8;  // rows 8..15 live in the second accumulator pair
                    const float w = __shfl_sync(0xffffffffu, hi ? pv[2 + (j & 1)] : pv[j & 1], src);
#pragma unroll
                    for (int d = 0; d < 16; d++) acc[j][d] = fmaf(w, vf[d], acc[j][d]);
                }
            }
            }
            __syncwarp();
            issue(r + DEPTH);  // refill the stage just consumed
        }
        cp_async_wait<0>();

        // ---- reduce inside the warp: V-row groups (sum, the max is shared), denominators over g ----
#pragma unroll
        for (int o = LPR; o < 32; o <<= 1)
#pragma unroll
            for (int j = 0; j < GT; j++)
#pragma unroll
                for (int d = 0; d < 16; d++) acc[j][d] += __shfl_xor_sync(0xffffffffu, acc[j][d], o);
#pragma unroll
        for (int k = 0; k < 2; k++) {
            l[k] += __shfl_xor_sync(0xffffffffu, l[k], 4);
            l[k] += __shfl_xor_sync(0xffffffffu, l[k], 8);
            l[k] += __shfl_xor_sync(0xffffffffu, l[k], 16);
        }
        if (bad) atomicOr(&s_bad, bad);
        __syncthreads();  // every warp is done with its ring before the merge buffer overlays it
#pragma unroll
        for (int j = 0; j < GT; j++) {
            const float mj = __shfl_sync(0xffffffffu, m[j & 1], j >> 1);
            const float lj = __shfl_sync(0xffffffffu, l[j & 1], j >> 1);
            if (unit == 0) {
                float* dst = sm + ((size_t)warp * GT + j) * PSTRIDE;
#pragma unroll
                for (int d = 0; d < 16; d++) dst[16 * sub + d] = acc[j][d];
                if (sub == 0) {
                    dst[HD] = mj;
                    dst[HD + 1] = lj;
                }
            }
        }
        __syncthreads();
        const unsigned bad_mask = s_bad;
        for (int e = tid; e < nh * HD; e += MMA_THREADS) {
            const int j = e / HD, d = e % HD;
            const bool any_bad = (bad_mask >> j) & 1u;
            float M = -1e20f, L = 0.0f, A = 0.0f;
#pragma unroll
            for (int w = 0; w < MMA_WARPS; w++) {
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

}  // namespace rvattn
