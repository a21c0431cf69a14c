// FP8-KV paged GQA decode attention with both products on the tensor cores.
//
// Same contract, grid, chunk rule and partial layout as paged_decode_fp8_kernel
// (paged_decode_fp8.cuh; reference semantics: v3/kernels/fp8_decode_v2.cu:199-325,339-624).
// Profiling the score-only tensor-core kernel (paged_decode_fp8_mma.cuh) showed it bound by
// instruction issue, not by HBM: dequantising V and the P.V FMAs cost ~60 warp-instructions per
// token and KV head where the memory system leaves room for ~20.  Here P.V is an MMA as well:
//
//   * scores: as before, K rows (16 tokens) x the query heads of the KV head, raw E4M3 codes on both
//     sides of mma.sync.m16n8k32.e4m3, scales applied to the 16 x 8 score tile afterwards.
//   * P.V: out^T[dims x heads] += V^T[dims x 16 tokens] . P[16 tokens x heads] with
//     mma.sync.m16n8k16.f16: V is the 16-row operand.  An E4M3 code is exact in f16, so the only
//     rounding is the probability (already multiplied by the token's V scale) to f16, 2^-11 relative;
//     accumulation stays f32.  Row r of V tile i stands for head dim r*(HD/16)+i: with that
//     permutation of the output dims a lane needs, of each token row, HD/16 *contiguous* bytes, so V
//     is fetched with the same few wide copies as before and one byte-permute pairs the codes of two
//     tokens for the converter (cvt.f16x2.e4m3x2).  Cost per 16 tokens and 16 dims: 4 permutes,
//     4 converts, 1 MMA.
//   * the probabilities leave the score MMA as (token, head) fragments and enter the second MMA as
//     (head, token) fragments: four shuffles of packed f16 pairs per tile.
//   * every (dim, head) of the accumulator lives in exactly one lane, so a warp needs no reduction
//     at the end; softmax state is per warp, merged over the CTA's warps through shared memory.
//   * cache-slot indices are computed once per token (one lane each) and handed round by shuffle.
#pragma once
#include <type_traits>
#include "paged_decode_fp8_mma.cuh"

namespace rvattn {

// cp.async of BYTES (4, 8 or 16) with compile-time offsets folded into both address operands
template <int BYTES, int SOFF, int GOFF>
__device__ __forceinline__ void cp_async_off(uint32_t smem_base, const void* gmem_base) {
    if constexpr (BYTES == 16)
        asm volatile("cp.async.cg.shared.global [%0 + %2], [%1 + %3], 16;" ::"r"(smem_base), "l"(gmem_base), "n"(SOFF), "n"(GOFF) : "memory");
    else if constexpr (BYTES == 8)
        asm volatile("cp.async.ca.shared.global [%0 + %2], [%1 + %3], 8;" ::"r"(smem_base), "l"(gmem_base), "n"(SOFF), "n"(GOFF) : "memory");
    else
        asm volatile("cp.async.ca.shared.global [%0 + %2], [%1 + %3], 4;" ::"r"(smem_base), "l"(gmem_base), "n"(SOFF), "n"(GOFF) : "memory");
}
template <int I, int N, typename F> __device__ __forceinline__ void static_for(F&& f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<I + 1, N>(f);
    }
}
// two E4M3 codes (low 16 bits) -> two f16 (exact)
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t pair) {
    uint32_t r;
    asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(r) : "r"(pair));
    return r;
}
__device__ __forceinline__ float fast_exp2(float x) {  // one MUFU; far-negative arguments give 0
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ void mma_f16_16x8x16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__host__ __device__ constexpr int tc_depth(int hd) { return hd <= 64 ? 4 : (hd <= 128 ? 3 : 2); }
#ifndef TC_VSTEP
#define TC_VSTEP 4
#endif
__host__ __device__ constexpr size_t tc_ring_bytes(int hd) {  // rings + block table + the Q operand (8 heads x hd bytes)
    return (size_t)MMA_WARPS * tc_depth(hd) * mma_stage_bytes(hd) + MMA_TBL_MAX * sizeof(int) + 8 * (size_t)hd;
}
__host__ __device__ constexpr size_t tc_smem_bytes(int hd, int gt) {
    return tc_ring_bytes(hd) > (size_t)MMA_WARPS * gt * (hd + 2) * sizeof(float)
               ? tc_ring_bytes(hd)
               : (size_t)MMA_WARPS * gt * (hd + 2) * sizeof(float);
}

// Cache slots are addressed with 32-bit indices here; the launcher checks
// num_blocks_total * block_size * kv_heads < 2^31 and uses the 64-bit kernel otherwise.
template <int HD, int GT, typename OutT>
__global__ void __launch_bounds__(MMA_THREADS, (HD <= 128 ? 4 : 3)) paged_decode_fp8_tc_kernel(Params p) {
    static_assert(GT <= 8, "at most 8 query heads per tile (the MMA's column count)");
    static_assert(HD == 64 || HD == 128 || HD == 256, "16 * HD/16 accumulators per lane: head_dim <= 256");
    constexpr int CH = HD / 64;          // 64-byte chunks per K row
    constexpr int DPL = HD / 16;         // V tiles (16 dims each) == contiguous V bytes a lane needs per row slot
    constexpr int VW = DPL / 4;          // 32-bit words per V piece
    constexpr int DEPTH = tc_depth(HD);
    constexpr int STAGE = mma_stage_bytes(HD);
    constexpr int STEP = MMA_WARPS * TILE_TOK;
    constexpr int PSTRIDE = HD + 2;
    constexpr bool Q_IN_SMEM = HD >= 256;  // keep the score B operand in shared memory instead of 4*CH registers

    extern __shared__ __align__(16) uint8_t sm_raw[];
    float* sm = reinterpret_cast<float*>(sm_raw);
    __shared__ unsigned s_bad;
    rv::pdl_launch();
    rv::pdl_wait();
    const int kvh = blockIdx.x, chunk = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;  // MMA fragment coordinates
    const int group = p.heads / p.kv_heads;
    OutT* out = reinterpret_cast<OutT*>(p.out);
    uint8_t* ring = sm_raw + (size_t)warp * DEPTH * STAGE;
    int* tbl = reinterpret_cast<int*>(sm_raw + (size_t)MMA_WARPS * DEPTH * STAGE);
    uint4* q_sm = reinterpret_cast<uint4*>(sm_raw + (size_t)MMA_WARPS * DEPTH * STAGE + MMA_TBL_MAX * sizeof(int));

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
    // cache slot index ((phys * block_size + off) * kv_heads + kvh) of a token; a table entry outside
    // the cache poisons the output (bad) and reads slot 0 instead, which is always inside the cache
    auto slot_of = [&](int tok) -> int {
        const int page = p.bs_shift >= 0 ? (tok >> p.bs_shift) : (tok / p.block_size);
        const int off = tok - page * p.block_size;
        int phys;
        if (tbl_in_smem) {
            phys = tbl[page - first_page];
        } else {
            phys = __ldg(table + (p.window_size_left >= 0 ? page % p.max_blocks_per_seq : page));
        }
        if ((unsigned)phys >= (unsigned)p.num_blocks_total) {
            bad = 0xffffffffu;
            return 0;
        }
        return (phys * p.block_size + off) * p.kv_heads + kvh;
    };
    // Stage layout: [K: 2*CH pieces x 32 lanes x 16 B][V: 8 pieces x 32 lanes x DPL B][16 k scales][16 v scales].
    // K piece (c, half) of lane (g, t) = bytes c*64+16t.. of token row g + 8*half.
    // V piece (x, ab) of lane (g, t)  = bytes (g+8*ab)*DPL.. of token row {2t, 2t+1, 2t+8, 2t+9}[x].
    // Rows past the end of the chunk copy the chunk's last token again (finite, attended data that the
    // masked probabilities multiply by zero), so the copies need no predicates and no zero fill.
    const uint8_t* k_lane = p.k_cache + 16 * t;
    const uint8_t* v_lane = p.v_cache + g * DPL;
    const float* sc_lane = lane < 16 ? p.k_scale_cache : p.v_scale_cache;  // lanes 0-15 fetch K scales, 16-31 V scales
    const float sc_scalar = lane < 16 ? k_ds_scalar : v_ds_scalar;
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
    auto issue = [&](int tok0, int stage) {
        if (tok0 < t_end) {  // warp-uniform
            const uint32_t st_s = ring_s + stage * STAGE;
            const int my_slot = slot_of(min(tok0 + (lane & 15), t_end - 1));
            if (sc_lane) cp_async_off<4, 2 * TILE_TOK * HD, 0>(st_s + lane * 4, sc_lane + my_slot);
            else reinterpret_cast<float*>(ring + stage * STAGE + 2 * TILE_TOK * HD)[lane] = sc_scalar;
            const uint32_t kdst = st_s + lane * 16, vdst = st_s + TILE_TOK * HD + lane * DPL;
            static_for<0, 2>([&](auto half) {
                const int slot = __shfl_sync(0xffffffffu, my_slot, g + 8 * half.value);
                const uint8_t* src = k_lane + (size_t)(unsigned)slot * HD;
                static_for<0, CH>([&](auto c) {
                    cp_async_off<16, (2 * c.value + half.value) * 512, c.value * 64>(kdst, src);
                });
            });
            static_for<0, 4>([&](auto x) {
                const int slot = __shfl_sync(0xffffffffu, my_slot, 2 * t + (x.value & 1) + 8 * (x.value >> 1));
                const uint8_t* src = v_lane + (size_t)(unsigned)slot * HD;
                static_for<0, 2>([&](auto ab) {
                    cp_async_off<DPL, (2 * x.value + ab.value) * 32 * DPL, 8 * ab.value * DPL>(vdst, src);
                });
            });
        }
        cp_async_commit();
    };

    for (int h0 = 0; h0 < group; h0 += GT) {
        const int nh = min(GT, group - h0);
        if (tid == 0) s_bad = 0;
        __syncthreads();
        bad = 0;
        // score B operand: raw Q codes of head column g (zero beyond the tile's heads), per 64-byte chunk
        uint4 qf[Q_IN_SMEM ? 1 : CH];
        {
            const int head = kvh * group + h0 + (g < nh ? g : 0);
            const uint8_t* qrow = p.q + ((size_t)b * p.heads + head) * HD;
            if constexpr (Q_IN_SMEM) {
                if (warp == 0) {
#pragma unroll
                    for (int c = 0; c < CH; c++)
                        q_sm[c * 32 + lane] = g < nh ? rv::ldg128(qrow + c * 64 + 16 * t) : make_uint4(0, 0, 0, 0);
                }
                __syncthreads();
            } else {
#pragma unroll
                for (int c = 0; c < CH; c++)
                    qf[c] = g < nh ? rv::ldg128(qrow + c * 64 + 16 * t) : make_uint4(0, 0, 0, 0);
            }
        }
        // this lane's score columns are heads 2t and 2t+1 of the tile: q scale * softmax scale * log2(e)
        // (softmax runs in base 2; the running max goes back to base e when it leaves the warp)
        float qsc[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int j = 2 * t + k;
            float v = 0.0f;
            if (j < nh) {
                const int head = kvh * group + h0 + j;
                const float q_ds = p.q_scale_cache ? p.q_scale_cache[(size_t)b * p.heads + head] : *p.q_descale;
                if (bad_scale(q_ds)) bad |= 1u << j;
                v = q_ds * p.scale * 1.4426950408889634f;
            }
            qsc[k] = v;
        }
        float m[2] = {-1e20f, -1e20f};  // running max (base-2 exponent) of heads 2t, 2t+1, uniform over g
        float l[2] = {0.0f, 0.0f};      // this lane's share of the softmax denominators
        // acc[i] = {out[dim g*DPL+i][head 2t], [same dim][head 2t+1], out[dim (g+8)*DPL+i][head 2t], [..][head 2t+1]}
        float acc[DPL][4];
#pragma unroll
        for (int i = 0; i < DPL; i++)
#pragma unroll
            for (int c = 0; c < 4; c++) acc[i][c] = 0.0f;
        // where this lane's P operand comes from: head g of tokens 2t / 2t+1 sits in lanes (2t | 2t+1, g>>1)
        const int src_a = (2 * t) * 4 + (g >> 1), src_b = (2 * t + 1) * 4 + (g >> 1);
        const unsigned half_sel = (g & 1) ? 0x7632u : 0x5410u;

        int tok_issue = t_begin + warp * TILE_TOK;
#pragma unroll 1
        for (int r = 0; r < DEPTH; r++, tok_issue += STEP) issue(tok_issue, r);
        int stage = 0;
#pragma unroll 1
        for (int tok0 = t_begin + warp * TILE_TOK; tok0 < t_end; tok0 += STEP, tok_issue += STEP) {
            cp_async_wait<DEPTH - 1>();
            __syncwarp();  // row scales are copied by one lane and read by others
            const uint8_t* st = ring + stage * STAGE;
            // ---- scores: 16 tokens x 8 head columns ----
            float S[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < CH; c++) {
                const uint4 ka = *reinterpret_cast<const uint4*>(st + ((2 * c) * 32 + lane) * 16);
                const uint4 kb = *reinterpret_cast<const uint4*>(st + ((2 * c + 1) * 32 + lane) * 16);
                uint4 qc;
                if constexpr (Q_IN_SMEM) qc = q_sm[c * 32 + lane];
                else qc = qf[c];
                mma_e4m3_16x8x32(S, ka.x, kb.x, ka.y, kb.y, qc.x, qc.y);
                mma_e4m3_16x8x32(S, ka.z, kb.z, ka.w, kb.w, qc.z, qc.w);
            }
            const float* sc = reinterpret_cast<const float*>(st + 2 * TILE_TOK * HD);
            const float kd0 = sc[g], kd1 = sc[g + 8], vd0 = sc[16 + g], vd1 = sc[16 + g + 8];
            {   // every scale must be a positive finite number: as unsigned bit patterns, in [1, 0x7f7fffff]
                const unsigned u0 = __float_as_uint(kd0), u1 = __float_as_uint(kd1), u2 = __float_as_uint(vd0),
                               u3 = __float_as_uint(vd1);
                if (min(min(u0, u1), min(u2, u3)) == 0u || max(max(u0, u1), max(u2, u3)) > 0x7f7fffffu)
                    bad = 0xffffffffu;
            }
            // all four quad lanes run the softmax; columns beyond the tile's heads carry zeros
            const bool tv0 = tok0 + g < t_end, tv1 = tok0 + g + 8 < t_end;
            float pv[4];  // p * v_scale for (token g | g+8, head 2t | 2t+1)
            float e0[2];
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const float s0 = tv0 ? S[k] * qsc[k] * kd0 : -1e30f;
                const float s1 = tv1 ? S[2 + k] * qsc[k] * kd1 : -1e30f;
                if (!isfinite(s0 + s1)) bad |= 1u << (2 * t + k);
                float tm = fmaxf(s0, s1);
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 4));
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 8));
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 16));
                const float m_new = fmaxf(m[k], tm);
                e0[k] = fast_exp2(m[k] - m_new);
                const float p0 = fast_exp2(s0 - m_new), p1 = fast_exp2(s1 - m_new);
                l[k] = l[k] * e0[k] + (p0 + p1);
                pv[k] = p0 * vd0;
                pv[2 + k] = p1 * vd1;
                m[k] = m_new;
            }
            if (e0[0] != 1.0f || e0[1] != 1.0f) {  // a running max moved: rescale this lane's columns
#pragma unroll
                for (int i = 0; i < DPL; i++) {
                    acc[i][0] *= e0[0];
                    acc[i][2] *= e0[0];
                    acc[i][1] *= e0[1];
                    acc[i][3] *= e0[1];
                }
            }
            // ---- P (token, head) fragments -> (head, token) operand of the second MMA ----
            const uint32_t plo = pack_f16x2(pv[0], pv[1]);  // token g,   heads 2t | 2t+1
            const uint32_t phi = pack_f16x2(pv[2], pv[3]);  // token g+8
            const uint32_t a_lo = __shfl_sync(0xffffffffu, plo, src_a), b_lo = __shfl_sync(0xffffffffu, plo, src_b);
            const uint32_t a_hi = __shfl_sync(0xffffffffu, phi, src_a), b_hi = __shfl_sync(0xffffffffu, phi, src_b);
            const uint32_t pb0 = __byte_perm(a_lo, b_lo, half_sel);  // {P[tok 2t][head g],   P[tok 2t+1][head g]}
            const uint32_t pb1 = __byte_perm(a_hi, b_hi, half_sel);  // {P[tok 2t+8][head g], P[tok 2t+9][head g]}
            // ---- P.V: V^T tiles (16 dims x 16 tokens) x P (16 tokens x 8 heads) ----
            // (at most 8 bytes of each of the lane's 8 pieces are live at a time)
            constexpr int VSTEP = TC_VSTEP < VW ? TC_VSTEP : VW;  // 32-bit words per piece per pass
#pragma unroll
            for (int w0 = 0; w0 < VW; w0 += VSTEP) {
                uint32_t vr[8][VSTEP];
#pragma unroll
                for (int pc = 0; pc < 8; pc++) {
                    const uint8_t* src = st + TILE_TOK * HD + (pc * 32 + lane) * DPL + 4 * w0;
                    if constexpr (VSTEP == 1) {
                        vr[pc][0] = *reinterpret_cast<const uint32_t*>(src);
                    } else if constexpr (VSTEP == 2) {
                        const uint2 v = *reinterpret_cast<const uint2*>(src);
                        vr[pc][0] = v.x;
                        vr[pc][1] = v.y;
                    } else {
                        const uint4 v = *reinterpret_cast<const uint4*>(src);
                        vr[pc][0] = v.x;
                        vr[pc][1] = v.y;
                        vr[pc][2] = v.z;
                        vr[pc][3] = v.w;
                    }
                }
#pragma unroll
                for (int ii = 0; ii < 4 * VSTEP; ii++) {
                    const int i = 4 * w0 + ii;                                // V tile: dims {r*DPL + i}
                    const unsigned sel = (ii & 3) | ((4 + (ii & 3)) << 4);   // byte i of the first word, then of the second
                    const int w = ii >> 2;
                    const uint32_t a0 = e4m3x2_to_f16x2(__byte_perm(vr[0][w], vr[2][w], sel));  // dims g..,   tokens 2t, 2t+1
                    const uint32_t a1 = e4m3x2_to_f16x2(__byte_perm(vr[1][w], vr[3][w], sel));  // dims g+8.., tokens 2t, 2t+1
                    const uint32_t a2 = e4m3x2_to_f16x2(__byte_perm(vr[4][w], vr[6][w], sel));  // dims g..,   tokens 2t+8, 2t+9
                    const uint32_t a3 = e4m3x2_to_f16x2(__byte_perm(vr[5][w], vr[7][w], sel));  // dims g+8.., tokens 2t+8, 2t+9
                    mma_f16_16x8x16(acc[i], a0, a1, a2, a3, pb0, pb1);
                }
            }
            __syncwarp();
            issue(tok_issue, stage);  // refill the stage just consumed
            stage = stage + 1 == DEPTH ? 0 : stage + 1;
        }
        cp_async_wait<0>();

#pragma unroll
        for (int k = 0; k < 2; k++) {  // denominators: sum the per-token-row shares over g
            l[k] += __shfl_xor_sync(0xffffffffu, l[k], 4);
            l[k] += __shfl_xor_sync(0xffffffffu, l[k], 8);
            l[k] += __shfl_xor_sync(0xffffffffu, l[k], 16);
        }
        if (bad) atomicOr(&s_bad, bad);
        __syncthreads();  // every warp is done with its ring before the merge buffer overlays it
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int j = 2 * t + k;
            if (j < GT) {
                float* dst = sm + ((size_t)warp * GT + j) * PSTRIDE;
#pragma unroll
                for (int i = 0; i < DPL; i++) {
                    dst[g * DPL + i] = acc[i][k];
                    dst[(g + 8) * DPL + i] = acc[i][2 + k];
                }
                if (g == 0) {
                    dst[HD] = m[k] * 0.6931471805599453f;
                    dst[HD + 1] = l[k];
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
