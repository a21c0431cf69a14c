// FP8-KV paged GQA decode attention on tcgen05 / TMEM / TMA (sm_100a).
//
// Same contract, grid, chunk rule and partial layout as paged_decode_fp8_kernel
// (paged_decode_fp8.cuh; reference semantics: v3/kernels/fp8_decode_v2.cu:199-325,339-624).
// The mma.sync kernels spend their time issuing instructions (address arithmetic, cp.async, byte
// permutes, conversions) around small register-level MMAs; a decode batch of a few dozen rows
// does not bring enough warps to hide that.  Here a CTA moves and multiplies whole pages:
//
//   tile    = 128 tokens of one KV head (whole cache pages, first and last tile masked).
//   warp 0  : producer.  One lane looks the pages up in the block table and issues one TMA
//             (cp.async.bulk.tensor.3d, 128-byte swizzle) per page and 128-byte panel of K and of V
//             into a ring of 16 KB units; completion is counted on an mbarrier per unit.
//   warp 1  : MMA issuer.  scores^T[128 tokens x 16 head columns] = K_tile . Q^T with
//             tcgen05.mma kind::f8f6f4 straight from the cache bytes (K rows are the K-major A
//             operand, the raw Q codes of the KV head's query heads the B operand), accumulator in
//             TMEM, double buffered.  Then out^T[head dims x 32] += V_tile^T . P, where V is the
//             *MN-major* A operand (the cache row already holds the head dims contiguously, which
//             is exactly that layout) and P the K-major B operand written by the softmax warps.
//   warps 2-5: softmax.  Thread i owns token i of the tile: reads its scores from TMEM
//             (tcgen05.ld), applies q/k scales and the mask, takes the tile maximum with its 127
//             peers, and writes its probabilities for the second MMA as three E4M3 terms
//             (hi + mid + lo, 2^-12 relative) into the P tile — the token's V scale is folded into
//             the exponent, so the second product also runs on raw cache bytes.  When a running
//             maximum moves, the same threads (thread i now owns head dim i of the accumulator)
//             rescale the TMEM accumulator in place.
//   Every wait on an mbarrier is bounded; a wait that runs out records its site in a status word
//   and the kernel walks on through all barriers and the TMEM release.
//
// Numerics: scores and the softmax are f32; V bytes enter the tensor core unconverted; a
// probability is rounded to three E4M3 terms.  Rows of a tile outside the attended interval are
// zeroed in shared memory before the second product (stale cache bytes could be NaN codes).
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>
#include <unordered_map>

#include "paged_decode_fp8.cuh"

namespace rvua {

using rvattn::Params;

constexpr int TOK = 128;          // tokens per tile == UMMA M of the score product
constexpr int PANEL = 128;        // bytes per operand panel row (one 128-byte swizzle atom)
constexpr int UNIT = TOK * PANEL; // 16 KB: one panel of K or V for one tile
constexpr int THREADS = 192;
constexpr int NQ = 16;            // score columns (UMMA N): up to 8 query heads, zero padded
constexpr int NP = 32;            // P rows (UMMA N of the second product): 3 terms x 8 heads, zero padded
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ int g_status = 0;  // 0 ok; otherwise (site << 16 | detail) of the first wait that gave up

// ---- PTX wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and records `site`) if the phase never completed.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int site) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicCAS(&g_status, 0, (site << 16) | (int)(blockIdx.x & 0xffff));
    return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void bar_softmax() { asm volatile("bar.sync 1, 128;" ::: "memory"); }  // warps 2-5 only

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* holder, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
// 4-byte store into the shared memory of cluster rank `rank`, at the offset `local_saddr` has in this CTA.
__device__ __forceinline__ void st_cluster_f32(uint32_t local_saddr, uint32_t rank, float v) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "st.shared::cluster.f32 [ra], %2;\n\t}" ::"r"(local_saddr), "r"(rank), "f"(v)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {  // one MUFU; far-negative arguments give 0
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// Shared-memory operand descriptors, 128-byte swizzle, 8-row groups 1024 B apart.
// K-major: rows are the M/N index, the 128 bytes of a row are K (the layout of a [rows x 128 B] TMA box).
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;            // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;            // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;            // SWIZZLE_128B
    return d;
}
// MN-major: rows are K (tokens), the 128 bytes of a row are 128 consecutive M indices (head dims).
// Stride between 8-row (8 tokens) groups = 1024 B; one 128-byte row covers the whole M = 128 of an MMA,
// so the offset between 128-wide M blocks (leading byte offset) is never used.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)(UNIT >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f8f6f4, E4M3 x E4M3 -> F32, M = 128; a_mn: A operand is MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool a_mn) {
    return (1u << 4) | (a_mn ? (1u << 15) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

constexpr int MAX_UNITS = 8;
template <int HD> struct Cfg {
    static constexpr int HALVES = HD / PANEL;            // 128-byte panels per K or V tile
    static constexpr int UPT = 2 * HALVES;               // ring units per tile: K panels, then V panels
    static constexpr int MIN_UNITS = HALVES == 1 ? 2 : 3;     // both K panels plus one more must fit
    static constexpr int TMEM_COLS = HALVES == 1 ? 64 : 128;  // scores 2 x 16, then HALVES x 32 accumulator columns
    static constexpr int O_COL = 32;
    static constexpr int P_BYTES = NP * PANEL;           // 4 KB
    static constexpr int Q_BYTES = HALVES * NQ * PANEL;  // 2 KB per panel
    static constexpr int AUX_BYTES = 1024;               // barriers, TMEM holder, reduction scratch
    static constexpr int smem_bytes(int units) { return 1024 + units * UNIT + P_BYTES + Q_BYTES + AUX_BYTES; }
    // cluster-combine form: partials of `chunks` CTAs x `group` query heads, [HD + 2] floats each, behind the rest
    static constexpr int recv_bytes(int chunks, int group) { return chunks * group * (HD + 2) * 4; }
};
constexpr int MAX_RECV_BYTES = 24 * 1024;

// Three-term E4M3 expansion of x in [0, 256]: x ~= hi + mid + lo with relative error ~2^-12.
__device__ __forceinline__ void split3(float x, uint8_t& hi, uint8_t& mid, uint8_t& lo) {
    hi = rv::f32_to_e4m3(x);
    float r = x - rv::e4m3x2_to_f32x2(hi).x;
    mid = rv::f32_to_e4m3(r);
    r -= rv::e4m3x2_to_f32x2(mid).x;
    lo = rv::f32_to_e4m3(r);
}

// CL: the cluster-merged split-KV form (Params::cluster_combine), an instantiation of its own: the plain one keeps
// its 64 registers — five CTAs of the shallowest ring share an SM (30 warps), which a batch-128 launch counts on.
template <int HD, int GT, typename OutT, bool CL>
__global__ void __launch_bounds__(THREADS, 1)
paged_decode_fp8_umma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, Params p,
                             int nunits) {
    static_assert(HD == 128 || HD == 256, "one or two 128-byte panels per cache row");
    static_assert(GT >= 1 && GT <= 8, "up to 8 query heads share the score tile");
    using C = Cfg<HD>;
    constexpr int HALVES = C::HALVES, UPT = C::UPT;
    const int NUNITS = nunits;  // ring depth in 16 KB units (sets the shared-memory footprint: CTAs per SM vs look-ahead)
    constexpr int PSTRIDE = HD + 2;
    extern __shared__ uint8_t raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = base;                                  // NUNITS x 16 KB
    uint8_t* p_tile = ring + NUNITS * UNIT;                // [32 rows][128 token bytes], swizzled
    uint8_t* q_tile = p_tile + C::P_BYTES;                 // HALVES x [16 rows][128 B], swizzled
    uint8_t* aux = q_tile + C::Q_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(aux);     // [NUNITS] TMA landed
    uint64_t* empty = full + MAX_UNITS;                    // [NUNITS] MMAs that read the unit are done
    uint64_t* s_ready = empty + MAX_UNITS;                    // [2] score tile in TMEM
    uint64_t* s_free = s_ready + 2;                        // [2] softmax has read the score tile
    uint64_t* p_ready = s_free + 2;                        // P tile written (and accumulator rescaled)
    uint64_t* pv_done = p_ready + 1;                       // the tile's second product has completed
    uint64_t* merge_bar = pv_done + 1;                     // cluster form, chunk 0: the other chunks' partials have landed
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(merge_bar + 1);
    float* red = reinterpret_cast<float*>(aux + 256);      // [2][4][8] tile maxima, then [4][8] sums (96 floats)
    unsigned* s_bad = reinterpret_cast<unsigned*>(aux + 256 + 96 * 4);
    float* recv = reinterpret_cast<float*>(aux + C::AUX_BYTES);  // cluster-combine form only: [chunk][head][HD + 2]

    rv::pdl_launch();
    const int kvh = blockIdx.x, chunk = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int group = p.heads / p.kv_heads;
    OutT* out = reinterpret_cast<OutT*>(p.out);

    // ---- set-up that does not depend on the preceding kernel ----
    if (tid == 0) {
        for (int i = 0; i < NUNITS; i++) {
            mbar_init(full + i, 1);
            mbar_init(empty + i, 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(s_ready + i, 1);
            mbar_init(s_free + i, 4);
        }
        mbar_init(p_ready, 4);
        mbar_init(pv_done, 1);
        if constexpr (CL) mbar_init(merge_bar, (uint32_t)(gridDim.y - 1) * 4u);  // four warps of every other CTA of the cluster
        *s_bad = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(tmem_holder, C::TMEM_COLS);
    for (int i = tid; i < (C::P_BYTES + C::Q_BYTES) / 16; i += THREADS)  // zero P and Q tiles (padding rows stay zero)
        reinterpret_cast<uint4*>(p_tile)[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async();  // the zeroes must be visible to the tensor core's (async-proxy) reads
    const bool early = p.early_meta != 0;
    if (!early) rv::pdl_wait();

    // ---- sequence geometry (same rules as the other variants) ----
    const int ctx = p.context_lens[b];
    const long long capacity = (long long)p.block_size * p.max_blocks_per_seq;
    bool active = true;
    int t_begin = 0, t_end = 0, nchunks = 1;
    if (ctx <= 0 || (p.window_size_left < 0 && (long long)ctx > capacity)) {
        active = false;
        if (chunk == 0) {
            const float fill = ctx == 0 ? 0.0f : CUDART_NAN_F;
            if (p.force_partial) {
                for (int i = tid; i < group * PSTRIDE; i += THREADS) {
                    const int hh = i / PSTRIDE, d = i % PSTRIDE;
                    float* ws = p.workspace + (((size_t)b * p.heads + (size_t)kvh * group + hh) * p.max_chunks) * PSTRIDE;
                    ws[d] = d < HD ? fill : (d == HD ? -1e20f : 0.0f);
                }
            } else {
                for (int i = tid; i < group * HD; i += THREADS)
                    out[((size_t)b * p.heads + (size_t)kvh * group) * HD + i] = rv::T16<OutT>::from_f32(fill);
                if (p.amax_out && tid == 0) p.amax_out[(size_t)b * p.kv_heads + kvh] = 0.0f;  // zeros, or NaN (ignored by a max)
            }
        }
    } else {
        int start, len;
        rvattn::attend_interval(ctx, p.window_size_left, start, len);
        nchunks = rvattn::chunks_for(len, p.max_chunks, p.min_chunk_tokens);
        if (chunk >= nchunks) {
            active = false;
        } else {
            const int chunk_size = (len + nchunks - 1) / nchunks;
            t_begin = start + chunk * chunk_size;
            t_end = min(t_begin + chunk_size, start + len);
        }
    }
    const int bs = p.block_size;
    const int tile0 = active ? (t_begin / bs) * bs : 0;              // first tile starts on a page boundary
    const int ntiles = active ? (t_end - tile0 + TOK - 1) / TOK : 0;
    const int* table = p.block_tables + (size_t)b * p.max_blocks_per_seq;

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // "this CTA runs and its barriers exist": the other CTAs of the cluster wait for this before they touch its memory
    if constexpr (CL) asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    const uint32_t tmem_base = *tmem_holder;
    const int nh = group < GT ? group : GT;  // query heads of this KV head (the launcher guarantees group <= GT)
    if (warp != 0) {
        // The producer warp goes straight to its loads; the other five warps stage Q meanwhile.
        if (early) rv::pdl_wait();  // Q, and the newest token's scales, come from the preceding kernel
        if (active) {
            // Q codes of the KV head's query heads -> B operand panels (K-major, swizzled by hand)
            for (int i = tid - 32; i < nh * (HD / 16); i += THREADS - 32) {
                const int n = i / (HD / 16), c = i % (HD / 16), h = c >> 3, cc = c & 7;
                const uint4 v = rv::ldg128(p.q + ((size_t)b * p.heads + (size_t)kvh * group + n) * HD + c * 16);
                *reinterpret_cast<uint4*>(q_tile + h * (NQ * PANEL) + n * PANEL + ((cc ^ (n & 7)) << 4)) = v;
            }
        }
        fence_proxy_async();  // P / Q tiles were written through the generic proxy; the MMAs read them through the async one
        asm volatile("bar.sync 2, 160;" ::: "memory");
    }

    // physical block of the page holding `tok` (integer divisions only off the common power-of-two path)
    auto phys_of = [&](int tok, bool& bad_page) -> int {
        const int page = p.bs_shift >= 0 ? (tok >> p.bs_shift) : tok / bs;
        const int ph = __ldg(table + (p.window_size_left >= 0 ? page % p.max_blocks_per_seq : page));
        if ((unsigned)ph >= (unsigned)p.num_blocks_total) {
            bad_page = true;
            return 0;
        }
        return ph;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (whole warp)
        // Lane j owns page j of every tile: one table load and one TMA per lane and panel, issued side
        // by side, instead of one thread walking the pages (serial address arithmetic and TMA issue
        // cost ~2 us per tile that way, more than the loads themselves).
        if (ntiles > 0) {
            const int ppt = TOK / bs;  // pages per tile (<= 16)
            bool alive = true, bad_page = false;
            int slot = 0, use = 0;  // ring position of the next unit (kept incrementally: NUNITS is a run-time value)
            for (int i = 0; i < ntiles && alive; i++) {
                if (early && i == ntiles - 1) rv::pdl_wait();  // the newest token's K / V rows are in the last tile
                const int tok_tile = tile0 + i * TOK;
                // pages of the tile that hold attended tokens; the rest are not fetched (their rows of the
                // unit keep stale bytes: masked in the scores, zeroed by the softmax warps for the V panels)
                const int np = min(ppt, (t_end - tok_tile + bs - 1) / bs);
                int z = 0;
                if (lane < np) z = phys_of(tok_tile + lane * bs, bad_page) * bs;
#pragma unroll 1
                for (int u = 0; u < UPT && alive; u++) {
                    if (use > 0) {
                        if (lane == 0) alive = mbar_wait(empty + slot, (uint32_t)(use - 1) & 1u, 1);
                        alive = __shfl_sync(0xffffffffu, (int)alive, 0) != 0;
                    }
                    if (!alive) break;
                    if (lane == 0) mbar_expect_tx(full + slot, (uint32_t)(np * bs * PANEL));
                    __syncwarp();
                    if (lane < np)
                        tma_load_3d(ring + (size_t)slot * UNIT + (size_t)lane * bs * PANEL, u < HALVES ? &map_k : &map_v,
                                    (u % HALVES) * PANEL, kvh, z, full + slot);
                    if (++slot == NUNITS) {
                        slot = 0;
                        use++;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && ntiles > 0) {
            constexpr uint32_t idesc_qk = instr_desc(NQ, false), idesc_pv = instr_desc(NP, true);
            const uint64_t qdesc = desc_kmajor(smem_u32(q_tile)), pdesc = desc_kmajor(smem_u32(p_tile));
            // Issue whichever product has its inputs first: the score MMA of the next tile (its K panels
            // have landed and its TMEM buffer is free) or the second product of the oldest open tile (its P
            // tile is written and its V panels have landed).  Waiting for one in program order would hold
            // the other back, and with it the release of the ring units the producer is waiting for.
            int next_qk = 0, next_pv = 0;
            uint32_t idle = 0;
            bool alive = true;
            // ring position (slot, use count) of the first K panel of tile next_qk and of the first V panel of
            // tile next_pv, advanced incrementally: NUNITS is a run-time value, and this loop polls
            int q_slot = 0, q_use = 0, v_slot = HALVES % NUNITS, v_use = HALVES / NUNITS;
            auto advance = [&](int& slot, int& use) {
                slot += UPT;
                while (slot >= NUNITS) {
                    slot -= NUNITS;
                    use++;
                }
            };
            // A unit's barrier may only be polled once the unit's previous occupant has been consumed here:
            // a parity wait cannot tell "this use has landed" from "the use before last has", so polling
            // while the previous use is still loading would report the data as present.
            auto prev_consumed = [&](int g) {
                g -= NUNITS;
                if (g < 0) return true;
                const int tile = g / UPT;
                return g % UPT < HALVES ? tile < next_qk : tile < next_pv;
            };
            while (next_pv < ntiles && alive) {
                bool did = false;
                if (next_qk < ntiles && next_qk <= next_pv + 2) {  // the score tile in TMEM is double buffered
                    const int i = next_qk;
                    bool ok = i < 2 || mbar_try_wait(s_free + (i & 1), (uint32_t)((i >> 1) - 1) & 1u);
                    int slot[HALVES];
#pragma unroll
                    for (int h = 0; h < HALVES; h++) {
                        int sl = q_slot + h, us = q_use;
                        if (sl >= NUNITS) {
                            sl -= NUNITS;
                            us++;
                        }
                        slot[h] = sl;
                        ok = ok && prev_consumed(i * UPT + h) && mbar_try_wait(full + sl, (uint32_t)us & 1u);
                    }
                    if (ok) {
                        tc_fence_after();
#pragma unroll
                        for (int h = 0; h < HALVES; h++) {
                            const uint64_t kdesc = desc_kmajor(smem_u32(ring + (size_t)slot[h] * UNIT));
                            const uint64_t qd = qdesc + (uint64_t)((h * NQ * PANEL) >> 4);
#pragma unroll
                            for (int k = 0; k < PANEL / 32; k++)
                                umma_f8(tmem_base + (uint32_t)(i & 1) * NQ, kdesc + (uint64_t)(2 * k), qd + (uint64_t)(2 * k),
                                        idesc_qk, (h > 0 || k > 0) ? 1u : 0u);
                            umma_commit(empty + slot[h]);
                        }
                        umma_commit(s_ready + (i & 1));
                        next_qk++;
                        advance(q_slot, q_use);
                        did = true;
                    }
                }
                if (next_pv < next_qk) {
                    const int i = next_pv;
                    bool ok = mbar_try_wait(p_ready, (uint32_t)i & 1u);
                    int slot[HALVES];
#pragma unroll
                    for (int h = 0; h < HALVES; h++) {
                        int sl = v_slot + h, us = v_use;
                        if (sl >= NUNITS) {
                            sl -= NUNITS;
                            us++;
                        }
                        slot[h] = sl;
                        ok = ok && prev_consumed(i * UPT + HALVES + h) && mbar_try_wait(full + sl, (uint32_t)us & 1u);
                    }
                    if (ok) {
                        tc_fence_after();
#pragma unroll
                        for (int h = 0; h < HALVES; h++) {
                            const uint64_t vdesc = desc_mnmajor(smem_u32(ring + (size_t)slot[h] * UNIT));
#pragma unroll
                            for (int k = 0; k < TOK / 32; k++)  // 32 tokens (rows of 128 B) per MMA
                                umma_f8(tmem_base + C::O_COL + (uint32_t)h * NP, vdesc + (uint64_t)((32 * PANEL * k) >> 4),
                                        pdesc + (uint64_t)(2 * k), idesc_pv, (i > 0 || k > 0) ? 1u : 0u);
                            umma_commit(empty + slot[h]);
                        }
                        umma_commit(pv_done);
                        next_pv++;
                        advance(v_slot, v_use);
                        did = true;
                    }
                }
                if (did) {
                    idle = 0;
                } else if (++idle > WAIT_LIMIT) {
                    atomicCAS(&g_status, 0, (2 << 16) | (int)(blockIdx.x & 0xffff));
                    alive = false;
                }
            }
        }
    } else if (ntiles > 0) {
        // ------------------------------------------------------------------ softmax (128 threads)
        const int quarter = warp & 3;             // TMEM lanes this warp may touch: 32 * quarter ..
        const int row = quarter * 32 + lane;      // token of the tile (scores) / head dim of the panel (accumulator)
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const bool k_perslot = p.k_scale_cache != nullptr, v_perslot = p.v_scale_cache != nullptr;
        const float k_scalar = k_perslot ? 0.0f : *p.k_descale, v_scalar = v_perslot ? 0.0f : *p.v_descale;
        unsigned bad = 0;
        float qsc[GT];  // q scale * softmax scale * log2(e): the softmax runs in base 2
#pragma unroll
        for (int k = 0; k < GT; k++) {
            qsc[k] = 0.0f;
            if (k < nh) {
                const int head = kvh * group + k;
                const float q_ds = p.q_scale_cache ? p.q_scale_cache[(size_t)b * p.heads + head] : *p.q_descale;
                if (rvattn::bad_scale(q_ds)) bad |= 1u << k;
                qsc[k] = q_ds * p.scale * 1.4426950408889634f;
            }
        }
        float m_run[GT], l_part[GT];
#pragma unroll
        for (int k = 0; k < GT; k++) {
            m_run[k] = -1e20f;
            l_part[k] = 0.0f;
        }
        // this thread's token of a tile: validity and its K / V scales (fetched one tile ahead)
        auto fetch = [&](int i, bool& valid, float& ks, float& vs) {
            const int tok = tile0 + i * TOK + row;
            valid = i < ntiles && tok >= t_begin && tok < t_end;
            ks = k_scalar;
            vs = v_scalar;
            if (valid) {
                bool bad_page = false;
                const int ph = phys_of(tok, bad_page);
                if (bad_page) bad = 0xffffffffu;  // a table entry outside the cache poisons the whole row
                const size_t sidx = ((size_t)ph * bs + (tok % bs)) * p.kv_heads + kvh;
                if (k_perslot) ks = __ldg(p.k_scale_cache + sidx);
                if (v_perslot) vs = __ldg(p.v_scale_cache + sidx);
            }
        };
        bool valid_n, alive = true;
        float ks_n, vs_n;
        fetch(0, valid_n, ks_n, vs_n);
        for (int i = 0; i < ntiles && alive; i++) {
            const bool valid = valid_n;
            const float ks = ks_n, vs = vs_n;
            fetch(i + 1, valid_n, ks_n, vs_n);
            if (valid && (rvattn::bad_scale(ks) || rvattn::bad_scale(vs))) bad = 0xffffffffu;
            const float lv = valid ? __log2f(vs) : 0.0f;
            // ---- scores of this token ----
            alive = mbar_wait(s_ready + (i & 1), (uint32_t)(i >> 1) & 1u, 6);
            if (!alive) break;
            tc_fence_after();
            uint32_t sraw[8];
            tmem_ld8(lane_base + (uint32_t)(i & 1) * NQ, sraw);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free + (i & 1));
            float s2[GT];  // base-2 score without / with the V scale folded in
            float* mx = red + (i & 1) * 32 + (warp - 2) * 8;
#pragma unroll
            for (int k = 0; k < GT; k++) {
                float s = __uint_as_float(sraw[k]) * qsc[k] * ks;
                if (valid && k < nh && !isfinite(s)) {
                    bad |= 1u << k;
                    s = -1e30f;
                }
                s2[k] = valid ? s : -1e30f;
                const float wm = rv::warp_max(s2[k] + lv);
                if (lane == 0) mx[k] = wm;
            }
            bar_softmax();
            float corr[GT];
            bool moved = false;
            uint8_t term[GT][3];
#pragma unroll
            for (int k = 0; k < GT; k++) {
                const float* all = red + (i & 1) * 32 + k;
                const float tm = fmaxf(fmaxf(all[0], all[8]), fmaxf(all[16], all[24]));
                const float m_new = fmaxf(m_run[k], tm);
                corr[k] = fast_exp2(m_run[k] - m_new);
                moved |= k < nh && m_new > m_run[k];
                m_run[k] = m_new;
                const float x = valid ? fast_exp2(s2[k] + lv - m_new + 8.0f) : 0.0f;  // p * v_scale, in (0, 256]
                const float y = valid ? fast_exp2(s2[k] - m_new + 8.0f) : 0.0f;       // p, same normalisation
                l_part[k] = l_part[k] * corr[k] + y;
                split3(x, term[k][0], term[k][1], term[k][2]);
            }
            // ---- the previous tile's second product must be done before P is overwritten / O rescaled ----
            if (i > 0) alive = mbar_wait(pv_done, (uint32_t)(i - 1) & 1u, 7);
            if (!alive) break;
#pragma unroll
            for (int k = 0; k < GT; k++)
                if (k < nh) {
                    const uint32_t off = (uint32_t)((((row >> 4) ^ k) << 4) + (row & 15));
#pragma unroll
                    for (int t = 0; t < 3; t++) p_tile[(t * 8 + k) * PANEL + off] = term[k][t];
                }
            // rows of the tile outside the attended interval: zero their V bytes (stale cache bytes may be NaN codes)
            if (tile0 + i * TOK < t_begin || tile0 + (i + 1) * TOK > t_end) {
                for (int h = 0; h < HALVES && alive; h++) {
                    const int g = i * UPT + HALVES + h, slot = g % NUNITS;
                    alive = mbar_wait(full + slot, (uint32_t)(g / NUNITS) & 1u, 8);
                    if (alive && !valid) {
                        uint4* vrow = reinterpret_cast<uint4*>(ring + (size_t)slot * UNIT + row * PANEL);
#pragma unroll
                        for (int c = 0; c < PANEL / 16; c++) vrow[c] = make_uint4(0, 0, 0, 0);
                    }
                }
                if (!alive) break;
            }
            if (i > 0 && moved) {  // block-uniform: every thread sees the same maxima
                tc_fence_after();
#pragma unroll
                for (int h = 0; h < HALVES; h++)
#pragma unroll
                    for (int t = 0; t < 3; t++) {
                        uint32_t o[8];
                        const uint32_t addr = lane_base + C::O_COL + (uint32_t)(h * NP + t * 8);
                        tmem_ld8(addr, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int k = 0; k < GT; k++) o[k] = __float_as_uint(__uint_as_float(o[k]) * corr[k]);
                        tmem_st8(addr, o);
                    }
                tmem_st_wait();
            }
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready);
        }
        // ---- epilogue: accumulator (thread = head dim) / denominators -> output or partial ----
        if (alive) alive = mbar_wait(pv_done, (uint32_t)(ntiles - 1) & 1u, 9);
        tc_fence_after();
        float* sums = red + 64 + (warp - 2) * 8;  // [4][8]
#pragma unroll
        for (int k = 0; k < GT; k++) {
            const float ws = rv::warp_sum(l_part[k]);
            if (lane == 0) sums[k] = ws;
        }
        if (bad) atomicOr(s_bad, bad);
        bar_softmax();
        const unsigned bad_mask = alive ? *s_bad : 0xffffffffu;
        float amax = 0.0f;  // max |output as stored| over this thread's values (what the per-token quantiser would scan)
#pragma unroll
        for (int h = 0; h < HALVES; h++) {
            float acc[GT];
#pragma unroll
            for (int k = 0; k < GT; k++) acc[k] = 0.0f;
#pragma unroll
            for (int t = 0; t < 3; t++) {
                uint32_t o[8];
                tmem_ld8(lane_base + C::O_COL + (uint32_t)(h * NP + t * 8), o);
                tmem_ld_wait();
#pragma unroll
                for (int k = 0; k < GT; k++) acc[k] += __uint_as_float(o[k]);
            }
            const int d = h * PANEL + row;
#pragma unroll
            for (int k = 0; k < GT; k++)
                if (k < nh) {
                    const float L = red[64 + k] + red[64 + 8 + k] + red[64 + 16 + k] + red[64 + 24 + k];
                    const bool any_bad = (bad_mask >> k) & 1u;
                    const int head = kvh * group + k;
                    if (nchunks == 1 && !p.force_partial) {
                        float v = L > 0.0f ? acc[k] / L : acc[k];
                        if (any_bad) v = CUDART_NAN_F;
                        const OutT stored = rv::T16<OutT>::from_f32(v);
                        out[((size_t)b * p.heads + head) * HD + d] = stored;
                        amax = fmaxf(amax, fabsf(rv::T16<OutT>::to_f32(stored)));  // fmaxf drops a NaN, as the quantiser does
                    } else if (CL) {
                        // staged in this CTA's own slot 0 (for chunk 0 that is its final place); sent to the
                        // chunk-0 CTA further down, once that CTA is known to run
                        float* st = recv + (size_t)k * PSTRIDE;
                        st[d] = any_bad ? CUDART_NAN_F : acc[k];
                        if (d == 0) {
                            st[HD] = (m_run[k] - 8.0f) * 0.6931471805599453f;
                            st[HD + 1] = any_bad ? CUDART_NAN_F : L;
                        }
                    } else {
                        float* ws = p.workspace + (((size_t)b * p.heads + head) * p.max_chunks + chunk) * PSTRIDE;
                        ws[d] = any_bad ? CUDART_NAN_F : acc[k];
                        if (d == 0) {
                            ws[HD] = (m_run[k] - 8.0f) * 0.6931471805599453f;  // back to base e
                            ws[HD + 1] = any_bad ? CUDART_NAN_F : L;
                        }
                    }
                }
        }
        if (p.amax_out && nchunks == 1 && !p.force_partial) {
            amax = rv::warp_max(amax);
            bar_softmax();  // everyone has read the sums: the scratch can be reused
            if (lane == 0) red[64 + (warp - 2)] = amax;
            bar_softmax();
            if (warp == 2 && lane == 0)
                p.amax_out[(size_t)b * p.kv_heads + kvh] = fmaxf(fmaxf(red[64], red[65]), fmaxf(red[66], red[67]));
        }
        tc_fence_before();
    }
    if constexpr (CL) {
        // Every thread of every CTA of the cluster, active or not, passes these barriers: first "all CTAs of the
        // cluster run" (the arrival was the kernel's first statement; shared memory of a CTA that has not started
        // must not be written), then "the partials are in the chunk-0 CTA's shared memory".
        asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
        // The partials travel without a second cluster-wide barrier: every softmax warp of every other CTA — with a
        // partial or not — arrives (release, cluster scope) on chunk 0's mbarrier after its stores; chunk 0 waits for
        // all of them; the others are done.
        if (chunk != 0 && warp >= 2) {
            if (active && nchunks > 1) {
                bar_softmax();  // the staged partial is complete
                const uint32_t dst = smem_u32(recv + (size_t)chunk * nh * PSTRIDE);
                for (int i = tid - 64; i < nh * PSTRIDE; i += 128) st_cluster_f32(dst + (uint32_t)i * 4u, 0u, recv[i]);
            }
            asm volatile("fence.acq_rel.cluster;" ::: "memory");  // every lane's stores, before the warp's one arrival
            __syncwarp();
            if (lane == 0)
                asm volatile(
                    "{\n\t.reg .b32 ra;\n\t"
                    "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
                    "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}" ::"r"(smem_u32(merge_bar)), "r"(0u)
                    : "memory");
        }
        bool merged = true;
        if (chunk == 0 && warp >= 2) {
            unsigned* s_flag = s_bad + 1;  // one thread waits (bounded), the four warps share its verdict
            if (tid == 64) {
                uint32_t ok = 0;
                for (uint32_t spin = 0; spin < WAIT_LIMIT && !ok; spin++)
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                        "selp.u32 %0, 1, 0, p;\n\t}"
                        : "=r"(ok)
                        : "r"(smem_u32(merge_bar)), "r"(0u)
                        : "memory");
                if (!ok) atomicCAS(&g_status, 0, (10 << 16) | (int)(blockIdx.x & 0xffff));
                *s_flag = ok;
            }
            bar_softmax();
            merged = *s_flag != 0;
        }
        if (chunk == 0 && active && nchunks > 1 && warp >= 2 && merged) {
            // The merge of the combine kernel, chunk by chunk in order (same arithmetic, same order), then the
            // store and the per-(sequence, KV head) maximum of the single-chunk path.
            const int row = (warp - 2) * 32 + lane;
            int m_start, m_len;
            rvattn::attend_interval(ctx, p.window_size_left, m_start, m_len);
            const int m_size = (m_len + nchunks - 1) / nchunks;
            float amax = 0.0f;
#pragma unroll
            for (int h = 0; h < HALVES; h++) {
                const int d = h * PANEL + row;
                for (int k = 0; k < nh; k++) {
                    float M = -1e20f, L = 0.0f, A = 0.0f;
                    for (int c = 0; c < nchunks && c * m_size < m_len; c++) {  // (a chunk past the end stored nothing)
                        const float* src = recv + (size_t)(c * nh + k) * PSTRIDE;
                        const float mc = src[HD], lc = src[HD + 1];
                        const float Mn = fmaxf(M, mc);
                        const float ea = __expf(M - Mn), eb = __expf(mc - Mn);
                        A = A * ea + src[d] * eb;
                        L = L * ea + lc * eb;
                        M = Mn;
                    }
                    const OutT stored = rv::T16<OutT>::from_f32(L > 0.0f ? A / L : A);
                    out[((size_t)b * p.heads + (size_t)kvh * group + k) * HD + d] = stored;
                    amax = fmaxf(amax, fabsf(rv::T16<OutT>::to_f32(stored)));
                }
            }
            if (p.amax_out) {
                amax = rv::warp_max(amax);
                bar_softmax();
                if (lane == 0) red[64 + (warp - 2)] = amax;
                bar_softmax();
                if (warp == 2 && lane == 0)
                    p.amax_out[(size_t)b * p.kv_heads + kvh] = fmaxf(fmaxf(red[64], red[65]), fmaxf(red[66], red[67]));
            }
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---- host side -------------------------------------------------------------------------
inline PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(sym);
    });
    return fn;
}

// Paged cache [slots][kv_heads][HD] fp8 -> 3-D map, box = (128 B, 1 head, block_size slots), 128-byte swizzle.
struct MapKey {
    const void* p;
    long long slots;
    int kv_heads, hd, bs;
    bool operator==(const MapKey& o) const {
        return p == o.p && slots == o.slots && kv_heads == o.kv_heads && hd == o.hd && bs == o.bs;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.p) ^ ((size_t)k.slots * 1000003u) ^ ((size_t)k.kv_heads << 20) ^ ((size_t)k.hd << 8) ^ (size_t)k.bs;
    }
};
inline bool cache_map(CUtensorMap* out, const void* base, long long slots, int kv_heads, int hd, int bs) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    MapKey key{base, slots, kv_heads, hd, bs};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    auto fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)kv_heads, (cuuint64_t)slots};
    cuuint64_t strides[2] = {(cuuint64_t)hd, (cuuint64_t)hd * kv_heads};
    cuuint32_t box[3] = {(cuuint32_t)PANEL, 1u, (cuuint32_t)bs};
    cuuint32_t estr[3] = {1, 1, 1};
    if (fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, hd <= 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return true;
}

// Shapes this kernel takes: head_dim 128 or 256, at most 8 query heads per KV head, pages of 8..128
// tokens that tile 128, 16-byte aligned caches.
inline bool supports(const Params& p, int head_dim) {
    const int group = p.heads / p.kv_heads;
    return (head_dim == 128 || head_dim == 256) && group <= 8 && p.block_size >= 8 && p.block_size <= TOK &&
           TOK % p.block_size == 0 && (long long)p.num_blocks_total * p.block_size < (1ll << 31);
}

// Ring depth.  A shallow ring lets more CTAs share an SM (the footprint is 8-10 KB + 16 KB per unit), a
// deep one lets a CTA run further ahead of its softmax.  The choice minimises
// ceil(CTAs / resident CTAs) x (relative time of one wave), with the per-wave weights measured on the
// decode shapes (batch 8 / 32 / 128, contexts 576 to 4096).
template <int HD> inline int pick_units(long long ctas, int extra_bytes = 0) {
    using C = Cfg<HD>;
    struct Cand {
        int units;
        double wave;
    };
    static const Cand c128[] = {{2, 1.25}, {3, 1.0}, {4, 0.87}, {6, 0.74}};
    static const Cand c256[] = {{4, 1.15}, {6, 1.0}};
    const Cand* cand = C::HALVES == 1 ? c128 : c256;
    const int n = C::HALVES == 1 ? 4 : 2;
    int best = cand[0].units;
    double best_cost = 1e300;
    for (int i = 0; i < n; i++) {
        const long long slots = ((228 * 1024) / (C::smem_bytes(cand[i].units) + extra_bytes + 1024)) * 148ll;
        const double cost = (double)((ctas + slots - 1) / slots) * cand[i].wave;
        if (cost < best_cost) {
            best_cost = cost;
            best = cand[i].units;
        }
    }
    return best;
}

inline int read_status(int* out, bool reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -2;
    *out = v;
    if (reset && v != 0) {
        int z = 0;
        if (cudaMemcpyToSymbol(g_status, &z, sizeof(int)) != cudaSuccess) return -2;
    }
    return 0;
}

}  // namespace rvua
