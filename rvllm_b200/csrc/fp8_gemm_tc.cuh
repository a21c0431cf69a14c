// tcgen05 / TMEM FP8 E4M3 GEMM for sm_100a:
//     D[m, n] = epilogue( a_scale[m] * ( w_scale[n] * sum_k A[m, k] * W[n, k] ) )
// Same operand layout and epilogue contract as the streaming kernel (A [M, K], W [N, K],
// both row-major fp8; reference: kernels/cutlass_fp8_gemm_channelscale.cu:98-161,
// kernels/cutlass_fp8_gemm_residual.cu:48-83).
//
// The roles are swapped relative to a textbook GEMM so that decode-sized batches still
// fill the 128-lane tensor-core tile: a 128-row slab of W is the MMA's M operand, the
// batch rows are its N operand (16..256), so the accumulator in TMEM is D^T
// [128 weight rows (lanes) x BN batch rows (columns)] in f32.
//
//   warp 0   : TMA producer — one lane issues cp.async.bulk.tensor.2d loads of a
//              128 x 128 B weight tile and a BN x 128 B activation tile per stage
//              (128-byte swizzle), completion counted on an mbarrier per stage.
//   warp 1   : allocates TMEM, then one lane issues four tcgen05.mma (K = 32) per stage
//              and commits the stage's "empty" barrier; a final commit signals the
//              epilogue.
//   warps 2-5: epilogue — tcgen05.ld of the warp's 32-lane quarter, scales, optional
//              residual, narrow, store (64 B contiguous per batch row per warp).
//
// Split-K uses a thread-block cluster along K exactly like the streaming kernel: each
// CTA parks its f32 tile in its own (now idle) stage memory, the cluster synchronises,
// and each CTA finishes an interleaved share by reading its peers through DSMEM in a
// fixed order — no global scratch, no atomics, bitwise reproducible.  No multicast loads
// are used anywhere.
//
// Every mbarrier wait is bounded; when one runs out the kernel records it in a device
// status word, stops waiting, and still walks through every barrier and the TMEM
// release so that neither it nor its cluster peers hang.
#pragma once
#include <cooperative_groups.h>
#include <cuda.h>
#include <cudaTypedefs.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

#include "host_util.h"

#include "common.cuh"

namespace rvhost {
int fail_msg(int code, const char* msg);
}
bool rv_pdl_enabled();

namespace rvtc {

namespace cg = cooperative_groups;

constexpr int TILE_W = 128;   // weight rows per CTA (UMMA M)
constexpr int BK = 128;       // K bytes per stage (one 128-byte swizzle atom)
constexpr int UMMA_K = 32;    // K per tcgen05.mma for 8-bit operands
constexpr int THREADS = 192;
constexpr int EPI_WARP0 = 2;
constexpr uint32_t WAIT_LIMIT = 1u << 24;

__device__ int g_status = 0;  // 0 ok; otherwise (site << 16 | detail) of the first wait that gave up

// Extra operands of the fused QKV epilogue (EPI_QKV_ROPE): what the RoPE + KV-write kernel takes.
struct RopeKv {
    uint8_t* q_fp8;          // [M, heads, 128] E4M3
    float* q_scale;          // [M, heads]
    uint8_t* k_cache;        // paged [slots, kv_heads, 128] E4M3
    uint8_t* v_cache;
    float* k_scale;          // [slots, kv_heads]
    float* v_scale;
    const void* cos_t;       // [max_positions, 64] in the activation type
    const void* sin_t;
    const int* positions;    // [M]
    const int* slot_mapping; // [M]
    int heads, kv_heads, max_positions, num_cache_slots;
};

struct TcParams {
    const float* a_scale;
    const float* w_scale;
    void* out;
    const void* residual;
    int M, N, K;
    int kblocks;  // ceil(K / BK)
    int stages;   // depth of the TMA ring (2..MAX_STAGES); sets the shared-memory footprint
    int push;     // split-K partials are pushed into the finishing CTA's receive buffer (behind the ring)
    RopeKv rope;  // EPI_QKV_ROPE only
    // EPI_RESIDUAL_A16 only: the activation operand arrives as 16-bit values [M, K] plus `amax_parts` partial
    // maxima of |value| per row; the kernel derives the per-row scale and quantises its own A tiles
    const void* a16;
    const float* amax_part;
    int amax_parts;
    // EPI_ARGMAX only: nothing is stored but each weight tile's best (value, output channel) per batch row,
    // arg_val / arg_idx [M][tiles]; softcap > 0 applies cap * tanh(x / cap) to the value first
    float* arg_val;
    int* arg_idx;
    float softcap;
    // timing aid (null = off): 8 points x {earliest, latest} %globaltimer stamps over the CTAs of this launch
    unsigned long long* trace;
};

// ---- PTX wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
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

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// Cluster barrier halves and a 4-byte store into a cluster peer's shared memory.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
// Arrive (release, cluster scope) on the mbarrier at the same shared-memory offset in cluster rank `rank`.
__device__ __forceinline__ void mbar_arrive_peer(uint64_t* local_bar, uint32_t rank) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}" ::"r"(smem_u32(local_bar)), "r"(rank)
        : "memory");
}
// Bounded wait with cluster-scope acquire (the data was written by other CTAs of the cluster).
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, int site) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    atomicCAS(&g_status, 0, (site << 16) | (int)(blockIdx.x & 0xffff));
    return false;
}
__device__ __forceinline__ void st_peer_f32(uint32_t local_saddr, uint32_t rank, float v) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "st.shared::cluster.f32 [ra], %2;\n\t}" ::"r"(local_saddr), "r"(rank), "f"(v)
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
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile [rows x 128 B], 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);  // start address
    d |= (uint64_t)1 << 16;                            // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                            // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return d;
}
// kind::f8f6f4, E4M3 x E4M3 -> F32, both operands K-major, M = 128, N = BN.
__host__ __device__ constexpr uint32_t instr_desc(int bn) {
    return (1u << 4) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(TILE_W >> 4) << 24);
}

constexpr int EPI_SCALE = 0, EPI_RESIDUAL = 1, EPI_F32 = 2, EPI_QKV_ROPE = 3, EPI_RESIDUAL_A16 = 4, EPI_ARGMAX = 5;

// Greedy-argmax candidates: a candidate wins if its value is greater, or equal with a lower index; index -1 = no
// candidate (NaN is never one); -inf may win.  The rule of the reference's argmax kernels (kernels/argmax.cu:16-25).
__device__ __forceinline__ bool arg_better(float cv, int ci, float bv, int bi) {
    if (ci < 0) return false;
    if (bi < 0) return true;
    return cv > bv || (cv == bv && ci < bi);
}

// Timing aid: the earliest and the latest CTA to pass point k of a launch (rvllm_fp8_gemm_tc_trace).  Compiled in
// only with -DRVLLM_TC_TRACE=1: even switched off, the seven tests and calls cost the decode step 1.2 % (measured).
#ifndef RVLLM_TC_TRACE
#define RVLLM_TC_TRACE 0
#endif
__device__ __forceinline__ void trace_point(unsigned long long* tr, int k) {
#if RVLLM_TC_TRACE
    if (tr != nullptr) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        atomicMin(tr + 2 * k, t);
        atomicMax(tr + 2 * k + 1, t);
    }
#else
    (void)tr;
    (void)k;
#endif
}

// Meeting point of the four epilogue warps alone (named barrier 1; the block-wide barrier is 0).
__device__ __forceinline__ void epi_warps_sync() {
    __syncwarp();
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

constexpr int MAX_STAGES = 8;
constexpr int HEADER_BYTES = 1024;  // barriers + TMEM address holder, in front of the ring

template <int BN> struct Cfg {
    static constexpr int STAGE_BYTES = TILE_W * BK + BN * BK;
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    // stages needed so that the split-K partial tile [BN][128] f32 fits in the (idle) ring
    static constexpr int MIN_STAGES = (TILE_W * BN * 4 + STAGE_BYTES - 1) / STAGE_BYTES < 2
                                          ? 2 : (TILE_W * BN * 4 + STAGE_BYTES - 1) / STAGE_BYTES;
    // receive buffer of the push reduction: [S][ceil(BN / S)][TILE_W] f32, S * ceil(BN / S) <= BN + 7
    static constexpr int RECV_BYTES = (BN + 7) * TILE_W * 4;
    static constexpr int smem_bytes(int stages, bool push = false) {
        return 1024 /*alignment slack*/ + HEADER_BYTES + stages * STAGE_BYTES + (push ? RECV_BYTES : 0);
    }
};

template <int BN, int EPI, typename OutT>
__global__ void __launch_bounds__(THREADS, 1)
fp8_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, TcParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t raw[];
    uint8_t* header = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = header + HEADER_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(header);
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* acc_ready = empty + MAX_STAGES;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_ready + 1);
    uint64_t* recv_bar = reinterpret_cast<uint64_t*>(header + 512);  // push reduction: all partials for this CTA have landed
    uint64_t* free_bar = recv_bar + 1;                               // ring push: every CTA of the cluster is done with its ring
    const int STAGES = p.stages;

    cg::cluster_group cluster = cg::this_cluster();
    const int S = gridDim.y, split = blockIdx.y;
    const int n0 = blockIdx.x * TILE_W, m0 = blockIdx.z * BN;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb_lo = (int)((long long)split * p.kblocks / S);
    const int kb_hi = (int)((long long)(split + 1) * p.kblocks / S);
    const int nkb = kb_hi - kb_lo;

    constexpr bool A16 = EPI == EPI_RESIDUAL_A16;           // A tiles are quantised here from 16-bit activations
    constexpr bool RES = EPI == EPI_RESIDUAL || A16;        // residual epilogue
    __shared__ float s_ascale[A16 ? BN : 1], s_ainv[A16 ? BN : 1];
    constexpr bool ARG = EPI == EPI_ARGMAX;                 // per-tile argmax partials instead of stored logits
    __shared__ float s_as[A16 ? 1 : BN];                    // unsplit epilogue: the batch rows' activation scales
    auto a_scale_of = [&](int m) -> float { return A16 ? s_ascale[m - m0] : p.a_scale[m]; };
    rv::pdl_launch();
    if (threadIdx.x == 0) {
        trace_point(p.trace, 0);  // the CTA runs
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full + s, A16 ? 5 : 1);  // the producer's arrival (+ one per converting warp)
            mbar_init(empty + s, 1);
        }
        mbar_init(acc_ready, 1);
        mbar_init(recv_bar, (uint32_t)gridDim.y * 4u);  // one arrival per epilogue warp of every CTA of the cluster
        mbar_init(free_bar, (uint32_t)gridDim.y);       // one arrival per CTA of the cluster
        fence_barrier_init();
        // This thread is also the TMA producer.  Weights never depend on the previous kernel: fill the ring
        // with weight tiles right away (before the block even meets; the barriers are this thread's own),
        // the activation tiles of those stages follow once the predecessor is done.
        const int pre = nkb < STAGES ? nkb : STAGES;
        for (int i = 0; i < pre; i++) {
            mbar_expect_tx(full + i, A16 ? TILE_W * BK : C::STAGE_BYTES);
            tma_load_2d(ring + (size_t)i * C::STAGE_BYTES, &map_w, (kb_lo + i) * BK, n0, full + i);
        }
    }
    if (warp == 1) tmem_alloc(tmem_holder, C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    // 16-bit activation form: the converting warps' first K block of values, fetched one block ahead of its use
    constexpr int CPT = (BN * 8 + 127) / 128;  // 16-byte output chunks per thread and K block (1 or 2)
    uint4 nx[A16 ? CPT : 1][2];
    auto fetch_a16 = [&](int i) {
        if constexpr (A16) {
            const int t = (int)threadIdx.x - EPI_WARP0 * 32;
            const OutT* a16 = reinterpret_cast<const OutT*>(p.a16);
#pragma unroll
            for (int q = 0; q < CPT; q++) {  // this thread's chunks: row r, 16-column group cc — the same for every K block
                const int c = t + q * 128, r = c >> 3, cc = c & 7;
                const int m = m0 + r, k0 = (kb_lo + i) * BK + cc * 16;
                nx[q][0] = nx[q][1] = make_uint4(0, 0, 0, 0);
                if (c < BN * 8 && i < nkb && m < p.M && k0 < p.K) {
                    const uint4* src = reinterpret_cast<const uint4*>(a16 + (size_t)m * p.K + k0);
                    nx[q][0] = rv::ldg128(src);
                    nx[q][1] = rv::ldg128(src + 1);
                }
            }
        }
    };
    if (A16) {
        // per-row activation scale from the partial maxima the producer of the activations left behind; the
        // converting warps' first loads go out beside those of the maxima, not after them
        rv::pdl_wait();
        if (warp >= EPI_WARP0) fetch_a16(0);
        if ((int)threadIdx.x < BN) {
            const int m = m0 + (int)threadIdx.x;
            float amax = 0.0f;
            if (m < p.M)
                for (int q = 0; q < p.amax_parts; q++) amax = fmaxf(amax, p.amax_part[(size_t)m * p.amax_parts + q]);
            const float sc = rv::row_scale(amax);
            s_ascale[threadIdx.x] = sc;
            s_ainv[threadIdx.x] = 1.0f / sc;
        }
        __syncthreads();
        if (threadIdx.x == 0) trace_point(p.trace, 1);  // predecessor complete, row scales known
    }
    const bool push = S > 1 && p.push != 0;
    // push == 3: the receive buffer is the (by then idle) ring itself — batch tiles of 64 / 128 rows, whose partials
    // would not fit behind it.  The cluster then meets after the main loops instead ("every ring is free").
    const bool push_ring = BN >= 64 && push && p.push >= 3;  // (a compile-time "no" for the small tiles)
    const bool push_mbar = p.push == 2 || p.push == 3;       // completion: arrivals on the owners' mbarriers (else a cluster barrier)
    // "this CTA runs": peers wait for it (long since complete) before their first remote store or arrival
    if (push && (!push_ring || push_mbar)) cluster_arrive();

    if (warp == 0) {
        if (lane == 0) {
            const int pre = nkb < STAGES ? nkb : STAGES;  // (their weight tiles are already on the way)
            if (!A16) {
                rv::pdl_wait();
                trace_point(p.trace, 1);  // the kernel ahead in the stream is complete
                for (int i = 0; i < pre; i++)
                    tma_load_2d(ring + (size_t)i * C::STAGE_BYTES + TILE_W * BK, &map_a, (kb_lo + i) * BK, m0, full + i);
            }
            bool alive = true;
            for (int i = pre; i < nkb; i++) {
                const int s = i % STAGES;
                const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
                alive = mbar_wait(empty + s, ph ^ 1u, 1);
                if (!alive) break;
                uint8_t* w_dst = ring + (size_t)s * C::STAGE_BYTES;
                mbar_expect_tx(full + s, A16 ? TILE_W * BK : C::STAGE_BYTES);
                tma_load_2d(w_dst, &map_w, (kb_lo + i) * BK, n0, full + s);
                if (!A16) tma_load_2d(w_dst + TILE_W * BK, &map_a, (kb_lo + i) * BK, m0, full + s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN);
            bool alive = true;
            for (int i = 0; i < nkb && alive; i++) {
                const int s = i % STAGES;
                const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
                alive = mbar_wait(full + s, ph, 2);
                if (!alive) break;
                if (i == 0) trace_point(p.trace, 2);  // both operands of the first K block are in shared memory
                tc_fence_after();
                const uint32_t w_addr = smem_u32(ring + (size_t)s * C::STAGE_BYTES);
                const uint64_t adesc = smem_desc_sw128(w_addr);
                const uint64_t bdesc = smem_desc_sw128(w_addr + TILE_W * BK);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; k++)
                    umma_f8(tmem_base, adesc + (uint64_t)(k * UMMA_K >> 4), bdesc + (uint64_t)(k * UMMA_K >> 4), idesc,
                            (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty + s);  // frees the stage once these MMAs have read it
            }
            umma_commit(acc_ready);  // arrives when every MMA issued above has completed
            trace_point(p.trace, 3);  // the last MMA is issued
        }
    }
    if (A16 && warp >= EPI_WARP0) {
        // The four epilogue warps are idle during the main loop: they turn the 16-bit activations into the
        // swizzled FP8 A tiles themselves (the per-token quantiser's arithmetic: scale = max(absmax / 448,
        // 1e-12), code = e4m3(x * (1 / scale))), so no separate quantiser launch and no FP8 copy in HBM.
        const int t = (int)threadIdx.x - EPI_WARP0 * 32;
        bool alive = true;
        for (int i = 0; i < nkb && alive; i++) {
            uint4 cur[CPT][2];
#pragma unroll
            for (int q = 0; q < CPT; q++) {
                cur[q][0] = nx[q][0];
                cur[q][1] = nx[q][1];
            }
            fetch_a16(i + 1);
            const int s = i % STAGES;
            if (i >= STAGES) alive = mbar_wait(empty + s, ((uint32_t)(i / STAGES) & 1u) ^ 1u, 5);
            if (!alive) break;
            uint8_t* a_tile = ring + (size_t)s * C::STAGE_BYTES + TILE_W * BK;
#pragma unroll
            for (int q = 0; q < CPT; q++) {
                const int c = t + q * 128, r = c >> 3, cc = c & 7;
                if (c < BN * 8) {
                    const float inv = s_ainv[r];
                    const uint32_t xs[8] = {cur[q][0].x, cur[q][0].y, cur[q][0].z, cur[q][0].w,
                                            cur[q][1].x, cur[q][1].y, cur[q][1].z, cur[q][1].w};
                    uint32_t w4[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float2 a = rv::T16<OutT>::to_f32x2(xs[2 * j]), b = rv::T16<OutT>::to_f32x2(xs[2 * j + 1]);
                        w4[j] = rv::f32x4_to_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
                    }
                    // (rows past M and columns past K were fetched as zeros: code 0)
                    *reinterpret_cast<uint4*>(a_tile + r * BK + ((cc ^ (r & 7)) << 4)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(full + s);
        }
    }
    __syncwarp();
    rv::pdl_wait();  // scales and the residual come from predecessors; also keeps completion ordered

    // ---- epilogue ----------------------------------------------------------------------
    if (push) {
        // Split-K, push form.  Batch column c of the tile is finished by the CTA of cluster rank c % S.
        // Every CTA stores its partial of column c straight into that CTA's receive buffer (slot = its
        // own rank), the cluster meets once, and each CTA sums the S slots of its columns in rank order:
        // one barrier, no remote loads, bitwise reproducible.  Measured ~2.5 us per launch less than
        // pulling the partials out of the peers' rings (two barriers and a remote-load round trip).
        float* recv = reinterpret_cast<float*>(push_ring ? ring : ring + (size_t)STAGES * C::STAGE_BYTES);  // [S][LC][TILE_W]
        const int LC = (BN + S - 1) / S;
        constexpr int PRE = 3;
        float pre_a[PRE], pre_w[PRE], pre_res[PRE];
#pragma unroll
        for (int j = 0; j < PRE; j++) {  // scales and residual of this thread's first output elements
            const int e = (int)threadIdx.x + j * THREADS;
            const int col = (e / TILE_W) * S + split;
            const int m = m0 + col, n = n0 + e % TILE_W;
            pre_a[j] = pre_w[j] = pre_res[j] = 0.0f;
            if (e < LC * TILE_W && col < BN && m < p.M && n < p.N) {
                pre_a[j] = a_scale_of(m);
                pre_w[j] = p.w_scale[n];
                if (RES)
                    pre_res[j] = rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(p.residual)[(size_t)m * p.N + n]);
            }
        }
        // Fused QKV epilogue: everything its first two rounds of tokens need besides the sums — activation scale,
        // position, cache slot, and (dependent on the position) the cos / sin pair — is fetched here, while the
        // main loop still runs; fetched inside the rounds, these are three L2 round trips in a row per round.
        constexpr int QPRE = 2;
        float q_as[QPRE], q_c[QPRE], q_s[QPRE], q_wlo = 0.0f, q_whi = 0.0f;
        int q_pos[QPRE], q_slot[QPRE];
        if constexpr (EPI == EPI_QKV_ROPE) {
            const RopeKv& rk = p.rope;
            const int grp = (int)threadIdx.x >> 6, d = (int)threadIdx.x & 63;
            const int kind = (int)blockIdx.x < rk.heads ? 0 : ((int)blockIdx.x < rk.heads + rk.kv_heads ? 1 : 2);
            q_wlo = p.w_scale[n0 + d];
            q_whi = p.w_scale[n0 + d + 64];
#pragma unroll
            for (int it = 0; it < QPRE; it++) {
                const int lc = it * 3 + grp, col = lc * S + split, m = m0 + col;
                q_as[it] = q_c[it] = q_s[it] = 0.0f;
                q_pos[it] = q_slot[it] = -1;
                if (lc < LC && col < BN && m < p.M) {
                    q_as[it] = a_scale_of(m);
                    q_pos[it] = rk.positions[m];
                    if (kind != 0) q_slot[it] = rk.slot_mapping[m];
                    if (kind != 2 && q_pos[it] >= 0 && q_pos[it] < rk.max_positions) {
                        q_c[it] = rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(rk.cos_t)[(size_t)q_pos[it] * 64 + d]);
                        q_s[it] = rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(rk.sin_t)[(size_t)q_pos[it] * 64 + d]);
                    }
                }
            }
        }
        bool ready = true;
        if (push_ring) {
            // own MMAs complete = every load into this CTA's ring has landed and been read: the ring is free;
            // once the whole cluster has said so, every ring may be written
            if (warp >= EPI_WARP0 && nkb > 0) ready = mbar_wait(acc_ready, 0, 3);
            if (threadIdx.x == EPI_WARP0 * 32) trace_point(p.trace, 4);  // the accumulator is complete
            if (push_mbar) {
                // one warp tells every CTA of the cluster (itself included); the pushing warps wait for all of them
                cluster_wait();  // (every CTA runs: its barriers exist)
                if (warp == EPI_WARP0) {
                    __syncwarp();
                    if (lane < S) mbar_arrive_peer(free_bar, (uint32_t)lane);
                }
                if (warp >= EPI_WARP0) mbar_wait_cluster(free_bar, 0, 8);
            } else {
                cluster_arrive();
            }
        }
        if (!(push_ring && push_mbar)) cluster_wait();  // every CTA of the cluster is running (and, in the ring + barrier form, done with its ring)
        if (warp >= EPI_WARP0) {
            const int quarter = warp & 3;
            const int r = quarter * 32 + lane;
            if (!push_ring && nkb > 0) ready = mbar_wait(acc_ready, 0, 3);
            if (!push_ring && threadIdx.x == EPI_WARP0 * 32) trace_point(p.trace, 4);  // the accumulator is complete
            tc_fence_after();
            const uint32_t slot = smem_u32(recv) + (uint32_t)((split * LC) * TILE_W + r) * 4u;  // [split][0][r]
            uint32_t owner = 0, lc_off = 0;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t v[16];
                if (nkb > 0 && ready) {
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    st_peer_f32(slot + lc_off, owner, __uint_as_float(v[j]));
                    if (++owner == (uint32_t)S) {
                        owner = 0;
                        lc_off += TILE_W * 4;
                    }
                }
            }
            tc_fence_before();
            if (push_mbar) {
                // point-to-point completion: tell every owner that this warp's partials for it are in place
                asm volatile("fence.acq_rel.cluster;" ::: "memory");
                __syncwarp();
                if (lane < S) mbar_arrive_peer(recv_bar, (uint32_t)lane);
            }
        }
        if (push_mbar) {
            mbar_wait_cluster(recv_bar, 0, 4);
        } else {
            cluster_arrive();
            cluster_wait();
        }
        if (threadIdx.x == 0) trace_point(p.trace, 5);  // the partials of this CTA's columns are in its receive buffer
        if constexpr (EPI == EPI_QKV_ROPE) {
            // Fused QKV epilogue.  The weight tile is one head (128 output channels): this CTA holds, for
            // each batch column it finishes, the whole head of one token.  Round to the activation type (the
            // bytes the unfused GEMM would have stored), rotate (half-split pairs d, d + 64), take the head's
            // absmax, quantise, and write Q / the paged K or V cache with their scales — the arithmetic of
            // the RoPE + KV-write kernel (v3/kernels/fused_rope_partial_fp8kv.cu:54-214), without the 16-bit
            // round trip through HBM and without the extra launch.  64 threads per token, 3 tokens at a time.
            __shared__ float s_amax[2][3][2];  // [round parity][token group][warp of the group]
            const RopeKv& rk = p.rope;
            const int tile = blockIdx.x;                       // == head index over Q heads, then K heads, then V heads
            const int kind = tile < rk.heads ? 0 : (tile < rk.heads + rk.kv_heads ? 1 : 2);
            const int head = kind == 0 ? tile : (kind == 1 ? tile - rk.heads : tile - rk.heads - rk.kv_heads);
            const int grp = (int)threadIdx.x >> 6, d = (int)threadIdx.x & 63;
            const float ws_lo = q_wlo, ws_hi = q_whi;
            for (int lc0 = 0; lc0 < LC; lc0 += 3) {            // uniform trip count: the barriers below are block-wide
                const int lc = lc0 + grp;
                const int col = lc * S + split, m = m0 + col;
                const bool live = lc < LC && col < BN && m < p.M;
                const int it = lc0 / 3;                         // rounds 0 and 1 were fetched ahead
                float lo = 0.0f, hi = 0.0f;
                int pos = -1;
                if (live) {
                    float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
                    for (int sp = 0; sp < 8; sp++)
                        if (sp < S) {
                            sum_lo += recv[(size_t)(sp * LC + lc) * TILE_W + d];
                            sum_hi += recv[(size_t)(sp * LC + lc) * TILE_W + d + 64];
                        }
                    const float as = it < QPRE ? q_as[it < QPRE ? it : 0] : a_scale_of(m);
                    const float a = rv::T16<OutT>::to_f32(rv::T16<OutT>::from_f32_sat(as * (ws_lo * sum_lo)));
                    const float b = rv::T16<OutT>::to_f32(rv::T16<OutT>::from_f32_sat(as * (ws_hi * sum_hi)));
                    pos = it < QPRE ? q_pos[it < QPRE ? it : 0] : rk.positions[m];
                    lo = a;
                    hi = b;
                    if (kind != 2 && pos >= 0 && pos < rk.max_positions) {
                        float c, sn;
                        if (it < QPRE) {
                            c = q_c[it < QPRE ? it : 0];
                            sn = q_s[it < QPRE ? it : 0];
                        } else {
                            c = rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(rk.cos_t)[(size_t)pos * 64 + d]);
                            sn = rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(rk.sin_t)[(size_t)pos * 64 + d]);
                        }
                        lo = a * c - b * sn;
                        hi = a * sn + b * c;
                    }
                }
                // head absmax over the group's 64 threads (+inf carries "a value was not finite")
                float am = (!isfinite(lo) || !isfinite(hi)) ? CUDART_INF_F : fmaxf(fabsf(lo), fabsf(hi));
                am = rv::warp_max(am);
                // the two warps of a token group meet on a barrier of their own (ids 2-4), once per round: the
                // rounds alternate between two copies of the scratch, and a warp cannot reach the round after next
                // before its partner has read this one
                float* sa = s_amax[it & 1][grp];
                if ((threadIdx.x & 31) == 0) sa[(threadIdx.x >> 5) & 1] = am;
                asm volatile("bar.sync %0, 64;" ::"r"(2 + grp) : "memory");
                am = fmaxf(sa[0], sa[1]);
                if (live && pos >= 0 && pos < rk.max_positions) {
                    const float sc = isinf(am) ? CUDART_NAN_F : fmaxf(am / 448.0f, 1e-12f);
                    const float inv = 1.0f / sc;
                    if (kind == 0) {
                        uint8_t* o = rk.q_fp8 + ((size_t)m * rk.heads + head) * TILE_W;
                        o[d] = rv::f32_to_e4m3(lo * inv);
                        o[d + 64] = rv::f32_to_e4m3(hi * inv);
                        if (d == 0) rk.q_scale[(size_t)m * rk.heads + head] = sc;
                    } else {
                        const int slot = it < QPRE ? q_slot[it < QPRE ? it : 0] : rk.slot_mapping[m];
                        if (slot >= 0 && slot < rk.num_cache_slots) {
                            const size_t sidx = (size_t)slot * rk.kv_heads + head;
                            uint8_t* o = (kind == 1 ? rk.k_cache : rk.v_cache) + sidx * TILE_W;
                            o[d] = rv::f32_to_e4m3(lo * inv);
                            o[d + 64] = rv::f32_to_e4m3(hi * inv);
                            if (d == 0) (kind == 1 ? rk.k_scale : rk.v_scale)[sidx] = sc;
                        }
                    }
                }
            }
        } else {
        auto finish = [&](int e, bool pre, float as_p, float ws_p, float res_p) {
            const int lc = e / TILE_W, r = e % TILE_W;
            const int col = lc * S + split;
            const int m = m0 + col, n = n0 + r;
            if (e >= LC * TILE_W || col >= BN || m >= p.M || n >= p.N) return;
            float sum = 0.0f;
#pragma unroll
            for (int sp = 0; sp < 8; sp++)
                if (sp < S) sum += recv[(size_t)(sp * LC + lc) * TILE_W + r];
            const float as = pre ? as_p : a_scale_of(m);
            const float ws = pre ? ws_p : p.w_scale[n];
            const size_t o = (size_t)m * p.N + n;
            if (EPI == EPI_F32) {
                reinterpret_cast<float*>(p.out)[o] = as * (ws * sum);  // same association as the unsplit epilogue
            } else {
                float val;
                if (RES)  // one rounding for scale-and-add, spelled out so that every form of the epilogue agrees
                    val = fmaf(as, ws * sum, pre ? res_p : rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(p.residual)[o]));
                else
                    val = as * (ws * sum);
                reinterpret_cast<OutT*>(p.out)[o] = rv::T16<OutT>::from_f32_sat(val);
            }
        };
#pragma unroll
        for (int j = 0; j < PRE; j++) finish((int)threadIdx.x + j * THREADS, true, pre_a[j], pre_w[j], pre_res[j]);
        // (larger batch tiles: the rest in groups as well — loads of a group before its stores, see the pull form)
#pragma unroll 1
        for (int e0 = (int)threadIdx.x + PRE * THREADS; e0 < LC * TILE_W; e0 += PRE * THREADS) {
            float g_a[PRE], g_w[PRE], g_res[PRE];
#pragma unroll
            for (int j = 0; j < PRE; j++) {
                const int e = e0 + j * THREADS;
                const int col = (e / TILE_W) * S + split;
                const int m = m0 + col, n = n0 + e % TILE_W;
                g_a[j] = g_w[j] = g_res[j] = 0.0f;
                if (e < LC * TILE_W && col < BN && m < p.M && n < p.N) {
                    g_a[j] = a_scale_of(m);
                    g_w[j] = p.w_scale[n];
                    if (RES)
                        g_res[j] = rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(p.residual)[(size_t)m * p.N + n]);
                }
            }
#pragma unroll
            for (int j = 0; j < PRE; j++) finish(e0 + j * THREADS, true, g_a[j], g_w[j], g_res[j]);
        }
        }
    } else if (EPI != EPI_QKV_ROPE) {  // (the fused QKV epilogue exists in the push form only; the host launches no other)
    float* part = reinterpret_cast<float*>(ring);  // [BN][TILE_W] f32: split-K partials, or the logits of the argmax form
    if (warp >= EPI_WARP0) {
        const int quarter = warp & 3;  // TMEM lanes this warp may touch: 32 * quarter ...
        const int r = quarter * 32 + lane;
        const int n = n0 + r;
        // Everything the epilogue needs besides the accumulator is fetched while the main loop still runs: a load
        // inside the column loop below cannot be moved above the stores between the columns, so each column
        // would pay a trip to L2 after the last MMA.
        const float ws = (n < p.N) ? p.w_scale[n] : 0.0f;
        if constexpr (!A16) {
            if (S == 1) {
                for (int c = r; c < BN; c += 128) s_as[c] = (m0 + c < p.M) ? p.a_scale[m0 + c] : 0.0f;
                epi_warps_sync();
            }
        }
        auto as_col = [&](int c) -> float { return A16 ? s_ascale[c] : s_as[c]; };  // (S == 1 only)
        // residual values one 16-column group ahead (out and residual may be one buffer: every element is read
        // before any store of its group, and by the thread that stores it)
        // (256-row batch tiles only, which run one CTA per SM: the smaller ones count on three, and the registers
        // this costs would take the third away)
        constexpr bool RES_AHEAD = RES && BN >= 256;
        float res_nx[RES_AHEAD ? 16 : 1];
        auto fetch_res = [&](int c0) {
            if constexpr (RES_AHEAD) {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int m = m0 + c0 + j;
                    res_nx[j] = (S == 1 && c0 + j < BN && m < p.M && n < p.N)
                                    ? rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(p.residual)[(size_t)m * p.N + n])
                                    : 0.0f;
                }
            }
        };
        fetch_res(0);
        bool ready = true;
        if (nkb > 0) ready = mbar_wait(acc_ready, 0, 3);
        if (threadIdx.x == EPI_WARP0 * 32) trace_point(p.trace, 4);  // the accumulator is complete
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
            uint32_t v[16];
            if (nkb > 0 && ready) {
                tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) v[j] = 0u;
            }
            float res_cur[RES_AHEAD ? 16 : 1];
            if constexpr (RES_AHEAD) {
#pragma unroll
                for (int j = 0; j < 16; j++) res_cur[j] = res_nx[j];
                if (S == 1) fetch_res(c0 + 16);
            }
            if constexpr (ARG) {
                // the logit this element would have been (soft-capped), into the idle ring as [batch row][channel]
                const float inv_cap = p.softcap > 0.0f ? 1.0f / p.softcap : 0.0f;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    float val = as_col(c0 + j) * (ws * __uint_as_float(v[j]));
                    if (p.softcap > 0.0f) val = p.softcap * tanhf(val * inv_cap);
                    part[(size_t)(c0 + j) * TILE_W + r] = val;
                }
            } else if (S > 1) {
#pragma unroll
                for (int j = 0; j < 16; j++) part[(size_t)(c0 + j) * TILE_W + r] = __uint_as_float(v[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int m = m0 + c0 + j;
                    if (m < p.M && n < p.N) {
                        float val = as_col(c0 + j) * (ws * __uint_as_float(v[j]));
                        const size_t o = (size_t)m * p.N + n;
                        if (EPI == EPI_F32) {
                            reinterpret_cast<float*>(p.out)[o] = val;
                        } else {
                            if (RES)
                                val = fmaf(as_col(c0 + j), ws * __uint_as_float(v[j]),
                                           RES_AHEAD ? res_cur[RES_AHEAD ? j : 0]
                                                     : rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(p.residual)[o]));
                            reinterpret_cast<OutT*>(p.out)[o] = rv::T16<OutT>::from_f32_sat(val);
                        }
                    }
                }
            }
        }
        tc_fence_before();
        if constexpr (ARG) {
            // The tile's winner per batch row.  Four threads share a row, 32 channels each; lane l starts at
            // channel l of its quarter, so the 32 lanes of a warp read 32 different banks.  The candidate rule
            // does not depend on the order in which candidates meet.
            epi_warps_sync();
            const int t = (int)threadIdx.x - EPI_WARP0 * 32, q = t & 3;
            for (int c = t >> 2; c < BN; c += 32) {
                float bv = -CUDART_INF_F;
                int bi = -1;
                const float* rowp = part + (size_t)c * TILE_W + q * 32;
#pragma unroll 8
                for (int i = 0; i < 32; i++) {
                    const int ch = (i + lane) & 31;
                    const float val = rowp[ch];
                    const int idx = n0 + q * 32 + ch;
                    if (val == val && idx < p.N && arg_better(val, idx, bv, bi)) {
                        bv = val;
                        bi = idx;
                    }
                }
#pragma unroll
                for (int o = 1; o <= 2; o <<= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (arg_better(ov, oi, bv, bi)) {
                        bv = ov;
                        bi = oi;
                    }
                }
                if (q == 0 && m0 + c < p.M) {
                    p.arg_val[(size_t)(m0 + c) * gridDim.x + blockIdx.x] = bv;
                    p.arg_idx[(size_t)(m0 + c) * gridDim.x + blockIdx.x] = bi;
                }
            }
        }
    }
    if (S > 1) {
        // This CTA finishes elements e = split*THREADS + tid (+ k * S*THREADS).  Their scales and residual
        // values do not depend on the MMAs: fetch the first few before the cluster meets, so that their
        // latency is not added to the end of the kernel.
        constexpr int PRE = 4;
        const int e_first = split * THREADS + (int)threadIdx.x, e_step = S * THREADS;
        float pre_a[PRE], pre_w[PRE], pre_res[PRE];
#pragma unroll
        for (int j = 0; j < PRE; j++) {
            const int e = e_first + j * e_step;
            pre_a[j] = 0.0f;
            pre_w[j] = 0.0f;
            pre_res[j] = 0.0f;
            if (e < BN * TILE_W) {
                const int m = m0 + e / TILE_W, n = n0 + e % TILE_W;
                if (m < p.M && n < p.N) {
                    pre_a[j] = a_scale_of(m);
                    pre_w[j] = p.w_scale[n];
                    if (RES)
                        pre_res[j] = rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(p.residual)[(size_t)m * p.N + n]);
                }
            }
        }
        cluster.sync();
        const float* peer[8];
#pragma unroll
        for (int s = 0; s < 8; s++) peer[s] = s < S ? cluster.map_shared_rank(part, s) : part;
        // same association as the unsplit epilogue: a_scale * (w_scale * sum)
        auto finish = [&](int e, float sum, float as, float ws, bool have_res, float res) {
            const int m = m0 + e / TILE_W, n = n0 + e % TILE_W;
            if (m < p.M && n < p.N) {
                const size_t o = (size_t)m * p.N + n;
                float val = as * (ws * sum);
                if (EPI == EPI_F32) {
                    reinterpret_cast<float*>(p.out)[o] = val;
                } else {
                    if (RES)
                        val = fmaf(as, ws * sum, have_res ? res : rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(p.residual)[o]));
                    reinterpret_cast<OutT*>(p.out)[o] = rv::T16<OutT>::from_f32_sat(val);
                }
            }
        };
        float sums[PRE];
#pragma unroll
        for (int j = 0; j < PRE; j++) {
            const int e = e_first + j * e_step;
            float sum = 0.0f;
            if (e < BN * TILE_W) {
#pragma unroll
                for (int s = 0; s < 8; s++)
                    if (s < S) sum += peer[s][e];
            }
            sums[j] = sum;
        }
        int e_rest_done = 0;
        if (e_first + PRE * e_step >= BN * TILE_W) {
            // every peer read of this CTA is done: let the others leave as soon as they are done too
            asm volatile("barrier.cluster.arrive.release;" ::: "memory");
            e_rest_done = 1;
        }
#pragma unroll
        for (int j = 0; j < PRE; j++) {
            const int e = e_first + j * e_step;
            if (e < BN * TILE_W) finish(e, sums[j], pre_a[j], pre_w[j], true, pre_res[j]);
        }
        // The rest in groups of PRE as well: all loads of a group, then its stores.  (A load placed after a
        // store cannot be moved above it — out and residual may be one buffer — so element-by-element code
        // pays a full load latency per element.)
        for (int e0 = e_first + PRE * e_step; e0 < BN * TILE_W; e0 += PRE * e_step) {
            float g_sum[PRE], g_a[PRE], g_w[PRE], g_res[PRE];
#pragma unroll
            for (int j = 0; j < PRE; j++) {
                const int e = e0 + j * e_step;
                g_sum[j] = g_a[j] = g_w[j] = g_res[j] = 0.0f;
                if (e < BN * TILE_W) {
                    float sum = 0.0f;
#pragma unroll
                    for (int s = 0; s < 8; s++)
                        if (s < S) sum += peer[s][e];
                    g_sum[j] = sum;
                    const int m = m0 + e / TILE_W, n = n0 + e % TILE_W;
                    if (m < p.M && n < p.N) {
                        g_a[j] = a_scale_of(m);
                        g_w[j] = p.w_scale[n];
                        if (RES)
                            g_res[j] = rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(p.residual)[(size_t)m * p.N + n]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < PRE; j++) {
                const int e = e0 + j * e_step;
                if (e < BN * TILE_W) finish(e, g_sum[j], g_a[j], g_w[j], true, g_res[j]);
            }
        }
        if (!e_rest_done) asm volatile("barrier.cluster.arrive.release;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    }
    }
    __syncthreads();
    if (threadIdx.x == 0) trace_point(p.trace, 6);  // every output of the CTA is stored
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// Second half of the fused greedy tail: the row's winner over the per-tile winners.  grid = rows, block = 256.
__global__ void __launch_bounds__(256) argmax_merge_kernel(const float* __restrict__ val, const int* __restrict__ idx,
                                                          int tiles, int* __restrict__ out) {
    __shared__ float sv[8];
    __shared__ int si[8];
    rv::pdl_launch();
    rv::pdl_wait();
    const int row = blockIdx.x;
    float bv = -CUDART_INF_F;
    int bi = -1;
    for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
        const float v = val[(size_t)row * tiles + t];
        const int i = idx[(size_t)row * tiles + t];
        if (arg_better(v, i, bv, bi)) {
            bv = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (arg_better(ov, oi, bv, bi)) {
            bv = ov;
            bi = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = bv;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++)
            if (arg_better(sv[w], si[w], bv, bi)) {
                bv = sv[w];
                bi = si[w];
            }
        out[row] = bi;
    }
}

// ---- host side -------------------------------------------------------------------------
struct TcArgs {
    void* out;
    int out_kind;
    const void* a;
    const void* w;
    const float* a_scale;
    const float* w_scale;
    const void* residual;
    int M, N, K;
    const void* a16 = nullptr;          // EPI_RESIDUAL_A16: 16-bit activations instead of `a` / `a_scale`
    const float* amax_part = nullptr;
    int amax_parts = 0;
    float* arg_val = nullptr;           // EPI_ARGMAX
    int* arg_idx = nullptr;
    float softcap = 0.0f;
};

inline size_t workspace_bytes(int, int, int) { return 0; }

// Which shapes go to the tensor-core kernel when the caller lets the library choose: all of
// them.  Measured at M = 1, 32 and 128 on the decode shapes it is as fast or faster than the
// mma.sync streaming kernel, which stays selectable (impl = 1) as an independent cross-check.
inline bool prefer_tc(int M, int N, int K) {
    (void)M;
    (void)N;
    return K % 16 == 0;
}

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

// Row-major fp8 matrix [rows, K] -> 2-D map with a (128 B x box_rows) box, 128-byte swizzle,
// zero fill outside the matrix (covers a ragged last K block and rows past the end).
inline bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    auto fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct MapKey {
    const void* p;
    int rows, K, box;
    bool operator==(const MapKey& o) const { return p == o.p && rows == o.rows && K == o.K && box == o.box; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.p) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.K << 20) ^ (size_t)k.box;
    }
};
// Tensor maps are pure functions of (pointer, shape); cache them so a decode step that
// reuses its buffers does not re-encode.
inline bool cached_map(CUtensorMap* out, const void* base, int rows, int K, int box) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    MapKey key{base, rows, K, box};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    if (!make_map(out, base, rows, K, box)) return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return true;
}

// Experiment hooks (0 = automatic): ring depth and split-K factor.
struct Tune {
    std::atomic<int> stages{0};
    std::atomic<int> splits{0};
    std::atomic<int> reduce{0};  // 1: force the pull form of the split-K reduction; 3: push completed by a cluster barrier (0 / 2: by mbarrier arrivals)
    std::atomic<int> split_target{0};  // CTAs a split launch aims for (0: the built-in 360)
    std::atomic<long long> split_for[4] = {};  // per-shape overrides: (N << 40) | (K << 8) | splits, 0 = unused
    std::atomic<unsigned long long*> trace{nullptr};  // timing aid: [trace_slots][16] u64 on the device, or null
    std::atomic<int> trace_slots{0};
    std::atomic<int> trace_next{0};                   // launches made since the buffer was set
};
inline Tune& tune() {
    static Tune t;
    return t;
}

template <int BN, int EPI, typename OutT>
int launch_one(const TcArgs& g, int splits, int stages, cudaStream_t s, const RopeKv* rope = nullptr) {
    using C = Cfg<BN>;
    CUtensorMap mw, ma;
    if (!cached_map(&mw, g.w, g.N, g.K, TILE_W) || (EPI == EPI_RESIDUAL_A16 ? (ma = mw, false) : !cached_map(&ma, g.a, g.M, g.K, BN)))
        return rvhost::fail_msg(-2, "cuTensorMapEncodeTiled failed (driver entry point missing or bad operand layout)");
    auto kern = fp8_gemm_tc_kernel<BN, EPI, OutT>;
    // Split-K with a small batch tile: push reduction (needs its receive buffer behind the ring);
    // otherwise the partial tile is parked in the ring itself, which must be large enough for it.
    const bool push = splits > 1 && BN <= 32 && tune().reduce != 1;
    // 64- and 128-row batch tiles: push as well, into the peers' idle rings (the partials would not fit behind them)
    const bool push_ring = splits > 1 && (BN == 64 || BN == 128) && tune().reduce != 1 &&
                           (EPI == EPI_SCALE || EPI == EPI_RESIDUAL || EPI == EPI_F32 || EPI == EPI_QKV_ROPE);
    const int ring_recv_bytes = push_ring ? splits * ((BN + splits - 1) / splits) * TILE_W * 4 : 0;
    const int min_stages = (push || push_ring) ? 2 : C::MIN_STAGES;
    if (stages < min_stages) stages = min_stages;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    // dynamic shared memory this instantiation may ask for: the 227 KB per-CTA limit less its static arrays
    // (per-row scales of the 16-bit activation form, per-warp winners of the argmax epilogue)
    constexpr int SMEM_LIMIT = 227 * 1024 - 8 * BN - 256;  // (static shared memory: at most two floats per batch row)
    while (stages > min_stages && C::smem_bytes(stages, push) > SMEM_LIMIT) stages--;
    static RvDeviceOnce smem_once;  // per kernel instantiation and device: allow the largest ring once
    {
        int most = MAX_STAGES;
        const bool may_push = BN <= 32;  // the largest footprint this instantiation can be launched with
        while (most > C::MIN_STAGES && C::smem_bytes(most, may_push) > SMEM_LIMIT) most--;
        if (rv_allow_smem(smem_once, kern, C::smem_bytes(most, may_push)))
            return rvhost::fail_msg(-2, "cannot raise dynamic shared memory for the tcgen05 GEMM");
    }
    TcParams p;
    p.a_scale = g.a_scale;
    p.w_scale = g.w_scale;
    p.out = g.out;
    p.residual = g.residual;
    p.M = g.M;
    p.N = g.N;
    p.K = g.K;
    p.kblocks = (g.K + BK - 1) / BK;
    p.stages = stages;
    // completion of the push: arrivals on the owners' mbarriers (2, the default: measured 1.3 us per layer faster in
    // the decode graph than the cluster-wide barrier) or one cluster barrier (1, tuning value 3)
    // (values: 1 small tiles + cluster barrier, 2 small tiles + mbarriers, 3 ring + mbarriers, 4 ring + cluster barrier)
    p.push = push ? (tune().reduce == 3 ? 1 : 2) : push_ring ? (tune().reduce == 3 ? 4 : 3) : 0;
    p.rope = rope ? *rope : RopeKv{};
    p.a16 = g.a16;
    p.amax_part = g.amax_part;
    p.amax_parts = g.amax_parts;
    p.arg_val = g.arg_val;
    p.arg_idx = g.arg_idx;
    p.softcap = g.softcap;
    p.trace = nullptr;
    if (unsigned long long* tr = tune().trace.load()) {  // every launch its own row, in launch order
        const int slots = tune().trace_slots.load();
        if (slots > 0) p.trace = tr + (size_t)(tune().trace_next.fetch_add(1) % slots) * 16;
    }
    if (EPI == EPI_ARGMAX && (splits != 1 || !g.arg_val || !g.arg_idx))
        return rvhost::fail_msg(-3, "the argmax epilogue needs an unsplit launch and its partial buffers");
    if (EPI == EPI_RESIDUAL_A16 && (!g.a16 || !g.amax_part || g.amax_parts <= 0 || BN > 32))
        return rvhost::fail_msg(-3, "the 16-bit activation form needs a16, partial maxima and a batch tile of at most 32 rows");
    if (EPI == EPI_QKV_ROPE && (!(push || push_ring) || !rope))
        return rvhost::fail_msg(-3, "the fused QKV epilogue needs a split-K launch with a batch tile of at most 128 rows");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((g.N + TILE_W - 1) / TILE_W, splits, (g.M + BN - 1) / BN);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = C::smem_bytes(stages, push);
    if (push_ring && stages * C::STAGE_BYTES < ring_recv_bytes)  // a few columns more than the ring holds (S not a power of two)
        cfg.dynamicSmemBytes += ring_recv_bytes - stages * C::STAGE_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = splits;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (rv_pdl_enabled()) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    if (cudaLaunchKernelEx(&cfg, kern, mw, ma, p) != cudaSuccess) {
        cudaGetLastError();
        return rvhost::fail_msg(-2, "tcgen05 GEMM launch failed");
    }
    return 0;
}

template <int BN>
int launch_epi(const TcArgs& g, int splits, int stages, cudaStream_t s) {
    if (g.out_kind == 2) return launch_one<BN, EPI_F32, __half>(g, splits, stages, s);
    if (g.out_kind == 0)
        return g.residual ? launch_one<BN, EPI_RESIDUAL, __half>(g, splits, stages, s)
                          : launch_one<BN, EPI_SCALE, __half>(g, splits, stages, s);
    return g.residual ? launch_one<BN, EPI_RESIDUAL, __nv_bfloat16>(g, splits, stages, s)
                      : launch_one<BN, EPI_SCALE, __nv_bfloat16>(g, splits, stages, s);
}

// Split-K factor: aim for ~2.5 CTAs per SM (measured best on the decode shapes: 64 weight
// tiles -> 6 splits, 42 tiles -> 8, 336 tiles -> 1), keeping at least four K blocks per CTA.
inline int pick_splits(int M, int N, int K, int bn) {
    const int tiles = ((N + TILE_W - 1) / TILE_W) * ((M + bn - 1) / bn);
    const int kblocks = (K + BK - 1) / BK;
    // 256-row batch tiles (M > 128) are tensor-bound, one CTA per SM: split only while the tiles leave SMs idle
    // (measured at M = 512 on the QKV shape: 117 us split three ways with the pull reduction, against 155 us for
    // four times the work unsplit)
    if (bn >= 256) {
        int s2 = 148 / tiles;
        if (s2 > 8) s2 = 8;
        while (s2 > 1 && kblocks / s2 < 4) s2--;
        return s2 < 1 ? 1 : s2;
    }
    for (int i = 0; i < 4; i++) {
        const long long e = tune().split_for[i].load();
        if (e != 0 && (e >> 40) == N && ((e >> 8) & 0xffffffffll) == K && bn <= 128) return (int)(e & 0xff);
    }
    const int target = tune().split_target.load() > 0 ? tune().split_target.load() : 360;
    int s = (target + tiles / 2) / tiles;
    if (s > 8) s = 8;
    while (s > 1 && kblocks / s < 4) s--;
    if (s < 1) s = 1;
    return s;
}

// Ring depth: a shallow ring lets three CTAs share an SM, so one CTA's prologue / epilogue overlaps
// the others' streaming; measured faster than a deeper ring with fewer CTAs per SM on every decode
// shape (gate|up at M = 32: 93 % vs 58 % of the HBM peak with 3 vs 8 stages; at M = 128: 77 % vs
// 56 % with 2 vs 3 stages).  ~60-66 KB per CTA either way: 3 stages of 20-24 KB up to a 64-row batch
// tile, 2 stages of 32 KB for a 128-row one.
inline int pick_stages(int bn, int splits) {
    // split launches with the push reduction: the ring shares the CTA's ~66 KB with the receive buffer (20 KB for a
    // 32-row batch tile: two stages; 12 KB for a 16-row one: three stages, measured 5 % faster on the batch-1 step)
    if (bn <= 32 && splits > 1) return bn <= 16 ? 3 : 2;
    return bn <= 64 ? 3 : bn == 128 ? 2 : 4;
}

// The launch plan of a shape: batch tile, split-K factor, ring depth.
struct Plan {
    int bn, splits, stages, kblocks;
};
inline Plan plan_for(int M, int N, int K) {
    Plan pl;
    pl.bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    const int t_splits = tune().splits.load(), t_stages = tune().stages.load();
    pl.splits = t_splits > 0 ? t_splits : pick_splits(M, N, K, pl.bn);
    pl.kblocks = (K + BK - 1) / BK;
    if (pl.splits > pl.kblocks) pl.splits = pl.kblocks;
    if (pl.splits > 8) pl.splits = 8;
    pl.stages = t_stages > 0 ? t_stages : pick_stages(pl.bn, pl.splits);
    return pl;
}

inline int launch(const TcArgs& g, void*, size_t, cudaStream_t s) {
    if (g.K % 16 != 0) return rvhost::fail_msg(-3, "tcgen05 GEMM needs K to be a multiple of 16");
    const Plan pl = plan_for(g.M, g.N, g.K);
    const int bn = pl.bn, splits = pl.splits, stages = pl.stages;
    switch (bn) {
        case 16: return launch_epi<16>(g, splits, stages, s);
        case 32: return launch_epi<32>(g, splits, stages, s);
        case 64: return launch_epi<64>(g, splits, stages, s);
        case 128: return launch_epi<128>(g, splits, stages, s);
        default: return launch_epi<256>(g, splits, stages, s);
    }
}

// QKV projection with RoPE, Q quantisation and the paged FP8 KV write in the epilogue.  head_dim is 128
// (one weight tile per head), N = (heads + 2 * kv_heads) * 128, M <= 32.  dtype: 0 f16, 1 bf16 (the type
// the unfused GEMM would have stored, and of the cos / sin tables).  -3: shape not taken, use the two kernels.
inline int launch_qkv_rope(const TcArgs& g, const RopeKv& rk, int dtype, cudaStream_t s) {
    if (g.K % 16 != 0 || g.M > 128 || g.N != (rk.heads + 2 * rk.kv_heads) * TILE_W)
        return rvhost::fail_msg(-3, "fused QKV epilogue: shape not taken");
    const Plan pl = plan_for(g.M, g.N, g.K);
    if (pl.splits < 2 || tune().reduce == 1) return rvhost::fail_msg(-3, "fused QKV epilogue: needs the split-K push form");
    switch (pl.bn) {
        case 16:
            return dtype == 0 ? launch_one<16, EPI_QKV_ROPE, __half>(g, pl.splits, pl.stages, s, &rk)
                              : launch_one<16, EPI_QKV_ROPE, __nv_bfloat16>(g, pl.splits, pl.stages, s, &rk);
        case 32:
            return dtype == 0 ? launch_one<32, EPI_QKV_ROPE, __half>(g, pl.splits, pl.stages, s, &rk)
                              : launch_one<32, EPI_QKV_ROPE, __nv_bfloat16>(g, pl.splits, pl.stages, s, &rk);
        case 64:  // (64- and 128-row tiles: the push goes into the peers' idle rings)
            return dtype == 0 ? launch_one<64, EPI_QKV_ROPE, __half>(g, pl.splits, pl.stages, s, &rk)
                              : launch_one<64, EPI_QKV_ROPE, __nv_bfloat16>(g, pl.splits, pl.stages, s, &rk);
        default:
            return dtype == 0 ? launch_one<128, EPI_QKV_ROPE, __half>(g, pl.splits, pl.stages, s, &rk)
                              : launch_one<128, EPI_QKV_ROPE, __nv_bfloat16>(g, pl.splits, pl.stages, s, &rk);
    }
}

// Residual GEMM whose activation operand is given as 16-bit values plus per-row partial maxima: the per-token
// quantiser is folded into the kernel (its idle epilogue warps build the FP8 A tiles).  M <= 32.
inline int launch_residual_a16(const TcArgs& g, int dtype, cudaStream_t s) {
    if (g.K % 16 != 0 || g.M > 32) return rvhost::fail_msg(-3, "16-bit activation form: shape not taken");
    const Plan pl = plan_for(g.M, g.N, g.K);
    if (pl.bn == 16)
        return dtype == 0 ? launch_one<16, EPI_RESIDUAL_A16, __half>(g, pl.splits, pl.stages, s)
                          : launch_one<16, EPI_RESIDUAL_A16, __nv_bfloat16>(g, pl.splits, pl.stages, s);
    return dtype == 0 ? launch_one<32, EPI_RESIDUAL_A16, __half>(g, pl.splits, pl.stages, s)
                      : launch_one<32, EPI_RESIDUAL_A16, __nv_bfloat16>(g, pl.splits, pl.stages, s);
}

// LM head with the greedy argmax in the epilogue: per-tile winners into arg_val / arg_idx [M][ceil(N / 128)], then the
// merge kernel.  Always an unsplit launch (a vocabulary-sized N has thousands of tiles; the plan would not split it).
inline int launch_argmax(const TcArgs& g, int* out_tokens, cudaStream_t s) {
    if (g.K % 16 != 0) return rvhost::fail_msg(-3, "tcgen05 GEMM needs K to be a multiple of 16");
    Plan pl = plan_for(g.M, g.N, g.K);
    pl.splits = 1;
    pl.stages = tune().stages.load() > 0 ? tune().stages.load() : pick_stages(pl.bn, 1);
    int rc;
    switch (pl.bn) {
        case 16: rc = launch_one<16, EPI_ARGMAX, __half>(g, 1, pl.stages, s); break;
        case 32: rc = launch_one<32, EPI_ARGMAX, __half>(g, 1, pl.stages, s); break;
        case 64: rc = launch_one<64, EPI_ARGMAX, __half>(g, 1, pl.stages, s); break;
        case 128: rc = launch_one<128, EPI_ARGMAX, __half>(g, 1, pl.stages, s); break;
        default: rc = launch_one<256, EPI_ARGMAX, __half>(g, 1, pl.stages, s); break;
    }
    if (rc) return rc;
    const int tiles = (g.N + TILE_W - 1) / TILE_W;
    if (rv_launch(argmax_merge_kernel, dim3(g.M), dim3(256), 0, s, dim3(1, 1, 1), (const float*)g.arg_val, (const int*)g.arg_idx,
                  tiles, out_tokens) != cudaSuccess) {
        cudaGetLastError();
        return rvhost::fail_msg(-2, "argmax merge launch failed");
    }
    return 0;
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

}  // namespace rvtc
