// One launch for everything between two attention calls of a decoder layer at decode batch sizes (M <= 32):
//
//   O projection (+residual)  ->  RMSNorm + FP8 quant  ->  gate|up projection  ->  act(gate)*up + FP8 quant
//   ->  down projection (+residual)  ->  RMSNorm + FP8 quant (the next layer's input)
//
// i.e. v3/crates/rvllm-runtime/src/layer_exec.rs:425-541 of the reference (quantize_fp8_per_token, O GEMM with
// residual, fused_rmsnorm_fp8_quant, gate|up GEMM, fused_silu_mul_fp8_quant, down GEMM with residual) plus the
// fused_rmsnorm_fp8_quant that opens the next layer (:205-222).  Every stage computes exactly what the
// stand-alone kernels of this library compute (same tiles, same split-K order, same reduction trees), so the
// bytes are those of the six-launch chain; what changes is that the weight stream never stops: a dependent
// chain of short kernels leaves HBM idle for a few microseconds at every boundary (tail of one kernel,
// completion, dependency release, activation fetch of the next), which at batch 32 costs a third of the
// step.  Here the CTAs stay resident, meet at grid-wide barriers, and each CTA's TMA producer keeps
// fetching the next stage's weight tiles (they depend on nothing) while the barrier is in flight.
//
// Geometry: hidden = 128 * T.  Grid (T, 8): G = 8 T CTAs, all resident at once (three per SM; the host checks
// the occupancy before it launches; no clusters, so nothing constrains where a CTA lands).  CTA (c, s), linear
// id j = 8 c + s:
//   O, down   : weight tile c (128 output channels), K slice s of 8; the f32 partial tile goes to a small
//               workspace in L2 (8 x 32 x hidden floats), the row's owner sums the eight slices in slice order.
//   gate|up   : unit j = 64 gate rows + the 64 up rows of the same columns as ONE 128-row tcgen05 operand
//               (two 64-row TMA boxes), whole K; gate and up of a column then sit in the same CTA, so
//               act(gate)*up needs no exchange.  ffn / 64 <= G units; CTAs beyond that idle in this stage.
//   rows      : CTA j < M owns batch row j: it finishes the split-K sum of the row (+ residual), and runs the
//               RMSNorm + quantisation on the values it just produced.
// Warp roles as in the stand-alone GEMM: warp 0 lane 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2-5 = A-tile builder (O stage) / epilogue / row kernels / grid barrier.
//
// Every wait is bounded: when one runs out the kernel records where in rvtc::g_status and carries on to its
// exit (results are then wrong, nothing hangs).  No multicast, no cross-GPU access.
#pragma once
#include "fp8_gemm_tc.cuh"
#include "rowq_act.cuh"

namespace rvblk {

using namespace rvtc;

constexpr int BN = 32;            // batch rows per tile (M <= 32)
constexpr int CL = 8;             // K slices of the O / down stages (gridDim.y)
constexpr int STAGES = 2;         // TMA ring depth: three CTAs of ~60 KB share an SM
constexpr int STAGE_BYTES = TILE_W * BK + BN * BK;   // 16 KB weights + 4 KB activations
constexpr int SCRATCH_BYTES = TILE_W * (BN + 1) * 4; // gate|up exchange tile [128][33] f32; also a row + its partial sums
constexpr int MAX_HIDDEN = 6144;  // a row (2 B / value) + 1024 partial sums must fit the scratch area
constexpr int BLK_HEADER = 2048;  // barriers, TMEM address, per-row scales and small reduction arrays, in front of the ring
constexpr int SMEM_BYTES = 1024 + BLK_HEADER + STAGES * STAGE_BYTES + SCRATCH_BYTES;
constexpr int EPI_THREADS = 128;

constexpr int PH_O = 1, PH_N1 = 2, PH_GU = 4, PH_D = 8, PH_N2 = 16;

struct BlkParams {
    int M, H, F, KO;          // batch rows, hidden, ffn, K of the O projection
    int phases;               // PH_* mask (all five in production; subsets let the tests check one stage at a time)
    int act;                  // 0 SiLU, 1 GELU-tanh
    float eps;
    // O projection, activations in one of two forms: 16-bit attention output + per-row partial maxima (the
    // per-token quantiser is folded in: attn16 != null), or FP8 rows + per-row scales (attn16 == null, map_ao)
    const void* attn16;
    const float* attn_amax;
    int amax_parts;
    const float* attn_scale;
    const float* o_wscale;
    void* residual;           // [M, H] 16-bit, updated in place by the O and the down stage
    const void* gamma1;       // RMSNorm gain before gate|up
    const void* gamma2;       // RMSNorm gain of the next layer's attention block
    uint8_t* x8;              // [M, H] FP8: RMSNorm output (input of gate|up; rewritten by the closing norm)
    float* xs;                // [M]
    const float* gu_wscale;   // [2 F]
    uint8_t* h8;              // [M, F] FP8: act(gate)*up
    float* hs;                // [M]
    const float* d_wscale;
    unsigned int* bar;        // [0] arrivals, [32] departures (separate 128-byte lines); zero between launches
    float* amax_ws;           // [F / 64][BN] partial row maxima of act(gate)*up
    float* part;              // [CL][BN][H] f32 split-K partial tiles of the O / down stage
    unsigned long long* trace;  // null, or [G][16] %globaltimer stamps of the stage boundaries (tuning runs)
};

// ---- small helpers -------------------------------------------------------------------------------------
// Barrier of the four epilogue warps (named barrier 1).  The warp is made convergent first: the barrier
// instruction is warp-aligned, and callers reach it right after single-thread sections.
__device__ __forceinline__ void epi_sync() {
    __syncwarp();
    asm volatile("bar.sync 1, 128;" ::: "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long v;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
    return v;
}
__device__ __forceinline__ float ldcg_f32(const float* p) { return __ldcg(p); }
// 16-bit value read through L2 (it may have been written by another SM earlier in this launch)
template <typename T> __device__ __forceinline__ float ld16_cg(const T* p) {
    const unsigned short b = __ldcg(reinterpret_cast<const unsigned short*>(p));
    return rv::T16<T>::to_f32(*reinterpret_cast<const T*>(&b));
}

// Grid-wide barrier of the epilogue warps (128 threads per CTA).  `target` = G * (number of barriers passed so
// far in this launch + 1): the arrival counter only grows during a launch and the last CTA to leave the kernel
// puts it back to zero.  Pattern of a cooperative-groups grid sync: block barrier, one thread releases /
// spins / acquires, block barrier.
__device__ __forceinline__ void grid_barrier(unsigned int* arrive, unsigned int target, int t, int site) {
    epi_sync();
    if (t == 0) {
        __threadfence();
        red_release_gpu_add(arrive, 1u);
        bool ok = false;
        for (uint32_t i = 0; i < (1u << 20); i++) {
            if (ld_acquire_gpu(arrive) >= target) {
                ok = true;
                break;
            }
            __nanosleep(32);
        }
        if (!ok) atomicCAS(&g_status, 0, (site << 16) | (int)((blockIdx.x * gridDim.y + blockIdx.y) & 0xffff));
        __threadfence();
    }
    epi_sync();
}

// RMSNorm + per-token FP8 quantisation of row `row` by the 128 epilogue threads, with the arithmetic of
// fused_rmsnorm_fp8_quant_kernel launched with NV = min(hidden, 1024) threads (kernels/fused_rmsnorm_fp8_quant.cu:
// 52-103): virtual thread v sums x[v], x[v + NV], ... in that order, the 32 lanes of a virtual warp reduce with
// the xor butterfly, the warp totals with the same butterfly; rsqrtf; (x * rms) * gamma; absmax / 448 floored at
// 1e-12; x * (1 / scale).  Bytes and scale equal that kernel's.  scratch: [H] 16-bit row, then NV floats.
template <typename T>
__device__ __forceinline__ void norm_quant_row(const BlkParams& p, const void* gamma_v, int row, int t, uint8_t* scratch,
                                               float* s_small, bool row_staged) {
    const int H = p.H;
    T* srow = reinterpret_cast<T*>(scratch);
    float* partial = reinterpret_cast<float*>(scratch + (((size_t)H * 2 + 15) & ~(size_t)15));
    const T* x = reinterpret_cast<const T*>(p.residual) + (size_t)row * H;
    const T* gamma = reinterpret_cast<const T*>(gamma_v);
    int NV = H < 1024 ? H : 1024;
    NV -= NV % 32;
    const int nvec = H >> 3;
    if (!row_staged) {  // (else the caller has just produced the row into `scratch`)
        for (int v = t; v < nvec; v += EPI_THREADS)
            reinterpret_cast<uint4*>(srow)[v] = __ldcg(reinterpret_cast<const uint4*>(x) + v);
        epi_sync();
    }
    for (int v = t; v < NV; v += EPI_THREADS) {
        float ss = 0.0f;
        for (int i = v; i < H; i += NV) {
            const float a = rv::T16<T>::to_f32(srow[i]);
            ss += a * a;
        }
        partial[v] = ss;
    }
    epi_sync();
    const int w4 = t >> 5, lane = t & 31, nw = NV >> 5;
    for (int vw = w4; vw < nw; vw += 4) {
        const float s = rv::warp_sum(partial[vw * 32 + lane]);
        if (lane == 0) s_small[vw] = s;
    }
    epi_sync();
    if (w4 == 0) {
        const float s = rv::warp_sum(lane < nw ? s_small[lane] : 0.0f);
        if (lane == 0) s_small[32] = s;
    }
    epi_sync();
    const float rms = rsqrtf(s_small[32] / (float)H + p.eps);
    epi_sync();  // s_small is reused below
    float amax = 0.0f;
    for (int v = t; v < nvec; v += EPI_THREADS) {
        const uint4 xv = reinterpret_cast<const uint4*>(srow)[v];
        const uint4 gv = rv::ldg128(reinterpret_cast<const uint4*>(gamma) + v);
        const uint32_t* xp = &xv.x;
        const uint32_t* gp = &gv.x;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 a = rv::T16<T>::to_f32x2(xp[j]), g = rv::T16<T>::to_f32x2(gp[j]);
            amax = fmaxf(amax, fmaxf(fabsf(a.x * rms * g.x), fabsf(a.y * rms * g.y)));
        }
    }
    amax = rv::warp_max(amax);
    if (lane == 0) s_small[w4] = amax;
    epi_sync();
    amax = fmaxf(fmaxf(s_small[0], s_small[1]), fmaxf(s_small[2], s_small[3]));
    const float scale = rv::row_scale(amax);
    if (t == 0) p.xs[row] = scale;
    const float inv = 1.0f / scale;
    uint8_t* out = p.x8 + (size_t)row * H;
    for (int v = t; v < nvec; v += EPI_THREADS) {
        const uint4 xv = reinterpret_cast<const uint4*>(srow)[v];
        const uint4 gv = rv::ldg128(reinterpret_cast<const uint4*>(gamma) + v);
        const uint32_t* xp = &xv.x;
        const uint32_t* gp = &gv.x;
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 a = rv::T16<T>::to_f32x2(xp[j]), g = rv::T16<T>::to_f32x2(gp[j]);
            f[2 * j] = a.x * rms * g.x * inv;
            f[2 * j + 1] = a.y * rms * g.y * inv;
        }
        uint2 o;
        o.x = rv::f32x4_to_e4m3x4(f[0], f[1], f[2], f[3]);
        o.y = rv::f32x4_to_e4m3x4(f[4], f[5], f[6], f[7]);
        reinterpret_cast<uint2*>(out)[v] = o;
    }
    epi_sync();  // scratch and s_small are free again
}

template <typename OutT>
__global__ void __launch_bounds__(THREADS, 3)
fp8_layer_block_kernel(const __grid_constant__ CUtensorMap map_wo, const __grid_constant__ CUtensorMap map_wgu,
                       const __grid_constant__ CUtensorMap map_wd, const __grid_constant__ CUtensorMap map_ao,
                       const __grid_constant__ CUtensorMap map_x8, const __grid_constant__ CUtensorMap map_h8,
                       BlkParams p) {
    extern __shared__ uint8_t raw[];
    uint8_t* header = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = header + BLK_HEADER;
    uint8_t* scratch = ring + STAGES * STAGE_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(header);        // [STAGES] TMA bytes of a stage have landed
    uint64_t* afull = full + STAGES;                             // [STAGES] O stage: the converted A tile is in place
    uint64_t* empty = afull + STAGES;                            // [STAGES] the MMAs have read the stage
    uint64_t* acc_ready = empty + STAGES;                        // the stage's accumulator is complete
    uint64_t* acc_free = acc_ready + 1;                          // the epilogue has read the accumulator
    uint64_t* gate = acc_free + 1;                               // the activations of the next GEMM stage exist
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(gate + 1);
    float* s_ascale = reinterpret_cast<float*>(header + 256);    // [BN] activation scale of the current GEMM stage
    float* s_ainv = s_ascale + BN;                               // [BN]
    float* s_small = s_ainv + BN;                                // [40] reductions of the row kernels
    float* s_part = s_small + 40;                                // [4][BN] per-warp row maxima of act(gate)*up

    const int tile = blockIdx.x, split = blockIdx.y;
    const int G = gridDim.x * gridDim.y;
    const int j = tile * CL + split;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int units = p.F / 64;
    const bool do_o = p.phases & PH_O, do_gu = (p.phases & PH_GU) && j < units, do_d = p.phases & PH_D;
    const int kbO = (p.KO + BK - 1) / BK, kbG = (p.H + BK - 1) / BK, kbD = (p.F + BK - 1) / BK;
    // K ranges (in 128-byte blocks) of this CTA in the three GEMM stages
    const int o_lo = do_o ? (int)((long long)split * kbO / CL) : 0, o_hi = do_o ? (int)((long long)(split + 1) * kbO / CL) : 0;
    const int d_lo = do_d ? (int)((long long)split * kbD / CL) : 0, d_hi = do_d ? (int)((long long)(split + 1) * kbD / CL) : 0;
    const int nO = o_hi - o_lo, nG = do_gu ? kbG : 0, nD = d_hi - d_lo;
    const bool o_a16 = p.attn16 != nullptr;  // O stage: A tiles built from 16-bit activations (else TMA from FP8 rows)

    rv::pdl_launch();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full + s, 1);
            mbar_init(afull + s, 4);
            mbar_init(empty + s, 1);
        }
        mbar_init(acc_ready, 1);
        mbar_init(acc_free, 4);
        mbar_init(gate, 1);
        fence_barrier_init();
        // This thread is also the TMA producer.  Weights depend on nothing: the first O-stage tiles are on their
        // way before the block, the cluster or the predecessor kernel are waited for.
        const int pre = nO < STAGES ? nO : STAGES;
        for (int i = 0; i < pre; i++) {
            mbar_expect_tx(full + i, o_a16 ? TILE_W * BK : STAGE_BYTES);
            tma_load_2d(ring + (size_t)i * STAGE_BYTES, &map_wo, (o_lo + i) * BK, tile * TILE_W, full + i);
        }
    }
    if (warp == 1) tmem_alloc(tmem_holder, 32);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        // ================================================================ TMA producer
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            uint32_t gate_uses = 0;
            auto slot_free = [&](int i) -> bool {  // the ring slot of iteration i was read by the MMAs of iteration i - STAGES
                if (i < STAGES) return true;
                return mbar_wait(empty + i % STAGES, ((uint32_t)(i / STAGES) & 1u) ^ 1u, 1);
            };
            // Three GEMM stages, one loop.  Weights run ahead by the ring depth; the activations of a stage are
            // fetched once they exist: after the predecessor kernel (O stage, FP8 form; in the 16-bit form the
            // epilogue warps build the A tiles), after the grid barrier that follows their producer (gate|up, down).
            for (int stage = 0; stage < 3 && alive; stage++) {
                const int n = stage == 0 ? nO : stage == 1 ? nG : nD;
                const int k0 = stage == 0 ? o_lo : stage == 1 ? 0 : d_lo;
                const CUtensorMap* mw = stage == 0 ? &map_wo : stage == 1 ? &map_wgu : &map_wd;
                const CUtensorMap* ma = stage == 0 ? &map_ao : stage == 1 ? &map_x8 : &map_h8;
                const bool a_tma = !(stage == 0 && o_a16);
                const uint32_t tx = a_tma ? STAGE_BYTES : TILE_W * BK;
                auto load_w = [&](int i, int slot) {
                    uint8_t* dst = ring + (size_t)slot * STAGE_BYTES;
                    if (stage == 1) {  // 64 gate rows and the 64 up rows of the same columns: one 128-row operand
                        tma_load_2d(dst, mw, (k0 + i) * BK, j * 64, full + slot);
                        tma_load_2d(dst + 64 * BK, mw, (k0 + i) * BK, p.F + j * 64, full + slot);
                    } else {
                        tma_load_2d(dst, mw, (k0 + i) * BK, tile * TILE_W, full + slot);
                    }
                };
                auto load_a = [&](int i, int slot) {
                    tma_load_2d(ring + (size_t)slot * STAGE_BYTES + TILE_W * BK, ma, (k0 + i) * BK, 0, full + slot);
                };
                const int pre = n < STAGES ? n : STAGES;
                if (stage > 0) {  // (the O stage's first weight tiles were issued before the block met)
                    for (int i = 0; i < pre && alive; i++) {
                        alive = slot_free(it + i);
                        if (!alive) break;
                        mbar_expect_tx(full + (it + i) % STAGES, tx);
                        load_w(i, (it + i) % STAGES);
                    }
                }
                if (stage == 0) {
                    if (a_tma) rv::pdl_wait();  // the FP8 activations come from the predecessor kernel
                } else {
                    // written through the generic proxy by other CTAs before the grid barrier the epilogue warps passed
                    if (alive) alive = mbar_wait(gate, gate_uses & 1u, 6);
                    gate_uses++;
                    fence_proxy_async_all();
                }
                if (a_tma)
                    for (int i = 0; i < pre && alive; i++) load_a(i, (it + i) % STAGES);
                for (int i = pre; i < n && alive; i++) {
                    alive = slot_free(it + i);
                    if (!alive) break;
                    const int slot = (it + i) % STAGES;
                    mbar_expect_tx(full + slot, tx);
                    load_w(i, slot);
                    if (a_tma) load_a(i, slot);
                }
                it += n;
            }
        }
    } else if (warp == 1) {
        // ================================================================ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN);
            int it = 0;
            uint32_t uses = 0;
            bool alive = true;
            for (int stage = 0; stage < 3 && alive; stage++) {
                const int n = stage == 0 ? nO : stage == 1 ? nG : nD;
                if (n == 0) continue;
                if (uses > 0) {  // the previous accumulator must have been read out of TMEM
                    alive = mbar_wait(acc_free, (uses - 1) & 1u, 7);
                    if (!alive) break;
                    tc_fence_after();
                }
                for (int i = 0; i < n && alive; i++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                    alive = mbar_wait(full + s, ph, 2);
                    if (alive && stage == 0 && o_a16) alive = mbar_wait(afull + s, ph, 8);
                    if (!alive) break;
                    tc_fence_after();
                    const uint32_t w_addr = smem_u32(ring + (size_t)s * STAGE_BYTES);
                    const uint64_t adesc = smem_desc_sw128(w_addr);
                    const uint64_t bdesc = smem_desc_sw128(w_addr + TILE_W * BK);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        umma_f8(tmem_base, adesc + (uint64_t)(k * UMMA_K >> 4), bdesc + (uint64_t)(k * UMMA_K >> 4), idesc,
                                (i > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty + s);
                }
                umma_commit(acc_ready);
                uses++;
            }
        }
    } else {
        // ================================================================ A-tile builder, epilogues, row kernels
        const int t = (int)threadIdx.x - EPI_WARP0 * 32;   // 0..127
        const int w4 = t >> 5;
        const int quarter = warp & 3;                      // TMEM lanes this warp may read: 32 * quarter ...
        const int r = quarter * 32 + lane;                 // row of the weight tile held by this thread
        unsigned int* bar_arrive = p.bar;
        unsigned int* bar_depart = p.bar + 32;
        uint32_t acc_uses = 0, barriers = 0;
        int it = 0;
        bool alive = true;
        auto stamp = [&](int k) {
            if (p.trace && t == 0) p.trace[(size_t)j * 16 + k] = global_timer();
        };
        stamp(0);

        // Epilogue of a split-K stage (O, down): this CTA's f32 partial tile [BN rows][128 channels] goes to the
        // workspace, slice-major, so that a warp stores 128 contiguous bytes per batch row.
        auto store_partial = [&](int n_kb, int stamp_id) {
            bool ready = true;
            if (n_kb > 0) ready = mbar_wait(acc_ready, acc_uses & 1u, 3);
            stamp(stamp_id);
            tc_fence_after();
            float* dst = p.part + ((size_t)split * BN) * p.H + (size_t)tile * TILE_W + r;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t v[16];
                if (n_kb > 0 && ready) {
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int q = 0; q < 16; q++) v[q] = 0u;
                }
#pragma unroll
                for (int q = 0; q < 16; q++)
                    if (c0 + q < p.M) __stcg(dst + (size_t)(c0 + q) * p.H, __uint_as_float(v[q]));
            }
            tc_fence_before();
            if (n_kb > 0) {
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_free);
                acc_uses++;
            }
        };

        // Row owner (CTA j < M, row j), after the grid barrier that follows a split-K stage: sum the eight slices in
        // slice order, scale, add the residual, store the new residual row — out = a_scale * (w_scale * sum) +
        // residual, the stand-alone GEMM's expression and summation order.  The row is left in `scratch` (16-bit) for
        // the RMSNorm that follows.
        auto finish_row = [&](int row, float a_scale, const float* w_scale) {
            OutT* srow = reinterpret_cast<OutT*>(scratch);
            OutT* res = reinterpret_cast<OutT*>(p.residual) + (size_t)row * p.H;
            const float* part = p.part + (size_t)row * p.H;
            const int nvec = p.H >> 2;
            for (int v = t; v < nvec; v += EPI_THREADS) {
                float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);  // (0 + first slice: the stand-alone kernel's order, signed zeros included)
#pragma unroll
                for (int sp = 0; sp < CL; sp++) {
                    const float4 x = __ldcg(reinterpret_cast<const float4*>(part + (size_t)sp * BN * p.H) + v);
                    sum.x += x.x;
                    sum.y += x.y;
                    sum.z += x.z;
                    sum.w += x.w;
                }
                const float4 ws = *reinterpret_cast<const float4*>(w_scale + 4 * v);
                const uint2 rb = __ldcg(reinterpret_cast<const uint2*>(res) + v);
                const float2 r01 = rv::T16<OutT>::to_f32x2(rb.x), r23 = rv::T16<OutT>::to_f32x2(rb.y);
                uint2 o;
                o.x = rv::pack2_sat<OutT>(fmaf(a_scale, ws.x * sum.x, r01.x), fmaf(a_scale, ws.y * sum.y, r01.y));
                o.y = rv::pack2_sat<OutT>(fmaf(a_scale, ws.z * sum.z, r23.x), fmaf(a_scale, ws.w * sum.w, r23.y));
                reinterpret_cast<uint2*>(res)[v] = o;
                reinterpret_cast<uint2*>(srow)[v] = o;
            }
            epi_sync();
        };

        rv::pdl_wait();  // everything below reads what earlier kernels wrote
        stamp(1);

        // ---------------------------------------------------------------- O projection
        if (do_o && !o_a16) {
            store_partial(nO, 2);
        } else if (do_o) {
            if (t < BN) {  // per-row activation scale from the partial maxima the attention kernel left
                float amax = 0.0f;
                if (t < p.M)
                    for (int q = 0; q < p.amax_parts; q++) amax = fmaxf(amax, p.attn_amax[(size_t)t * p.amax_parts + q]);
                const float sc = rv::row_scale(amax);
                s_ascale[t] = sc;
                s_ainv[t] = 1.0f / sc;
            }
            epi_sync();
            // build the FP8 A tiles of this CTA's K blocks (the per-token quantiser's arithmetic), one block ahead
            const OutT* a16 = reinterpret_cast<const OutT*>(p.attn16);
            const int rr = t >> 3, cc = t & 7;  // row and 16-column group of this thread's 16-byte chunk (BN * 8 = 256 chunks: two per thread)
            uint4 nx[2][2];
            auto fetch = [&](int i) {
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const int m = rr + q * 16, k0 = (o_lo + i) * BK + cc * 16;
                    nx[q][0] = nx[q][1] = make_uint4(0, 0, 0, 0);
                    if (i < nO && m < p.M && k0 < p.KO) {
                        const uint4* src = reinterpret_cast<const uint4*>(a16 + (size_t)m * p.KO + k0);
                        nx[q][0] = rv::ldg128(src);
                        nx[q][1] = rv::ldg128(src + 1);
                    }
                }
            };
            fetch(0);
            for (int i = 0; i < nO && alive; i++, it++) {
                uint4 cur[2][2];
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    cur[q][0] = nx[q][0];
                    cur[q][1] = nx[q][1];
                }
                fetch(i + 1);
                const int s = it % STAGES;
                if (it >= STAGES) alive = mbar_wait(empty + s, ((uint32_t)(it / STAGES) & 1u) ^ 1u, 5);
                if (!alive) break;
                uint8_t* a_tile = ring + (size_t)s * STAGE_BYTES + TILE_W * BK;
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const int m = rr + q * 16;
                    const float inv = s_ainv[m];
                    const uint32_t xs[8] = {cur[q][0].x, cur[q][0].y, cur[q][0].z, cur[q][0].w,
                                            cur[q][1].x, cur[q][1].y, cur[q][1].z, cur[q][1].w};
                    uint32_t w4v[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float2 a = rv::T16<OutT>::to_f32x2(xs[2 * e]), b = rv::T16<OutT>::to_f32x2(xs[2 * e + 1]);
                        w4v[e] = rv::f32x4_to_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
                    }
                    *reinterpret_cast<uint4*>(a_tile + m * BK + ((cc ^ (m & 7)) << 4)) = make_uint4(w4v[0], w4v[1], w4v[2], w4v[3]);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(afull + s);
            }
            store_partial(nO, 2);
        }
        stamp(3);
        barriers++;
        grid_barrier(bar_arrive, (unsigned int)G * barriers, t, 10);
        stamp(4);

        // ---------------------------------------------------------------- rows: finish O, RMSNorm + quant (input of gate|up)
        if (j < p.M) {
            if (do_o) {
                float a_scale;
                if (o_a16) {  // the per-token quantiser's scale from the partial maxima the attention kernel left
                    float amax = 0.0f;
                    for (int q = 0; q < p.amax_parts; q++) amax = fmaxf(amax, p.attn_amax[(size_t)j * p.amax_parts + q]);
                    a_scale = rv::row_scale(amax);
                } else {
                    a_scale = p.attn_scale[j];
                }
                finish_row(j, a_scale, p.o_wscale);
            }
            if (p.phases & PH_N1) norm_quant_row<OutT>(p, p.gamma1, j, t, scratch, s_small, /*row_staged=*/do_o);
        }
        stamp(5);
        barriers++;
        grid_barrier(bar_arrive, (unsigned int)G * barriers, t, 11);
        stamp(6);
        if (t == 0) mbar_arrive(gate);  // x8 / xs exist: the producer may fetch the gate|up activations
        it += nG;                       // (the ring iterations of the gate|up stage belong to the producer and the MMA warp)

        // ---------------------------------------------------------------- gate|up + act(gate)*up + quant
        float y[16];
#pragma unroll
        for (int q = 0; q < 16; q++) y[q] = 0.0f;
        if (do_gu) {
            // activation scales of the rows (written by the row kernels above)
            if (t < BN) s_ascale[t] = t < p.M ? __ldcg(p.xs + t) : 0.0f;
            epi_sync();
            bool ready = mbar_wait(acc_ready, acc_uses & 1u, 3);
            stamp(7);
            tc_fence_after();
            // TMEM lane r = row r of the operand: rows 0..63 gate channels 64 j + r, rows 64..127 up channels of the same columns
            const int wrow = r < 64 ? j * 64 + r : p.F + j * 64 + (r - 64);
            const float ws = p.gu_wscale[wrow];
            float* tileT = reinterpret_cast<float*>(scratch);  // [128][BN + 1]: the projections as the 16-bit GEMM would have stored them
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t v[16];
                if (ready) {
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int q = 0; q < 16; q++) v[q] = 0u;
                }
#pragma unroll
                for (int q = 0; q < 16; q++) {
                    const float val = s_ascale[c0 + q] * (ws * __uint_as_float(v[q]));
                    tileT[r * (BN + 1) + c0 + q] = rv::T16<OutT>::to_f32(rv::T16<OutT>::from_f32_sat(val));
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_free);
            acc_uses++;
            epi_sync();
            // thread (w4, lane): batch row m = lane, columns 16 w4 .. 16 w4 + 15 of the unit
            bool nonfinite = false;
            float amax = 0.0f;
#pragma unroll
            for (int q = 0; q < 16; q++) {
                const int c = w4 * 16 + q;
                const float g = tileT[c * (BN + 1) + lane], u = tileT[(64 + c) * (BN + 1) + lane];
                y[q] = (p.act == 0 ? rvact::act<rvact::ACT_SILU>(g) : rvact::act<rvact::ACT_GELU>(g)) * u;
                nonfinite |= !isfinite(y[q]);
                amax = fmaxf(amax, fabsf(y[q]));
            }
            s_part[w4 * BN + lane] = nonfinite ? CUDART_INF_F : amax;  // +inf carries "a product was not finite"
            epi_sync();
            if (w4 == 0)
                p.amax_ws[(size_t)j * BN + lane] = fmaxf(fmaxf(s_part[lane], s_part[BN + lane]),
                                                         fmaxf(s_part[2 * BN + lane], s_part[3 * BN + lane]));
        }
        stamp(8);
        barriers++;
        grid_barrier(bar_arrive, (unsigned int)G * barriers, t, 12);
        stamp(9);
        if (p.phases & PH_GU) {
            // row maxima over all units: thread (w4, lane) takes units w4, w4 + 4, ... of row `lane`
            float am = 0.0f;
            for (int u = w4; u < units; u += 4) am = fmaxf(am, ldcg_f32(p.amax_ws + (size_t)u * BN + lane));
            epi_sync();  // (s_part of the partial pass has been read)
            s_part[w4 * BN + lane] = am;
            epi_sync();
            am = fmaxf(fmaxf(s_part[lane], s_part[BN + lane]), fmaxf(s_part[2 * BN + lane], s_part[3 * BN + lane]));
            const float scale = isinf(am) ? CUDART_NAN_F : rv::row_scale(am);
            if (j == 0 && w4 == 0 && lane < p.M) p.hs[lane] = scale;
            if (do_gu && lane < p.M) {
                const float inv = 1.0f / scale;
                uint4 o;
                o.x = rv::f32x4_to_e4m3x4(y[0] * inv, y[1] * inv, y[2] * inv, y[3] * inv);
                o.y = rv::f32x4_to_e4m3x4(y[4] * inv, y[5] * inv, y[6] * inv, y[7] * inv);
                o.z = rv::f32x4_to_e4m3x4(y[8] * inv, y[9] * inv, y[10] * inv, y[11] * inv);
                o.w = rv::f32x4_to_e4m3x4(y[12] * inv, y[13] * inv, y[14] * inv, y[15] * inv);
                *reinterpret_cast<uint4*>(p.h8 + (size_t)lane * p.F + (size_t)j * 64 + w4 * 16) = o;
            }
        }
        stamp(10);
        barriers++;
        grid_barrier(bar_arrive, (unsigned int)G * barriers, t, 13);
        stamp(11);
        if (t == 0) mbar_arrive(gate);  // h8 / hs exist
        it += nD;

        // ---------------------------------------------------------------- down projection
        if (do_d) store_partial(nD, 12);
        stamp(13);
        barriers++;
        grid_barrier(bar_arrive, (unsigned int)G * barriers, t, 14);
        stamp(14);

        // ---------------------------------------------------------------- rows: finish down, RMSNorm + quant for the next layer
        if (j < p.M) {
            if (do_d) finish_row(j, __ldcg(p.hs + j), p.d_wscale);
            if ((p.phases & PH_N2) && p.gamma2) norm_quant_row<OutT>(p, p.gamma2, j, t, scratch, s_small, /*row_staged=*/do_d);
        }

        // leave: the last CTA out puts the barrier words back to zero for the next launch
        stamp(15);
        epi_sync();
        if (t == 0) {
            __threadfence();
            const unsigned int old = atomicAdd(bar_depart, 1u);
            if (old == (unsigned int)G - 1u) {
                *bar_arrive = 0u;
                *bar_depart = 0u;
                __threadfence();
            }
        }
    }
    __syncwarp();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 32);
    }
}

// ---- host side -------------------------------------------------------------------------------------------
// Tuning runs: a device buffer of G x 16 u64 that the next launches stamp with %globaltimer at their stage
// boundaries (null = off, the default).
inline std::atomic<unsigned long long*>& trace_buffer() {
    static std::atomic<unsigned long long*> p{nullptr};
    return p;
}

struct BlkArgs {
    int M, H, F, KO, act, dtype, phases;
    float eps;
    const void* attn16;      // 16-bit form (with attn_amax / amax_parts), or
    const float* attn_amax;
    int amax_parts;
    const void* attn_fp8;    // FP8 form (with attn_scale)
    const float* attn_scale;
    const void* o_w;
    const float* o_wscale;
    void* residual;
    const void* gamma1;
    const void* gamma2;
    void* x8;
    float* xs;
    const void* gu_w;
    const float* gu_wscale;
    void* h8;
    float* hs;
    const void* d_w;
    const float* d_wscale;
    void* workspace;
    size_t workspace_bytes;
};

// workspace: 256 bytes of barrier words (zero before the first launch; every launch leaves them zero), the
// [ffn / 64][32] partial row maxima, the [8][32][hidden] f32 split-K partial tiles
inline size_t blk_amax_bytes(int F) { return ((size_t)(F / 64) * BN * sizeof(float) + 255) & ~(size_t)255; }
inline size_t blk_workspace_bytes(int F, int H) { return 256 + blk_amax_bytes(F) + (size_t)CL * BN * H * sizeof(float); }

// Whether the shape is taken: M <= 32, hidden a multiple of 128 up to 6144, ffn a multiple of 64 with at most
// one gate|up unit per CTA (ffn <= 4 * hidden), K of the O projection a multiple of 16.
inline bool blk_shape_ok(int M, int H, int F, int KO) {
    return M >= 1 && M <= BN && H >= TILE_W && H % TILE_W == 0 && H <= MAX_HIDDEN && F >= 64 && F % 64 == 0 &&
           F / 64 <= (H / TILE_W) * CL && KO >= 16 && KO % 16 == 0 && H % 16 == 0;
}

template <typename OutT> int launch_block_t(const BlkArgs& g, cudaStream_t s) {
    auto kern = fp8_layer_block_kernel<OutT>;
    static RvDeviceOnce smem_once;
    if (rv_allow_smem(smem_once, kern, SMEM_BYTES)) return rvhost::fail_msg(-2, "cannot raise dynamic shared memory for the layer-block kernel");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(g.H / TILE_W, CL, 1);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = s;
    // The grid-wide barriers need every CTA resident at once: refuse grids larger than the device holds.
    {
        static std::mutex mu;
        static std::unordered_map<int, int> capacity;  // device -> CTAs of this kernel resident at once
        const int dev = rv_current_device();
        std::lock_guard<std::mutex> lock(mu);
        auto it = capacity.find(dev);
        int cap = 0;
        if (it == capacity.end()) {
            int per_sm = 0, sms = 0;
            if (block_capacity_of(kern, &per_sm, &sms) != 0) per_sm = sms = 0;
            cap = per_sm * sms;
            capacity.emplace(dev, cap);
        } else {
            cap = it->second;
        }
        if (cap < (int)(cfg.gridDim.x * cfg.gridDim.y))
            return rvhost::fail_msg(-3, "layer block: the grid would not be resident at once on this device");
    }
    cudaLaunchAttribute attr[1];
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (rv_pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 1;
    }
    CUtensorMap mwo, mwgu, mwd, mao, mx8, mh8;
    if (g.attn16) mao = CUtensorMap{};  // unused in the 16-bit form
    else if (!cached_map(&mao, g.attn_fp8, g.M, g.KO, BN))
        return rvhost::fail_msg(-2, "cuTensorMapEncodeTiled failed for the O-projection activations");
    if (!cached_map(&mwo, g.o_w, g.H, g.KO, TILE_W) || !cached_map(&mwgu, g.gu_w, 2 * g.F, g.H, 64) ||
        !cached_map(&mwd, g.d_w, g.H, g.F, TILE_W) || !cached_map(&mx8, g.x8, g.M, g.H, BN) ||
        !cached_map(&mh8, g.h8, g.M, g.F, BN))
        return rvhost::fail_msg(-2, "cuTensorMapEncodeTiled failed (driver entry point missing or bad operand layout)");
    BlkParams p = {};
    p.M = g.M;
    p.H = g.H;
    p.F = g.F;
    p.KO = g.KO;
    p.phases = g.phases;
    p.act = g.act;
    p.eps = g.eps;
    p.attn16 = g.attn16;
    p.attn_amax = g.attn_amax;
    p.amax_parts = g.amax_parts;
    p.attn_scale = g.attn_scale;
    p.o_wscale = g.o_wscale;
    p.residual = g.residual;
    p.gamma1 = g.gamma1;
    p.gamma2 = g.gamma2;
    p.x8 = (uint8_t*)g.x8;
    p.xs = g.xs;
    p.gu_wscale = g.gu_wscale;
    p.h8 = (uint8_t*)g.h8;
    p.hs = g.hs;
    p.d_wscale = g.d_wscale;
    p.bar = (unsigned int*)g.workspace;
    p.amax_ws = (float*)((char*)g.workspace + 256);
    p.part = (float*)((char*)g.workspace + 256 + blk_amax_bytes(g.F));
    p.trace = trace_buffer().load();
    if (cudaLaunchKernelEx(&cfg, kern, mwo, mwgu, mwd, mao, mx8, mh8, p) != cudaSuccess) {
        cudaGetLastError();
        return rvhost::fail_msg(-2, "layer-block kernel launch failed");
    }
    return 0;
}

// CTAs of the kernel one SM holds, from the per-SM limits: shared memory (dynamic + the per-CTA reservation),
// registers (allocated per warp in units of 256), threads, and tensor memory (512 columns, 32 per CTA).  The
// runtime's occupancy query is not used: it answers 1 for every kernel that allocates tensor memory, whatever its
// footprint, while the hardware co-schedules such CTAs as long as their columns fit (a profiler capture of the
// stand-alone GEMM, 63 KB and 84 registers, shows three per SM).
template <typename K> inline int block_capacity_of(K kern, int* per_sm, int* sms) {
    const int dev = rv_current_device();
    cudaFuncAttributes fa;
    int smem_sm = 0, smem_res = 0, regs_sm = 0, thr_sm = 0;
    if (dev < 0 || cudaFuncGetAttributes(&fa, kern) != cudaSuccess ||
        cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&smem_res, cudaDevAttrReservedSharedMemoryPerBlock, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&regs_sm, cudaDevAttrMaxRegistersPerMultiprocessor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&thr_sm, cudaDevAttrMaxThreadsPerMultiProcessor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    const int regs_warp = ((fa.numRegs * 32 + 255) / 256) * 256;
    int n = smem_sm / (SMEM_BYTES + (int)fa.sharedSizeBytes + smem_res);
    // (registers belong to the SM's four schedulers, a quarter each: whole warps per scheduler, not per SM)
    const int by_regs = 4 * ((regs_sm / 4) / regs_warp) / (THREADS / 32), by_thr = thr_sm / THREADS, by_tmem = 512 / 32;
    n = n < by_regs ? n : by_regs;
    n = n < by_thr ? n : by_thr;
    n = n < by_tmem ? n : by_tmem;
    *per_sm = n;
    return 0;
}
inline int block_capacity(int* per_sm, int* sms, int) {
    return block_capacity_of(fp8_layer_block_kernel<__nv_bfloat16>, per_sm, sms);
}

inline int launch_block(const BlkArgs& g, cudaStream_t s) {
    return g.dtype == 0 ? launch_block_t<__half>(g, s) : launch_block_t<__nv_bfloat16>(g, s);
}

}  // namespace rvblk
