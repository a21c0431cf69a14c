// Weight-streaming FP8 E4M3 GEMM for decode-sized M (HBM-bound):
//     D[m, n] = epilogue( a_scale[m] * ( w_scale[n] * sum_k A[m, k] * W[n, k] ) )
// A [M, K] row-major fp8 (per-token scale), W [N, K] row-major fp8 (per-output-channel
// scale) — the operand layout of the reference's channel-scale GEMM
// (kernels/cutlass_fp8_gemm_channelscale.cu:98-161) and of its M=1 GEMV family
// (v3/kernels/fp8_channelscale_gemv_ktiled.cu:29-101).
//
// Shape of the kernel
//   * Weights are the 16-row operand of mma.sync.m16n8k32.e4m3 and the batch rows are
//     the 8-column operand, so one weight byte fetched from HBM is used for every
//     batch row while it sits in a register.  Each thread pulls its weight bytes with
//     128-bit streaming loads straight into fragment registers: the K index inside a
//     64-byte chunk is permuted identically for both operands (thread t of a quad owns
//     bytes 16t..16t+15), which a dot product does not notice.
//   * A CTA is 8 warps = 2 row-warps x 4 k-warps over a 64-row weight tile; every warp
//     owns 32 weight rows so an activation fragment (an L1 hit) feeds two MMAs.
//   * Split-K across a thread-block cluster: the S CTAs of a cluster take consecutive K
//     slices of the same weight tile, park their f32 partials in their own shared
//     memory, and after a cluster barrier each CTA reduces a share of the tile by
//     reading its peers' shared memory (DSMEM) in a fixed order.  No global scratch,
//     no atomics, bitwise reproducible.
//   * Epilogues: scale + narrow to 16 bit (f16 saturates), the same with a residual
//     add (in place allowed), or f32 (logits).
//   * M larger than the 64-row register tile is covered by gridDim.z M-blocks.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace rvgemm {

namespace cg = cooperative_groups;

constexpr int EPI_SCALE = 0;     // out16 = cast(a_s * (w_s * acc))
constexpr int EPI_RESIDUAL = 1;  // out16 = cast(a_s * (w_s * acc) + residual16)
constexpr int EPI_F32 = 2;       // out32 = a_s * (w_s * acc)

constexpr int TILE_N = 64;   // weight rows per CTA
constexpr int ROW_WARPS = 2; // 32 rows each
constexpr int K_WARPS = 4;
constexpr int THREADS = 32 * ROW_WARPS * K_WARPS;
constexpr int CHUNK = 64;    // K bytes one quad-row of threads covers per step

struct StreamParams {
    const uint8_t* a;
    const uint8_t* w;
    const float* a_scale;
    const float* w_scale;
    void* out;
    const void* residual;
    int M, N, K;
    int ldo;  // output / residual row stride in elements
};

__device__ __forceinline__ void mma_e4m3(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT8: batch rows handled per CTA, in units of 8 (1..8).
template <int NT8, int EPI, typename OutT>
__global__ void __launch_bounds__(THREADS, (NT8 <= 4 ? 2 : 1)) fp8_gemm_stream_kernel(StreamParams p) {
    constexpr int MB = NT8 * 8;
    extern __shared__ __align__(16) float part[];  // [K_WARPS][MB][TILE_N]
    cg::cluster_group cluster = cg::this_cluster();
    const int S = gridDim.y;           // cluster = (1, S, 1): rank == blockIdx.y
    const int split = blockIdx.y;
    const int n0 = blockIdx.x * TILE_N;
    const int m0 = blockIdx.z * MB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rw = warp % ROW_WARPS, kw = warp / ROW_WARPS;

    // K chunks are dealt out evenly over the S * K_WARPS k-warps of the cluster.
    const int chunks = p.K / CHUNK;
    const int j = split * K_WARPS + kw;
    const int c_lo = (int)((long long)j * chunks / (S * K_WARPS));
    const int c_hi = (int)((long long)(j + 1) * chunks / (S * K_WARPS));

    // Weight row pointers: two m16 tiles (rows g, g+8, g+16, g+24 of the warp's 32).
    const uint8_t* wrow[4];
#pragma unroll
    for (int r = 0; r < 4; r++) {
        int n = n0 + rw * 32 + g + 8 * r;
        n = n < p.N ? n : p.N - 1;  // rows past N are loaded from a valid row and dropped later
        wrow[r] = p.w + (size_t)n * p.K + 16 * t;
    }
    const uint8_t* arow[NT8];
#pragma unroll
    for (int i = 0; i < NT8; i++) {
        int m = m0 + 8 * i + g;
        m = m < p.M ? m : p.M - 1;
        arow[i] = p.a + (size_t)m * p.K + 16 * t;
    }

    rv::pdl_launch();
    rv::pdl_wait();  // activations and the residual come from the previous kernel
    float acc[2][NT8][4];
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int i = 0; i < NT8; i++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[r][i][q] = 0.0f;

    int c = c_lo;
    for (; c + 1 < c_hi; c += 2) {
        uint4 wv[2][4];
#pragma unroll
        for (int u = 0; u < 2; u++)
#pragma unroll
            for (int r = 0; r < 4; r++) wv[u][r] = rv::ld_stream128(wrow[r] + (size_t)(c + u) * CHUNK);
#pragma unroll
        for (int u = 0; u < 2; u++) {
#pragma unroll
            for (int i = 0; i < NT8; i++) {
                const uint4 av = rv::ldg128(arow[i] + (size_t)(c + u) * CHUNK);
                mma_e4m3(acc[0][i], wv[u][0].x, wv[u][1].x, wv[u][0].y, wv[u][1].y, av.x, av.y);
                mma_e4m3(acc[0][i], wv[u][0].z, wv[u][1].z, wv[u][0].w, wv[u][1].w, av.z, av.w);
                mma_e4m3(acc[1][i], wv[u][2].x, wv[u][3].x, wv[u][2].y, wv[u][3].y, av.x, av.y);
                mma_e4m3(acc[1][i], wv[u][2].z, wv[u][3].z, wv[u][2].w, wv[u][3].w, av.z, av.w);
            }
        }
    }
    if (c < c_hi) {
        uint4 wv[4];
#pragma unroll
        for (int r = 0; r < 4; r++) wv[r] = rv::ld_stream128(wrow[r] + (size_t)c * CHUNK);
#pragma unroll
        for (int i = 0; i < NT8; i++) {
            const uint4 av = rv::ldg128(arow[i] + (size_t)c * CHUNK);
            mma_e4m3(acc[0][i], wv[0].x, wv[1].x, wv[0].y, wv[1].y, av.x, av.y);
            mma_e4m3(acc[0][i], wv[0].z, wv[1].z, wv[0].w, wv[1].w, av.z, av.w);
            mma_e4m3(acc[1][i], wv[2].x, wv[3].x, wv[2].y, wv[3].y, av.x, av.y);
            mma_e4m3(acc[1][i], wv[2].z, wv[3].z, wv[2].w, wv[3].w, av.z, av.w);
        }
    }

    // Park partials: part[kw][m][n_local]; accumulator (row, col) = (weight row, batch row).
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int i = 0; i < NT8; i++) {
            const int nl = rw * 32 + r * 16 + g;
            const int ml = 8 * i + 2 * t;
            float* base = part + (size_t)kw * MB * TILE_N;
            base[(ml)*TILE_N + nl] = acc[r][i][0];
            base[(ml + 1) * TILE_N + nl] = acc[r][i][1];
            base[(ml)*TILE_N + nl + 8] = acc[r][i][2];
            base[(ml + 1) * TILE_N + nl + 8] = acc[r][i][3];
        }
    cluster.sync();

    // Each CTA of the cluster finishes an interleaved share of the MB x TILE_N tile.
    const float* peer[8];
#pragma unroll
    for (int s = 0; s < 8; s++) peer[s] = s < S ? cluster.map_shared_rank(part, s) : part;
    for (int e = split * THREADS + threadIdx.x; e < MB * TILE_N; e += S * THREADS) {
        const int ml = e / TILE_N, nl = e % TILE_N;
        const int m = m0 + ml, n = n0 + nl;
        float sum = 0.0f;
#pragma unroll
        for (int s = 0; s < 8; s++)
            if (s < S) {
#pragma unroll
                for (int k = 0; k < K_WARPS; k++) sum += peer[s][(size_t)k * MB * TILE_N + e];
            }
        if (m < p.M && n < p.N) {
            float v = p.a_scale[m] * (p.w_scale[n] * sum);
            const size_t o = (size_t)m * p.ldo + n;
            if (EPI == EPI_F32) {
                reinterpret_cast<float*>(p.out)[o] = v;
            } else {
                if (EPI == EPI_RESIDUAL) v += rv::T16<OutT>::to_f32(reinterpret_cast<const OutT*>(p.residual)[o]);
                reinterpret_cast<OutT*>(p.out)[o] = rv::T16<OutT>::from_f32_sat(v);
            }
        }
    }
    cluster.sync();  // peers may still be reading this CTA's shared memory
}

}  // namespace rvgemm
