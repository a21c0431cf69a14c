// PTX module `argmax`: greedy token selection over f32 (or f16) logits.
//
// Entry-point contracts (reference kernels/argmax.cu:34,81,132; launcher
// v3/crates/rvllm-fused/src/launcher.rs:369-397):
//   argmax_kernel / argmax_f16_kernel : grid = (num_tokens), block = min(vocab, 1024),
//       a power of two; any other block shape writes -1.
//   argmax_grid_f32_kernel            : grid = (ceil(vocab / 1024), num_tokens), block = 256,
//       output pre-set by the caller (cuMemsetD32Async to 0); partial winners are
//       merged into the output cell with compare-and-swap.
// Ordering rule everywhere: a candidate wins if its value is greater, or equal with a
// lower index; NaN is never a candidate; -inf may win; a row with no candidate gives -1.
//
// Each thread scans with 128-bit loads, four in flight, so one CTA keeps enough bytes
// outstanding to stream a 1 MB row; the winner is reduced with shuffles, then across
// warps through 64 words of shared memory.
#include "common.cuh"

namespace {

struct Cand {
    float v;
    int i;
};
__device__ __forceinline__ bool better(float cv, int ci, float bv, int bi) {
    if (ci < 0) return false;
    if (bi < 0) return true;
    return cv > bv || (cv == bv && ci < bi);
}
__device__ __forceinline__ void take(Cand& b, float v, int i) {
    if (v == v && better(v, i, b.v, b.i)) {
        b.v = v;
        b.i = i;
    }
}
__device__ __forceinline__ Cand warp_best(Cand b) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
        int oi = __shfl_xor_sync(0xffffffffu, b.i, o);
        if (better(ov, oi, b.v, b.i)) {
            b.v = ov;
            b.i = oi;
        }
    }
    return b;
}
__device__ __forceinline__ Cand block_best(Cand b, float* sv, int* si) {
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    b = warp_best(b);
    if (l == 0) {
        sv[w] = b.v;
        si[w] = b.i;
    }
    __syncthreads();
    Cand r;
    r.v = l < nw ? sv[l] : -CUDART_INF_F;
    r.i = l < nw ? si[l] : -1;
    return warp_best(r);  // every warp computes the same winner
}
__device__ __forceinline__ bool launch_ok(int vocab) {
    const int n = blockDim.x;
    return vocab > 0 && n > 0 && n <= 1024 && (n & (n - 1)) == 0 && blockDim.y == 1 && blockDim.z == 1;
}

// scan x[begin, end) of one row; indices reported relative to the row start
__device__ __forceinline__ Cand scan_f32(const float* __restrict__ x, long long begin, long long end) {
    Cand b;
    b.v = -CUDART_INF_F;
    b.i = -1;
    const int tid = threadIdx.x, nt = blockDim.x;
    long long head = begin;
    // peel until 16-byte aligned
    while (head < end && (reinterpret_cast<uintptr_t>(x + head) & 15) != 0) head++;
    if (head > end) head = end;
    for (long long i = begin + tid; i < head; i += nt) take(b, x[i], (int)i);
    const long long nvec = (end - head) >> 2;
    const float4* xv = reinterpret_cast<const float4*>(x + head);
    long long v = tid;
    for (; v + 3LL * nt < nvec; v += 4LL * nt) {
        float4 a0 = __ldcs(xv + v), a1 = __ldcs(xv + v + nt), a2 = __ldcs(xv + v + 2LL * nt),
               a3 = __ldcs(xv + v + 3LL * nt);
        const float4 q[4] = {a0, a1, a2, a3};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            int idx = (int)(head + 4 * (v + (long long)k * nt));
            take(b, q[k].x, idx);
            take(b, q[k].y, idx + 1);
            take(b, q[k].z, idx + 2);
            take(b, q[k].w, idx + 3);
        }
    }
    for (; v < nvec; v += nt) {
        float4 a = __ldcs(xv + v);
        int idx = (int)(head + 4 * v);
        take(b, a.x, idx);
        take(b, a.y, idx + 1);
        take(b, a.z, idx + 2);
        take(b, a.w, idx + 3);
    }
    for (long long i = head + 4 * nvec + tid; i < end; i += nt) take(b, x[i], (int)i);
    return b;
}

}  // namespace

extern "C" __global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    __shared__ float sv[32];
    __shared__ int si[32];
    rv::pdl_launch();
    rv::pdl_wait();
    const int row = blockIdx.x;
    if (logits == nullptr || out == nullptr || !launch_ok(vocab)) {
        if (out != nullptr && threadIdx.x == 0) out[row] = -1;
        return;
    }
    Cand b = scan_f32(logits + (long long)row * vocab, 0, vocab);
    b = block_best(b, sv, si);
    if (threadIdx.x == 0) out[row] = b.i;
}

extern "C" __global__ void argmax_f16_kernel(const __half* __restrict__ logits, int* __restrict__ out, int vocab) {
    __shared__ float sv[32];
    __shared__ int si[32];
    rv::pdl_launch();
    rv::pdl_wait();
    const int row = blockIdx.x;
    if (logits == nullptr || out == nullptr || !launch_ok(vocab)) {
        if (out != nullptr && threadIdx.x == 0) out[row] = -1;
        return;
    }
    const __half* x = logits + (long long)row * vocab;
    Cand b;
    b.v = -CUDART_INF_F;
    b.i = -1;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) take(b, __half2float(x[i]), i);
    b = block_best(b, sv, si);
    if (threadIdx.x == 0) out[row] = b.i;
}

extern "C" __global__ void argmax_grid_f32_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    __shared__ float sv[32];
    __shared__ int si[32];
    rv::pdl_launch();
    rv::pdl_wait();
    if (logits == nullptr || out == nullptr || !launch_ok(vocab)) return;
    const int row = blockIdx.y, parts = gridDim.x;
    const long long chunk = ((long long)vocab + parts - 1) / parts;
    const long long begin = (long long)blockIdx.x * chunk;
    const long long end = begin + chunk < vocab ? begin + chunk : vocab;
    const float* x = logits + (long long)row * vocab;
    Cand b = scan_f32(x, begin < end ? begin : end, end);
    b = block_best(b, sv, si);
    if (threadIdx.x != 0 || b.i < 0) return;
    // Merge into the caller-initialised cell: replace the current holder when it is not a
    // valid index, holds a NaN, or loses under the ordering rule.
    int* cell = out + row;
    int cur = *cell;
    for (;;) {
        bool replace;
        if (cur < 0 || cur >= vocab) {
            replace = true;
        } else {
            float cv = x[cur];
            replace = (cv != cv) || b.v > cv || (b.v == cv && b.i < cur);
        }
        if (!replace) break;
        int old = atomicCAS(cell, cur, b.i);
        if (old == cur) break;
        cur = old;
    }
}
