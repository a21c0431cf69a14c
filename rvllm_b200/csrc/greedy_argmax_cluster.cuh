// Greedy argmax over f32 logits with each row spread over a thread-block cluster.  Included after
// greedy_argmax.cu (same translation unit): it reuses that file's candidate ordering, row scan and
// block reduction, so the winner is the one the one-CTA-per-row entry point reports -- greatest value,
// lowest index on ties, NaN never a candidate, -1 for a row without candidates.  A decode batch has a
// few dozen rows of about 1 MB each; one CTA per row leaves most SMs idle and streams at a fraction
// of the HBM rate, eight CTAs per row read the same bytes as one short burst.
// Geometry: grid = (CL, num_tokens), cluster = (CL, 1, 1), block = a multiple of 32 up to ARGMAX_CLUSTER_THREADS.
#pragma once
#include <cooperative_groups.h>

namespace rvargmax {

constexpr int ARGMAX_CLUSTER_THREADS = 1024;

__global__ void __launch_bounds__(ARGMAX_CLUSTER_THREADS)
argmax_cluster_f32_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    namespace cg = cooperative_groups;
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float win_v[8];  // rank 0's table of the CTAs' winners
    __shared__ int win_i[8];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank(), cl = (int)cluster.num_blocks();
    const int row = blockIdx.y;
    rv::pdl_launch();
    cluster.barrier_arrive();  // "this CTA runs": awaited before the store into rank 0
    rv::pdl_wait();
    // slices in whole 16-byte pieces of the row, so that every CTA scans with vector loads
    const long long pieces = ((long long)vocab + 3) >> 2;
    long long begin = 4 * (pieces * rank / cl), end = 4 * (pieces * (rank + 1) / cl);
    if (begin > vocab) begin = vocab;
    if (end > vocab) end = vocab;
    Cand b = scan_f32(logits + (long long)row * vocab, begin, end);
    b = block_best(b, sv, si);
    cluster.barrier_wait();
    if (threadIdx.x == 0) {
        *cluster.map_shared_rank(&win_v[rank], 0) = b.v;
        *cluster.map_shared_rank(&win_i[rank], 0) = b.i;
    }
    cluster.sync();
    if (rank == 0 && threadIdx.x == 0) {
        Cand r;
        r.v = -CUDART_INF_F;
        r.i = -1;
        for (int k = 0; k < cl; k++)
            if (better(win_v[k], win_i[k], r.v, r.i)) {
                r.v = win_v[k];
                r.i = win_i[k];
            }
        out[row] = r.i;
    }
}

}  // namespace rvargmax
