// C-ABI entry points of FP8-KV paged decode attention: validation, workspace contract, launches.
#include <limits.h>
#include <math.h>

#include "../../include/rvllm_b200.h"
#include "../../include/rvllm_b200_tuning.h"
#include <atomic>
#include <mutex>

#include "host_util.h"
#include "paged_decode_fp8_tc.cuh"
#include "paged_decode_fp8_umma.cuh"

// Tuning overrides (declared in rvllm_b200_tuning.h).  Atomics: a setter racing a launch on another thread
// yields the old or the new value, never a torn one; a workspace query and its launch must still not
// straddle a change.
static std::atomic<int> g_target_ctas{rvattn::TARGET_CTAS};
static std::atomic<int> g_min_chunk_tokens{rvattn::MIN_CHUNK_TOKENS};
static std::atomic<int> g_cluster_combine{1};
static std::atomic<int> g_early_meta{0};       // 0: when the caller hinted it (below), 1: always, -1: never
static thread_local int t_early_meta_once = 0;  // one-shot hint of the calling thread, taken by its next launch
static std::atomic<int> g_cluster_min_tokens{rvua::TOK};  // smallest chunk of the cluster-merged split-KV form
// CTAs the cluster-merged form aims for: chunks cost it neither workspace traffic nor a second launch
constexpr int CLUSTER_TARGET_CTAS = rvattn::TARGET_CTAS;
static std::atomic<int> g_cluster_target{CLUSTER_TARGET_CTAS};
static std::atomic<int> g_ring_units{0};  // tcgen05 kernel: K/V ring depth in 16 KB units, 0 = automatic
static std::atomic<int> g_variant{0};  // 0 automatic (tcgen05 kernel where the shape allows, else 3, else 2), 1 FP32-pipe kernel,
                           // 2 mma.sync scores + FP32-pipe P.V, 3 both products on mma.sync, 4 tcgen05 / TMA

extern "C" {

void rvllm_paged_decode_tune(int target_ctas, int min_chunk_tokens, int variant) {
    g_variant = variant >= 0 && variant <= 4 ? variant : 0;
    g_target_ctas = target_ctas > 0 ? target_ctas : rvattn::TARGET_CTAS;
    g_min_chunk_tokens = min_chunk_tokens > 0 ? min_chunk_tokens : rvattn::MIN_CHUNK_TOKENS;
}
// ---------------------------------------------------------------- stage 3: attention
int rvllm_paged_decode_fp8_validate(int batch_size, int num_heads, int num_kv_heads, int head_dim,
                                    int block_size, int max_blocks_per_seq, int num_blocks_total,
                                    int window_size_left, float scale) {
    if (batch_size <= 0 || num_heads <= 0 || num_kv_heads <= 0)
        return rv_fail(RVLLM_E_INVALID, "batch, heads and kv_heads must be > 0");
    if (num_heads % num_kv_heads != 0) return rv_fail(RVLLM_E_INVALID, "heads must be a multiple of kv_heads");
    if (num_heads / num_kv_heads > 32) return rv_fail(RVLLM_E_INVALID, "GQA group larger than 32");
    if (head_dim != 64 && head_dim != 128 && head_dim != 256 && head_dim != 512)
        return rv_fail(RVLLM_E_INVALID, "head_dim must be 64, 128, 256 or 512");
    if (block_size <= 0 || max_blocks_per_seq <= 0 || num_blocks_total <= 0)
        return rv_fail(RVLLM_E_INVALID, "paging dimensions must be > 0");
    if (window_size_left < -1 || window_size_left == INT_MAX)
        return rv_fail(RVLLM_E_INVALID, "window_size_left must be >= -1");
    if (!isfinite(scale) || scale <= 0.0f) return rv_fail(RVLLM_E_INVALID, "scale must be finite and > 0");
    if (batch_size > INT_MAX / num_heads) return rv_fail(RVLLM_E_INVALID, "batch * heads overflows");
    const long long capacity = (long long)block_size * max_blocks_per_seq;
    if (window_size_left >= 0 && (long long)window_size_left + 1 > capacity)
        return rv_fail(RVLLM_E_INVALID, "window does not fit the block table");
    long long elems = (long long)num_blocks_total * block_size;
    if (elems > LLONG_MAX / num_kv_heads / head_dim) return rv_fail(RVLLM_E_INVALID, "cache size overflows");
    return RVLLM_OK;
}

int rvllm_paged_decode_max_chunks(int batch_size, int num_kv_heads) {
    return rvattn::pick_max_chunks(batch_size, num_kv_heads, g_target_ctas);
}

uint64_t rvllm_paged_decode_workspace_size(int batch_size, int num_heads, int num_kv_heads, int head_dim) {
    if (batch_size <= 0 || num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0 ||
        num_heads / num_kv_heads > 32 ||
        (head_dim != 64 && head_dim != 128 && head_dim != 256 && head_dim != 512))
        return UINT64_MAX;
    const int chunks = rvattn::pick_max_chunks(batch_size, num_kv_heads, g_target_ctas);
    if (chunks <= 1) return 0;
    unsigned long long v = (unsigned long long)batch_size * (unsigned long long)num_heads;
    if (v > (1ULL << 40)) return UINT64_MAX;
    return v * (unsigned long long)chunks * (unsigned long long)(head_dim + 2) * sizeof(float);
}

int rvllm_paged_decode_kernel_for(int num_heads, int num_kv_heads, int head_dim, int block_size, int num_blocks_total) {
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return rv_fail(RVLLM_E_INVALID, "bad head counts");
    rvattn::Params p = {};
    p.heads = num_heads;
    p.kv_heads = num_kv_heads;
    p.block_size = block_size;
    p.num_blocks_total = num_blocks_total;
    if ((g_variant == 4 || g_variant == 0) && rvua::supports(p, head_dim)) return 4;
    if (g_variant == 1) return 1;
    if (g_variant != 2 && head_dim <= 256 &&
        (long long)num_blocks_total * block_size * num_kv_heads < (1ll << 31))
        return 3;
    return 2;
}

void rvllm_paged_decode_early_meta(int mode) { g_early_meta = mode > 0 ? 1 : (mode < 0 ? -1 : 0); }
void rvllm_paged_decode_hint_early_meta(void) { t_early_meta_once = 1; }
void rvllm_paged_decode_cluster_combine(int enabled) { g_cluster_combine = enabled != 0; }
void rvllm_paged_decode_cluster_tune(int target_ctas, int min_chunk_tokens) {
    g_cluster_target = target_ctas > 0 ? target_ctas : CLUSTER_TARGET_CTAS;
    g_cluster_min_tokens = min_chunk_tokens > 0 ? min_chunk_tokens : rvua::TOK;
}

void rvllm_paged_decode_ring(int units) { g_ring_units = units > 0 ? units : 0; }

int rvllm_paged_decode_tc_status(int* status, int reset) {
    if (!status) return rv_fail(RVLLM_E_INVALID, "null status pointer");
    return rvua::read_status(status, reset != 0) ? rv_fail(RVLLM_E_LAUNCH, "cannot read the attention status word") : RVLLM_OK;
}

uint64_t rvllm_paged_decode_quant_workspace_size(int batch_size, int num_heads, int num_kv_heads, int head_dim) {
    if (rvllm_paged_decode_workspace_size(batch_size, num_heads, num_kv_heads, head_dim) == UINT64_MAX) return UINT64_MAX;
    const int chunks = rvattn::pick_max_chunks(batch_size, num_kv_heads, g_target_ctas);
    return (unsigned long long)batch_size * (unsigned long long)num_heads * (unsigned long long)(chunks < 1 ? 1 : chunks) *
           (unsigned long long)(head_dim + 2) * sizeof(float);
}

}  // extern "C"

namespace {

struct QuantOut {
    uint8_t* fp8 = nullptr;  // when set: fused combine + per-token quantisation instead of a 16-bit output
    float* scale = nullptr;
    float* amax = nullptr;   // when set (tcgen05 kernel, one chunk): max |stored output| per (sequence, kv_head)
};

// tcgen05 / TMA main kernel (head_dim 128 or 256, up to 8 query heads per KV head)
template <int HD, int GT, typename OutT, bool CL>
int launch_umma_form(const rvattn::Params& p, cudaStream_t s) {
    if constexpr (HD == 128 || HD == 256) {
        CUtensorMap mk, mv;
        const long long slots = (long long)p.num_blocks_total * p.block_size;
        if (!rvua::cache_map(&mk, p.k_cache, slots, p.kv_heads, HD, p.block_size) ||
            !rvua::cache_map(&mv, p.v_cache, slots, p.kv_heads, HD, p.block_size))
            return rv_fail(RVLLM_E_LAUNCH, "cuTensorMapEncodeTiled failed for the KV cache");
        auto kern = rvua::paged_decode_fp8_umma_kernel<HD, GT, OutT, CL>;
        using C = rvua::Cfg<HD>;
        static RvDeviceOnce smem_once;  // per kernel instantiation and device
        if (rv_allow_smem(smem_once, kern, C::smem_bytes(rvua::MAX_UNITS)))
            return rv_fail(RVLLM_E_LAUNCH, "cannot raise dynamic shared memory for decode attention");
        const int ring = g_ring_units.load();
        // cluster-combine form: the chunks of a (sequence, KV head) are one cluster, the receive area sits behind the rest
        // (and counts when the ring depth is chosen: a third of the footprint at eight chunks)
        const size_t recv = p.cluster_combine ? (size_t)C::recv_bytes(p.max_chunks, p.heads / p.kv_heads) : 0;
        int units = ring > 0 ? ring : rvua::pick_units<HD>((long long)p.kv_heads * p.max_chunks * p.batch, (int)recv);
        if (units < C::MIN_UNITS) units = C::MIN_UNITS;
        if (units > rvua::MAX_UNITS) units = rvua::MAX_UNITS;
        while (units > C::MIN_UNITS && C::smem_bytes(units) + recv > (size_t)C::smem_bytes(rvua::MAX_UNITS)) units--;
        rv_launch(kern, dim3(p.kv_heads, p.max_chunks, p.batch), dim3(rvua::THREADS), (size_t)C::smem_bytes(units) + recv, s,
                  dim3(1, p.cluster_combine ? p.max_chunks : 1, 1), mk, mv, p, units);
        return rv_launched("paged_decode_fp8 (tcgen05)");
    } else {
        return rv_fail(RVLLM_E_UNSUPPORTED, "tcgen05 decode attention needs head_dim 128 or 256");
    }
}

template <int HD, int GT, typename OutT>
int launch_umma(const rvattn::Params& p, cudaStream_t s) {
    return p.cluster_combine ? launch_umma_form<HD, GT, OutT, true>(p, s) : launch_umma_form<HD, GT, OutT, false>(p, s);
}

template <int HD, int GT, typename OutT>
int launch_main(const rvattn::Params& p, cudaStream_t s) {
    dim3 grid(p.kv_heads, p.max_chunks, p.batch);
    if ((g_variant == 4 || g_variant == 0) && rvua::supports(p, HD)) {
        const int group = p.heads / p.kv_heads;
        if (group <= 1) return launch_umma<HD, 1, OutT>(p, s);
        if (group <= 2) return launch_umma<HD, 2, OutT>(p, s);
        if (group <= 4) return launch_umma<HD, 4, OutT>(p, s);
        return launch_umma<HD, 8, OutT>(p, s);
    }
    return 1;  // not handled here
}

template <int HD, int GT, typename OutT>
int launch_attn(const rvattn::Params& p, const QuantOut& qo, cudaStream_t s) {
    dim3 grid(p.kv_heads, p.max_chunks, p.batch);
    int handled = launch_main<HD, GT, OutT>(p, s);
    if (handled < 0) return handled;
    if (handled == 0) {
        // launched by launch_main
    } else if (g_variant == 1) {
        auto kern = rvattn::paged_decode_fp8_kernel<HD, GT, OutT>;
        const size_t smem = rvattn::smem_bytes(HD, GT);
        static RvDeviceOnce smem_once;  // per kernel instantiation and device
        if (smem > 48 * 1024 && rv_allow_smem(smem_once, kern, (int)smem))
            return rv_fail(RVLLM_E_LAUNCH, "cannot raise dynamic shared memory for decode attention");
        rv_launch(kern, grid, dim3(rvattn::THREADS), smem, s, dim3(1, 1, 1), p);
    } else if (g_variant != 2 && HD <= 256 &&
               (long long)p.num_blocks_total * p.block_size * p.kv_heads < (1ll << 31)) {
        if constexpr (HD <= 256) {
            auto kern = rvattn::paged_decode_fp8_tc_kernel<HD, GT, OutT>;
            const size_t smem = rvattn::tc_smem_bytes(HD, GT);
            static RvDeviceOnce smem_once;  // per kernel instantiation and device
            if (smem > 48 * 1024 && rv_allow_smem(smem_once, kern, (int)smem))
                return rv_fail(RVLLM_E_LAUNCH, "cannot raise dynamic shared memory for decode attention");
            rv_launch(kern, grid, dim3(rvattn::MMA_THREADS), smem, s, dim3(1, 1, 1), p);
        }
    } else {
        auto kern = rvattn::paged_decode_fp8_mma_kernel<HD, GT, OutT>;
        const size_t smem = rvattn::mma_smem_bytes(HD, GT);
        static RvDeviceOnce smem_once;  // per kernel instantiation and device
        if (smem > 48 * 1024 && rv_allow_smem(smem_once, kern, (int)smem))
            return rv_fail(RVLLM_E_LAUNCH, "cannot raise dynamic shared memory for decode attention");
        rv_launch(kern, grid, dim3(rvattn::MMA_THREADS), smem, s, dim3(1, 1, 1), p);
    }
    int rc = rv_launched("paged_decode_fp8");
    if (rc) return rc;
    if (qo.fp8) {
        auto qk = rvattn::paged_decode_fp8_combine_quant_kernel<HD, OutT>;
        const size_t qsmem = (size_t)p.heads * HD * sizeof(float);
        static RvDeviceOnce q_once;
        if (qsmem > 48 * 1024 && rv_allow_smem(q_once, qk, 160 * 1024))
            return rv_fail(RVLLM_E_LAUNCH, "cannot raise dynamic shared memory for the attention quant pass");
        if (qsmem > 160 * 1024) return rv_fail(RVLLM_E_UNSUPPORTED, "heads * head_dim too large for the fused quant pass");
        rv_launch(qk, dim3(p.batch), dim3(512), qsmem, s, dim3(1, 1, 1), (const float*)p.workspace, qo.fp8, qo.scale,
                  (const int*)p.context_lens, p.heads, p.block_size, p.max_blocks_per_seq, p.window_size_left,
                  p.max_chunks, p.min_chunk_tokens);
        return rv_launched("paged_decode_fp8_combine_quant");
    }
    if (p.max_chunks > 1 && !p.cluster_combine) {
        rv_launch((rvattn::paged_decode_fp8_combine_kernel<HD, OutT>), dim3(p.batch * p.heads), dim3(HD < 256 ? HD : 256), 0,
                  s, dim3(1, 1, 1), (const float*)p.workspace, (OutT*)p.out, (const int*)p.context_lens, p.heads, p.block_size, p.max_blocks_per_seq,
            p.window_size_left, p.max_chunks, p.min_chunk_tokens);
        rc = rv_launched("paged_decode_fp8_combine");
    }
    return rc;
}

template <int HD, typename OutT>
int launch_attn_gt(const rvattn::Params& p, const QuantOut& qo, cudaStream_t s) {
    const int group = p.heads / p.kv_heads;
    if (group == 1) return launch_attn<HD, 1, OutT>(p, qo, s);
    if (group == 2) return launch_attn<HD, 2, OutT>(p, qo, s);
    return launch_attn<HD, 4, OutT>(p, qo, s);
}

template <typename OutT>
int launch_attn_hd(const rvattn::Params& p, const QuantOut& qo, int head_dim, cudaStream_t s) {
    switch (head_dim) {
        case 64: return launch_attn_gt<64, OutT>(p, qo, s);
        case 128: return launch_attn_gt<128, OutT>(p, qo, s);
        case 256: return launch_attn_gt<256, OutT>(p, qo, s);
        default: return launch_attn_gt<512, OutT>(p, qo, s);
    }
}

}  // namespace

extern "C" {

static int decode_core(const QuantOut& qo, const void* q_fp8, const void* k_cache_fp8, const void* v_cache_fp8, void* output,
                           int out_dtype, const int32_t* block_tables, const int32_t* context_lens,
                           void* workspace, size_t workspace_bytes, const float* k_scale_cache,
                           const float* v_scale_cache, const float* q_scale_cache, const float* q_descale,
                           const float* k_descale, const float* v_descale, float scale, int batch_size,
                           int num_heads, int num_kv_heads, int head_dim, int block_size,
                           int max_blocks_per_seq, int num_blocks_total, int window_size_left, void* stream) {
    int rc = rvllm_paged_decode_fp8_validate(batch_size, num_heads, num_kv_heads, head_dim, block_size,
                                             max_blocks_per_seq, num_blocks_total, window_size_left, scale);
    if (rc) return rc;
    if (!q_fp8 || !k_cache_fp8 || !v_cache_fp8 || (!output && !qo.fp8) || !block_tables || !context_lens)
        return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if ((!q_scale_cache && !q_descale) || (!k_scale_cache && !k_descale) || (!v_scale_cache && !v_descale))
        return rv_fail(RVLLM_E_INVALID, "each of Q, K, V needs a scale cache or a scalar descale");
    if (!rv_aligned(q_fp8, 16) || !rv_aligned(k_cache_fp8, 16) || !rv_aligned(v_cache_fp8, 16))
        return rv_fail(RVLLM_E_INVALID, "q / k_cache / v_cache must be 16-byte aligned");
    if (out_dtype != RVLLM_F16 && out_dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "bad output dtype");
    const int chunks = rvattn::pick_max_chunks(batch_size, num_kv_heads, g_target_ctas);
    const uint64_t need = qo.fp8 ? rvllm_paged_decode_quant_workspace_size(batch_size, num_heads, num_kv_heads, head_dim)
                                 : rvllm_paged_decode_workspace_size(batch_size, num_heads, num_kv_heads, head_dim);
    if (need == UINT64_MAX) return rv_fail(RVLLM_E_INVALID, "workspace size overflows");
    if ((chunks > 1 || qo.fp8) && (!workspace || !rv_aligned(workspace, sizeof(float)) || (uint64_t)workspace_bytes < need))
        return rv_fail(RVLLM_E_WORKSPACE, "attention workspace missing, misaligned or smaller than the query reports");
    rvattn::Params p;
    p.q = (const uint8_t*)q_fp8;
    p.k_cache = (const uint8_t*)k_cache_fp8;
    p.v_cache = (const uint8_t*)v_cache_fp8;
    p.out = output;
    p.workspace = (float*)workspace;
    p.block_tables = block_tables;
    p.context_lens = context_lens;
    p.k_scale_cache = k_scale_cache;
    p.v_scale_cache = v_scale_cache;
    p.q_scale_cache = q_scale_cache;
    p.q_descale = q_descale;
    p.k_descale = k_descale;
    p.v_descale = v_descale;
    p.scale = scale;
    p.batch = batch_size;
    p.heads = num_heads;
    p.kv_heads = num_kv_heads;
    p.block_size = block_size;
    p.bs_shift = -1;
    for (int sft = 0; sft < 31; sft++)
        if ((1 << sft) == block_size) p.bs_shift = sft;
    p.max_blocks_per_seq = max_blocks_per_seq;
    p.num_blocks_total = num_blocks_total;
    p.window_size_left = window_size_left;
    p.max_chunks = chunks;
    p.min_chunk_tokens = g_min_chunk_tokens;
    p.force_partial = qo.fp8 ? 1 : 0;
    p.amax_out = qo.amax;
    p.cluster_combine = 0;
    {
        const int mode = g_early_meta.load(), hinted = t_early_meta_once;
        t_early_meta_once = 0;
        p.early_meta = mode > 0 || (mode == 0 && hinted);
    }
    const bool umma = (g_variant == 4 || g_variant == 0) && rvua::supports(p, head_dim);
    const int cchunks = rvattn::pick_max_chunks(batch_size, num_kv_heads, g_cluster_target);
    if (umma && cchunks > 1 && !qo.fp8 && g_cluster_combine.load() != 0) {
        // Split-KV without the workspace round trip and the combine launch: up to 8 chunks of at least one
        // 128-token tile, one thread-block cluster per (sequence, KV head), merged in the chunk-0 CTA.
        int cc = cchunks < 8 ? cchunks : 8;
        const int group = num_heads / num_kv_heads;
        while (cc > 1 && cc * group * (head_dim + 2) * 4 > rvua::MAX_RECV_BYTES) cc--;
        if (cc > 1) {
            p.max_chunks = cc;
            p.min_chunk_tokens = g_cluster_min_tokens.load();
            p.cluster_combine = 1;
        }
    }
    if (qo.amax && !(umma && (chunks == 1 || p.cluster_combine)))
        return rv_fail(RVLLM_E_UNSUPPORTED, "the per-token absmax output needs the tcgen05 kernel with one chunk or the cluster merge");
    cudaStream_t s = (cudaStream_t)stream;
    return out_dtype == RVLLM_F16 ? launch_attn_hd<__half>(p, qo, head_dim, s)
                                  : launch_attn_hd<__nv_bfloat16>(p, qo, head_dim, s);
}

int rvllm_paged_decode_fp8(const void* q_fp8, const void* k_cache_fp8, const void* v_cache_fp8, void* output,
                           int out_dtype, const int32_t* block_tables, const int32_t* context_lens,
                           void* workspace, size_t workspace_bytes, const float* k_scale_cache,
                           const float* v_scale_cache, const float* q_scale_cache, const float* q_descale,
                           const float* k_descale, const float* v_descale, float scale, int batch_size,
                           int num_heads, int num_kv_heads, int head_dim, int block_size,
                           int max_blocks_per_seq, int num_blocks_total, int window_size_left, void* stream) {
    return decode_core(QuantOut(), q_fp8, k_cache_fp8, v_cache_fp8, output, out_dtype, block_tables, context_lens,
                       workspace, workspace_bytes, k_scale_cache, v_scale_cache, q_scale_cache, q_descale, k_descale,
                       v_descale, scale, batch_size, num_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq,
                       num_blocks_total, window_size_left, stream);
}

int rvllm_paged_decode_fp8_amax(const void* q_fp8, const void* k_cache_fp8, const void* v_cache_fp8, void* output,
                                int out_dtype, float* amax_out, const int32_t* block_tables, const int32_t* context_lens,
                                void* workspace, size_t workspace_bytes, const float* k_scale_cache,
                                const float* v_scale_cache, const float* q_scale_cache, const float* q_descale,
                                const float* k_descale, const float* v_descale, float scale, int batch_size,
                                int num_heads, int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                                int num_blocks_total, int window_size_left, void* stream) {
    if (!amax_out) return rv_fail(RVLLM_E_INVALID, "null device pointer");
    QuantOut qo;
    qo.amax = amax_out;
    return decode_core(qo, q_fp8, k_cache_fp8, v_cache_fp8, output, out_dtype, block_tables, context_lens, workspace,
                       workspace_bytes, k_scale_cache, v_scale_cache, q_scale_cache, q_descale, k_descale, v_descale,
                       scale, batch_size, num_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq,
                       num_blocks_total, window_size_left, stream);
}

int rvllm_paged_decode_fp8_quant(const void* q_fp8, const void* k_cache_fp8, const void* v_cache_fp8, void* out_fp8,
                                 float* out_scale, int round_dtype, const int32_t* block_tables,
                                 const int32_t* context_lens, void* workspace, size_t workspace_bytes,
                                 const float* k_scale_cache, const float* v_scale_cache, const float* q_scale_cache,
                                 const float* q_descale, const float* k_descale, const float* v_descale, float scale,
                                 int batch_size, int num_heads, int num_kv_heads, int head_dim, int block_size,
                                 int max_blocks_per_seq, int num_blocks_total, int window_size_left, void* stream) {
    if (!out_fp8 || !out_scale) return rv_fail(RVLLM_E_INVALID, "null device pointer");
    QuantOut qo;
    qo.fp8 = (uint8_t*)out_fp8;
    qo.scale = out_scale;
    return decode_core(qo, q_fp8, k_cache_fp8, v_cache_fp8, nullptr, round_dtype, block_tables, context_lens, workspace,
                       workspace_bytes, k_scale_cache, v_scale_cache, q_scale_cache, q_descale, k_descale, v_descale,
                       scale, batch_size, num_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq,
                       num_blocks_total, window_size_left, stream);
}

// ---- decode attention for callers that cannot allocate ---------------------------------------
// The split-KV partials normally live in a workspace the caller allocates.  Some callers have no
// allocator to ask: a runtime that carved all of its device memory into fixed regions at start-up
// and has nothing left over, or a plug-in whose host forbids it to call the CUDA allocator
// (an allocation can synchronise the device and stall every other stream).  For them the
// partials go into a scratch array that is part of this library's device image.
constexpr size_t STATIC_SCRATCH_BYTES = 8u << 20;  // every GPU that loads the library holds these 8 MiB
static __device__ __align__(256) float g_static_scratch[STATIC_SCRATCH_BYTES / sizeof(float)];

namespace {
// Device address of g_static_scratch per device ordinal.  In host code the array's name is only
// a handle for the runtime, never an address a kernel may use; cudaGetSymbolAddress translates it
// for the device that is current.
constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {nullptr};
std::mutex g_scratch_mu;

int static_scratch_ptr(float** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        cudaGetLastError();
        return rv_fail(RVLLM_E_NO_DEVICE, "no current CUDA device (or ordinal above %d)", MAX_DEVICES - 1);
    }
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return rv_fail(RVLLM_E_LAUNCH, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        }
        g_scratch_addr[dev] = (float*)p;
    }
    *out = g_scratch_addr[dev];
    return RVLLM_OK;
}
}  // namespace

size_t rvllm_paged_decode_static_scratch_bytes(void) { return STATIC_SCRATCH_BYTES; }

int rvllm_paged_decode_fp8_static_scratch(const void* q_fp8, const void* k_cache_fp8, const void* v_cache_fp8,
                                          void* output, int out_dtype, const int32_t* block_tables,
                                          const int32_t* context_lens, const float* k_scale_cache,
                                          const float* v_scale_cache, const float* q_scale_cache,
                                          const float* q_descale, const float* k_descale, const float* v_descale,
                                          float scale, int batch_size, int num_heads, int num_kv_heads, int head_dim,
                                          int block_size, int max_blocks_per_seq, int num_blocks_total,
                                          int window_size_left, void* stream) {
    const uint64_t need = rvllm_paged_decode_workspace_size(batch_size, num_heads, num_kv_heads, head_dim);
    if (need == UINT64_MAX) return rv_fail(RVLLM_E_INVALID, "shape rejected by the workspace query");
    if (need > STATIC_SCRATCH_BYTES)
        return rv_fail(RVLLM_E_WORKSPACE,
                       "this launch needs %llu bytes of split-KV scratch but the built-in scratch holds %llu; use "
                       "rvllm_paged_decode_fp8 with a caller-allocated workspace",
                       (unsigned long long)need, (unsigned long long)STATIC_SCRATCH_BYTES);
    float* scratch = nullptr;
    int rc = static_scratch_ptr(&scratch);  // first call on a device resolves the address
    if (rc) return rc;
    // Nothing in the scratch has to start at zero: every partial a launch reads back was written by
    // that same launch, so the previous call's contents are simply overwritten.
    return decode_core(QuantOut(), q_fp8, k_cache_fp8, v_cache_fp8, output, out_dtype, block_tables, context_lens,
                       scratch, STATIC_SCRATCH_BYTES, k_scale_cache, v_scale_cache, q_scale_cache, q_descale, k_descale,
                       v_descale, scale, batch_size, num_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq,
                       num_blocks_total, window_size_left, stream);
}

int rvllm_fa_sm89_abi_version(void) { return 2; }
int fa_sm89_fp8_output_dtype(void) { return 1; }
int fa_sm89_fp8_output_element_size(void) { return 2; }

uint64_t fa_sm89_decode_workspace_size(int batch_size, int num_heads, int num_kv_heads, int head_dim) {
    if (head_dim != 128 && head_dim != 256 && head_dim != 512) return UINT64_MAX;
    return rvllm_paged_decode_workspace_size(batch_size, num_heads, num_kv_heads, head_dim);
}

int fa_sm89_paged_decode_fp8(void* q_fp8, void* k_cache_fp8, void* v_cache_fp8, void* output,
                             void* block_tables, void* context_lens, void* workspace, size_t workspace_bytes,
                             void* k_scale_cache, void* v_scale_cache, void* q_scale_cache, float* q_descale,
                             float* k_descale, float* v_descale, float scale, int batch_size, int num_heads,
                             int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                             int num_blocks_total, int window_size_left, void* stream) {
    if (head_dim != 128 && head_dim != 256 && head_dim != 512) return -1;
    int rc = rvllm_paged_decode_fp8(q_fp8, k_cache_fp8, v_cache_fp8, output, RVLLM_F16, (const int32_t*)block_tables,
                                    (const int32_t*)context_lens, workspace, workspace_bytes,
                                    (const float*)k_scale_cache, (const float*)v_scale_cache,
                                    (const float*)q_scale_cache, q_descale, k_descale, v_descale, scale, batch_size,
                                    num_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq,
                                    num_blocks_total, window_size_left, stream);
    return rc == RVLLM_OK ? 0 : -1;
}

int fa_sm89_paged_decode(void*, void*, void*, void*, void*, void*, void*, size_t, float, int, int, int, int, int,
                         int, int, int, void*) {
    rv_fail(RVLLM_E_UNSUPPORTED, "f16-KV decode is outside the FP8 decode path");
    return -1;
}
int fa_sm89_paged_prefill_fp8(void*, void*, void*, void*, void*, void*, void*, void*, size_t, void*, void*, void*,
                              float*, float*, float*, float, int, int, int, int, int, int, int, int, int, int,
                              void*) {
    rv_fail(RVLLM_E_UNSUPPORTED, "FP8 prefill is outside the FP8 decode path");
    return -1;
}


}  // extern "C"
