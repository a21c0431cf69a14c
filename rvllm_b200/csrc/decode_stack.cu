// Decode stack: one decode step of a whole decoder stack recorded into a CUDA graph.
// Host-side orchestration only; every kernel is launched through the same C-ABI entry
// points a caller of the library would use, so the graph contains exactly those launches.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <vector>

#include "../../include/rvllm_b200.h"
#include "../../include/rvllm_b200_stack.h"
#include "../../include/rvllm_b200_tuning.h"
#include "common.cuh"
#include "host_util.h"

namespace {

struct LayerState {
    bool global;
    int head_dim, q_dim, kv_dim, qkv_n;
    int max_blocks;    // block-table length per sequence
    int num_blocks;    // physical blocks in this layer's cache
    int window_left;   // -1 for global layers
    uint8_t *k_cache, *v_cache;
    float *k_scale, *v_scale;
};

// physical block of (sequence b, page p) = an affine shuffle of b * max_blocks + p
// (mul coprime with n, chosen on the host from the seed)
__global__ void fill_tables_kernel(int* tables, int n, unsigned long long mul, unsigned long long add) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        tables[i] = (int)(((unsigned long long)i * mul + add) % (unsigned long long)n);
}

// Per-step bookkeeping, on the device so that a graph replay needs no host input: slot of the token written at
// position `pos`, for the global and the ring (sliding) layout, and the context length that includes it.
__device__ __forceinline__ void place_token(int b, int pos, const int* __restrict__ tables_global,
                                            const int* __restrict__ tables_sliding, int* __restrict__ slots_global,
                                            int* __restrict__ slots_sliding, int* __restrict__ ctx_lens, int block_size,
                                            int mb_global, int mb_sliding) {
    const int page = pos / block_size, off = pos % block_size;
    const int blk = page < mb_global ? tables_global[b * mb_global + page] : -1;  // -1: no block dealt to this page
    slots_global[b] = blk >= 0 ? blk * block_size + off : -1;
    slots_sliding[b] = mb_sliding > 0 ? tables_sliding[b * mb_sliding + page % mb_sliding] * block_size + off : -1;
    ctx_lens[b] = pos + 1;
}
// After a reset or a seeding: the bookkeeping of the first step.  Every later step finds what its predecessor's
// advance_kernel left, so that inside a step nothing writes slots, context lengths or block tables: kernels of the step
// may read them without waiting for the kernel before them.
__global__ void prepare_step_kernel(const int* __restrict__ positions, const int* __restrict__ tables_global,
                                    const int* __restrict__ tables_sliding, int* __restrict__ slots_global,
                                    int* __restrict__ slots_sliding, int* __restrict__ ctx_lens, int batch,
                                    int block_size, int mb_global, int mb_sliding) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch) return;
    place_token(b, positions[b], tables_global, tables_sliding, slots_global, slots_sliding, ctx_lens, block_size, mb_global,
                mb_sliding);
}

// After argmax: record the emitted token, choose the next input token (prompt while it lasts,
// then greedy feedback), advance the position and the step counter, and place the next step's token.  One block.
__global__ void advance_kernel(int* __restrict__ tokens, const int* __restrict__ next, int* __restrict__ positions,
                               const int* __restrict__ prompt, int prompt_len, int* __restrict__ history,
                               int* __restrict__ step_counter, int max_steps, int batch,
                               const int* __restrict__ tables_global, const int* __restrict__ tables_sliding,
                               int* __restrict__ slots_global, int* __restrict__ slots_sliding, int* __restrict__ ctx_lens,
                               int block_size, int mb_global, int mb_sliding) {
    rv::pdl_launch();
    rv::pdl_wait();
    const int step = *step_counter;
    for (int b = threadIdx.x; b < batch; b += blockDim.x) {
        const int pos = positions[b];
        const int emitted = next[b];
        if (step < max_steps) history[(size_t)step * batch + b] = emitted;
        tokens[b] = (pos + 1 < prompt_len) ? prompt[(size_t)b * prompt_len + pos + 1] : emitted;
        positions[b] = pos + 1;
        place_token(b, pos + 1, tables_global, tables_sliding, slots_global, slots_sliding, ctx_lens, block_size, mb_global,
                    mb_sliding);
    }
    __syncthreads();
    if (threadIdx.x == 0) *step_counter = step + 1;
}

__global__ void fill_f32_kernel(float* dst, size_t n, float v) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = v;
}
template <typename T>
__global__ void rope_table_kernel(T* cos_t, T* sin_t, int max_pos, int half, float theta);
template <>
__global__ void rope_table_kernel<__half>(__half* cos_t, __half* sin_t, int max_pos, int half, float theta) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= max_pos * half) return;
    const int pos = i / half, j = i % half;
    const float inv = powf(theta, -(float)j / (float)half);
    cos_t[i] = __float2half(cosf(pos * inv));
    sin_t[i] = __float2half(sinf(pos * inv));
}
template <>
__global__ void rope_table_kernel<__nv_bfloat16>(__nv_bfloat16* cos_t, __nv_bfloat16* sin_t, int max_pos, int half,
                                                 float theta) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= max_pos * half) return;
    const int pos = i / half, j = i % half;
    const float inv = powf(theta, -(float)j / (float)half);
    cos_t[i] = __float2bfloat16(cosf(pos * inv));
    sin_t[i] = __float2bfloat16(sinf(pos * inv));
}

inline size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

}  // namespace

struct rvllm_stack {
    rvllm_stack_config cfg;
    std::vector<rvllm_layer_weights> layers;
    rvllm_head_weights head;
    std::vector<LayerState> ls;
    cudaStream_t stream = nullptr;
    int skip_mask = 0;  // timing aid: launches left out of the step (rvllm_stack_debug_skip at creation time)
    bool capturing = false;  // enqueue_step is recording the graph (its kernels then run behind a complete predecessor step)
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int launches = 0;
    int steps_done = 0;
    int start_pos = 0;  // largest position any sequence had after the last reset / seeding (host-side copy)
    // one arena; everything below points into it
    uint8_t* arena = nullptr;
    size_t arena_bytes = 0;
    // scratch
    void* residual;      // [B, hidden] 16-bit
    uint8_t* x_fp8;      // [B, max(hidden, ffn, q_dim)]
    float* x_scale;      // [B]
    void* qkv;           // [B, max qkv_n] 16-bit
    uint8_t* q_fp8;      // [B, max q_dim]
    float* q_scale;      // [B, heads]
    void* attn_out;      // [B, max q_dim] 16-bit
    float* attn_amax;    // [B, kv_heads] max |attention output| per (sequence, kv_head)
    void* gateup;        // [B, 2*ffn] 16-bit
    uint8_t* attn_fp8;   // [B, max q_dim] attention output quantised per token (split-KV form)
    float* attn_scale;   // [B]
    uint8_t* h_fp8;      // [B, ffn] act(gate)*up of the layer-block kernel
    float* h_scale;      // [B]
    void* blk_ws;        // layer-block kernel: grid-barrier words + partial row maxima
    size_t blk_ws_bytes;
    void* arg_ws;        // fused greedy tail: per-tile (logit, token) winners
    size_t arg_ws_bytes;
    float* logits;       // [B, vocab]
    void* attn_ws;
    size_t attn_ws_bytes;
    void* gemm_ws;
    size_t gemm_ws_bytes;
    void *cos_s, *sin_s, *cos_g, *sin_g;
    int *tokens, *next_tokens, *positions, *ctx_lens, *slots_global, *slots_sliding, *tables_global, *tables_sliding;
    int *prompt, *history, *step_counter;
    int mb_global, mb_sliding;
    int32_t* pinned = nullptr;  // [2 * batch] staging for the host-buffer step
};

namespace {

int validate_cfg(const rvllm_stack_config* c) {
    if (!c) return rv_fail(RVLLM_E_INVALID, "config is null");
    if (c->hidden <= 0 || c->hidden % 64 || c->ffn <= 0 || c->ffn % 64)
        return rv_fail(RVLLM_E_INVALID, "hidden and ffn must be positive multiples of 64");
    if (c->vocab <= 0 || c->num_layers <= 0 || c->batch <= 0) return rv_fail(RVLLM_E_INVALID, "vocab, layers, batch must be > 0");
    if (c->heads <= 0 || c->kv_heads <= 0 || c->heads % c->kv_heads || c->heads / c->kv_heads > 32)
        return rv_fail(RVLLM_E_INVALID, "bad head counts");
    const int hds[2] = {c->sliding_head_dim, c->global_head_dim};
    for (int hd : hds)
        if (hd != 64 && hd != 128 && hd != 256 && hd != 512) return rv_fail(RVLLM_E_INVALID, "head_dim must be 64/128/256/512");
    if (c->sliding_window < 1 || c->global_every < 0) return rv_fail(RVLLM_E_INVALID, "bad window / layer pattern");
    if (c->act != RVLLM_ACT_SILU && c->act != RVLLM_ACT_GELU_TANH) return rv_fail(RVLLM_E_INVALID, "unknown activation");
    if (c->dtype != RVLLM_F16 && c->dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    if (c->block_size <= 0 || c->max_context <= 0 || c->max_steps <= 0 || c->prompt_len < 0)
        return rv_fail(RVLLM_E_INVALID, "bad paging / step capacities");
    if (c->prompt_len > c->max_context) return rv_fail(RVLLM_E_INVALID, "prompt longer than the cache");
    if (!isfinite(c->rms_eps) || c->rms_eps < 0 || !isfinite(c->rope_theta) || c->rope_theta <= 1.0f)
        return rv_fail(RVLLM_E_INVALID, "bad eps / rope theta");
    if (c->gemm_impl < 0 || c->gemm_impl > 2) return rv_fail(RVLLM_E_INVALID, "gemm_impl must be 0, 1 or 2");
    if (c->kv_pool_blocks < 0) return rv_fail(RVLLM_E_INVALID, "kv_pool_blocks must be >= 0");
    if (c->fused_block != 0 && c->fused_block != 1) return rv_fail(RVLLM_E_INVALID, "fused_block must be 0 or 1");
    if (c->fused_argmax != 0 && c->fused_argmax != 1) return rv_fail(RVLLM_E_INVALID, "fused_argmax must be 0 or 1");
    if (!isfinite(c->logit_softcap) || c->logit_softcap < 0.0f) return rv_fail(RVLLM_E_INVALID, "logit_softcap must be >= 0");
    return RVLLM_OK;
}

bool is_global(const rvllm_stack_config& c, int layer) {
    if (c.global_every == 0) return false;
    return (layer + 1) % c.global_every == 0;
}

// Lays the stack's buffers out in one arena.  With base == nullptr only the size is computed.
size_t layout(rvllm_stack* s, uint8_t* base) {
    const rvllm_stack_config& c = s->cfg;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        uint8_t* p = base ? base + off : nullptr;
        off += align256(bytes);
        return p;
    };
    const int B = c.batch;
    int max_q = 0, max_qkv = 0;
    s->ls.resize(c.num_layers);
    s->mb_global = (c.max_context + c.block_size - 1) / c.block_size;
    s->mb_sliding = (c.sliding_window + c.block_size - 1) / c.block_size + 1;
    bool any_sliding = false;
    for (int l = 0; l < c.num_layers; l++) {
        LayerState& L = s->ls[l];
        L.global = is_global(c, l);
        any_sliding |= !L.global;
        L.head_dim = L.global ? c.global_head_dim : c.sliding_head_dim;
        L.q_dim = c.heads * L.head_dim;
        L.kv_dim = c.kv_heads * L.head_dim;
        L.qkv_n = L.q_dim + 2 * L.kv_dim;
        L.max_blocks = L.global ? s->mb_global : s->mb_sliding;
        // a global layer's physical blocks: one full table per sequence, or the shared pool of a ragged batch
        L.num_blocks = (L.global && c.kv_pool_blocks > 0) ? c.kv_pool_blocks : B * L.max_blocks;
        L.window_left = L.global ? -1 : c.sliding_window - 1;
        max_q = L.q_dim > max_q ? L.q_dim : max_q;
        max_qkv = L.qkv_n > max_qkv ? L.qkv_n : max_qkv;
        const size_t slots = (size_t)L.num_blocks * c.block_size;
        L.k_cache = take(slots * L.kv_dim);
        L.v_cache = take(slots * L.kv_dim);
        L.k_scale = (float*)take(slots * c.kv_heads * sizeof(float));
        L.v_scale = (float*)take(slots * c.kv_heads * sizeof(float));
    }
    if (!any_sliding) s->mb_sliding = 0;
    int widest = c.hidden > c.ffn ? c.hidden : c.ffn;
    widest = widest > max_q ? widest : max_q;
    s->residual = take((size_t)B * c.hidden * 2);
    s->x_fp8 = take((size_t)B * widest);
    s->x_scale = (float*)take((size_t)B * sizeof(float));
    s->qkv = take((size_t)B * max_qkv * 2);
    s->q_fp8 = take((size_t)B * max_q);
    s->q_scale = (float*)take((size_t)B * c.heads * sizeof(float));
    s->attn_out = take((size_t)B * max_q * 2);
    s->attn_amax = (float*)take((size_t)B * c.kv_heads * sizeof(float));
    s->gateup = take((size_t)B * 2 * c.ffn * 2);
    s->attn_fp8 = take((size_t)B * max_q);
    s->attn_scale = (float*)take((size_t)B * sizeof(float));
    s->h_fp8 = take((size_t)B * c.ffn);
    s->h_scale = (float*)take((size_t)B * sizeof(float));
    s->blk_ws_bytes = rvllm_fp8_layer_block_workspace(c.hidden, c.ffn);   // (0 when the shape is never taken: the kernel is not used then)
    s->blk_ws = take(s->blk_ws_bytes ? s->blk_ws_bytes : 256);  // zeroed with the arena: the barrier words start at zero
    s->arg_ws_bytes = rvllm_fp8_gemm_lm_head_argmax_workspace(B, c.vocab);
    s->arg_ws = take(s->arg_ws_bytes);
    s->logits = (float*)take((size_t)B * c.vocab * sizeof(float));
    uint64_t aw = 0;
    for (int hd : {c.sliding_head_dim, c.global_head_dim}) {
        uint64_t w = rvllm_paged_decode_quant_workspace_size(B, c.heads, c.kv_heads, hd);
        aw = w > aw ? w : aw;
    }
    s->attn_ws_bytes = (size_t)aw;
    s->attn_ws = take(aw ? aw : 256);
    size_t gw = rvllm_fp8_gemm_workspace(B, c.vocab > 2 * c.ffn ? c.vocab : 2 * c.ffn, c.hidden > c.ffn ? c.hidden : c.ffn);
    s->gemm_ws_bytes = gw;
    s->gemm_ws = take(gw ? gw : 256);
    const int max_pos = c.max_context;
    s->cos_s = take((size_t)max_pos * (c.sliding_head_dim / 2) * 2);
    s->sin_s = take((size_t)max_pos * (c.sliding_head_dim / 2) * 2);
    s->cos_g = take((size_t)max_pos * (c.global_head_dim / 2) * 2);
    s->sin_g = take((size_t)max_pos * (c.global_head_dim / 2) * 2);
    s->tokens = (int*)take(B * 4);
    s->next_tokens = (int*)take(B * 4);
    s->positions = (int*)take(B * 4);
    s->ctx_lens = (int*)take(B * 4);
    s->slots_global = (int*)take(B * 4);
    s->slots_sliding = (int*)take(B * 4);
    s->tables_global = (int*)take((size_t)B * s->mb_global * 4);
    s->tables_sliding = (int*)take((size_t)B * (s->mb_sliding > 0 ? s->mb_sliding : 1) * 4);
    s->prompt = (int*)take((size_t)B * (c.prompt_len > 0 ? c.prompt_len : 1) * 4);
    s->history = (int*)take((size_t)c.max_steps * B * 4);
    s->step_counter = (int*)take(256);
    return off;
}

}  // namespace

namespace {

#define RV_TRY(expr)                 \
    do {                             \
        int rc_ = (expr);            \
        if (rc_ != RVLLM_OK) return rc_; \
    } while (0)

// Timing aid (rvllm_stack_debug_skip): launches left out of the steps of stacks created while it is set.
std::atomic<int> g_skip_mask{0};

// Enqueues one decode step on the stack's stream; counts launches when asked.
// The bookkeeping of the first step after the positions were set from the host (plain launch, stream order).
int place_first_tokens(rvllm_stack* s) {
    const rvllm_stack_config& c = s->cfg;
    prepare_step_kernel<<<(c.batch + 127) / 128, 128, 0, s->stream>>>(s->positions, s->tables_global, s->tables_sliding,
                                                                      s->slots_global, s->slots_sliding, s->ctx_lens, c.batch,
                                                                      c.block_size, s->mb_global, s->mb_sliding);
    return rv_launched("prepare_step");
}

int enqueue_step(rvllm_stack* s, int* launches) {
    const int skip = s->skip_mask;
    auto on = [skip](int bit) { return (skip & bit) == 0; };
    const rvllm_stack_config& c = s->cfg;
    const int B = c.batch, H = c.hidden;
    void* st = (void*)s->stream;
    int n = 0;
    // (slots, context lengths and block tables of this step were left by the previous step's advance_kernel, or by
    // reset / seeding: nothing below writes them)
    RV_TRY(rvllm_embedding_gather_launch(s->residual, s->head.embedding, s->tokens, B, H, c.vocab, st));
    n++;
    // x_fp8 / x_scale hold the current layer's attention-block input (RMSNorm + quant of the residual) when the
    // previous layer's block kernel has already produced it
    bool x_ready = false;
    for (int l = 0; l < c.num_layers; l++) {
        const LayerState& L = s->ls[l];
        const rvllm_layer_weights& W = s->layers[l];
        const int es = 2;
        if (!x_ready && on(1)) {
            RV_TRY(rvllm_fused_rmsnorm_fp8_quant_launch(B, H, c.rms_eps, s->x_fp8, s->x_scale, s->residual,
                                                        W.attn_norm_gamma, c.dtype, st));
            n++;
        }
        x_ready = false;
        // QKV projection, RoPE, Q quantisation and the paged KV write: one launch where the library
        // takes the shape (head_dim 128, batch <= 32, tensor-core GEMM), else the GEMM and the RoPE kernel
        int fused = RVLLM_E_UNSUPPORTED;
        if (!on(2)) fused = RVLLM_OK, n--;  // (left out: timing aid)
        else if (L.head_dim == 128 && c.gemm_impl != 1)
            fused = rvllm_fp8_gemm_qkv_rope_fp8kv(s->x_fp8, W.qkv_w, s->x_scale, W.qkv_scale, B, H, c.heads, c.kv_heads,
                                                  L.head_dim, c.dtype, s->q_fp8, s->q_scale, L.k_cache, L.v_cache,
                                                  L.k_scale, L.v_scale, L.global ? s->cos_g : s->cos_s,
                                                  L.global ? s->sin_g : s->sin_s, s->positions,
                                                  L.global ? s->slots_global : s->slots_sliding, c.max_context,
                                                  L.num_blocks * c.block_size, st);
        if (fused == RVLLM_E_UNSUPPORTED) {
            RV_TRY(rvllm_fp8_gemm_channelscale(s->qkv, c.dtype, s->x_fp8, W.qkv_w, s->x_scale, W.qkv_scale, nullptr, B,
                                               L.qkv_n, H, c.gemm_impl, s->gemm_ws, s->gemm_ws_bytes, st));
            const char* qkv = (const char*)s->qkv;
            RV_TRY(rvllm_rope_fp8kv_launch(qkv, qkv + (size_t)es * L.q_dim, qkv + (size_t)es * (L.q_dim + L.kv_dim),
                                           L.qkv_n, s->q_fp8, L.k_cache, L.v_cache, L.k_scale, L.v_scale, s->q_scale,
                                           L.global ? s->cos_g : s->cos_s, L.global ? s->sin_g : s->sin_s,
                                           s->positions, L.global ? s->slots_global : s->slots_sliding, B, c.heads,
                                           c.kv_heads, L.head_dim, L.head_dim, c.max_context,
                                           L.num_blocks * c.block_size, c.dtype, st));
            n += 2;
        } else {
            RV_TRY(fused);
            n++;
        }
        const float sm_scale = 1.0f / sqrtf((float)L.head_dim);
        const int* tables = L.global ? s->tables_global : s->tables_sliding;
        // Attention leaves its output in one of two forms.  (a) 16-bit values + per-(row, kv_head) maxima: the tcgen05
        // kernel at batch <= 32 — the O projection quantises its own A tiles.  (b) FP8 rows + per-row scales: split-KV
        // through the workspace, the combine pass quantises (same bytes as attention -> per-token quantiser); also
        // what the plain call + quantiser produce.
        bool have16 = false;
        const bool try16 = B <= 32 && c.gemm_impl != 1 &&
                           rvllm_paged_decode_kernel_for(c.heads, c.kv_heads, L.head_dim, c.block_size, L.num_blocks) == 4;
        if (!on(4)) {
            have16 = try16;  // (left out: timing aid)
        } else {
            // (a) first: single chunk, or split-KV merged inside a thread-block cluster (small batches)
            // In the graph the step's bookkeeping (context lengths, slots) and every older cache row were complete
            // before the step began — they come from the previous graph launch or from reset / seeding — so attention
            // need not wait for the QKV kernel before it reads them.  Eager launches chain across steps: no hint.
            int a16 = RVLLM_E_UNSUPPORTED;
            if (s->capturing) rvllm_paged_decode_hint_early_meta();
            if (try16)
                a16 = rvllm_paged_decode_fp8_amax(s->q_fp8, L.k_cache, L.v_cache, s->attn_out, c.dtype, s->attn_amax,
                                                  tables, s->ctx_lens, s->attn_ws, s->attn_ws_bytes, L.k_scale,
                                                  L.v_scale, s->q_scale, nullptr, nullptr, nullptr, sm_scale, B,
                                                  c.heads, c.kv_heads, L.head_dim, c.block_size, L.max_blocks,
                                                  L.num_blocks, L.window_left, st);
            if (a16 == RVLLM_OK) {
                have16 = true;
                n++;
            } else if (a16 != RVLLM_E_UNSUPPORTED) {
                RV_TRY(a16);
            } else if (rvllm_paged_decode_max_chunks(B, c.kv_heads) > 1) {
                if (s->capturing) rvllm_paged_decode_hint_early_meta();
                RV_TRY(rvllm_paged_decode_fp8_quant(s->q_fp8, L.k_cache, L.v_cache, s->attn_fp8, s->attn_scale, c.dtype, tables,
                                                    s->ctx_lens, s->attn_ws, s->attn_ws_bytes, L.k_scale, L.v_scale,
                                                    s->q_scale, nullptr, nullptr, nullptr, sm_scale, B, c.heads,
                                                    c.kv_heads, L.head_dim, c.block_size, L.max_blocks, L.num_blocks,
                                                    L.window_left, st));
                n += 2;
            } else {
                if (s->capturing) rvllm_paged_decode_hint_early_meta();
                RV_TRY(rvllm_paged_decode_fp8(s->q_fp8, L.k_cache, L.v_cache, s->attn_out, c.dtype, tables,
                                              s->ctx_lens, s->attn_ws, s->attn_ws_bytes, L.k_scale, L.v_scale,
                                              s->q_scale, nullptr, nullptr, nullptr, sm_scale, B, c.heads, c.kv_heads,
                                              L.head_dim, c.block_size, L.max_blocks, L.num_blocks, L.window_left, st));
                RV_TRY(rvllm_quantize_fp8_per_token_launch(B, L.q_dim, s->attn_fp8, s->attn_scale, s->attn_out, c.dtype, st));
                n += 2;
            }
        }
        // Everything up to the next attention in one launch where the library takes the shape (batch <= 32, hidden a
        // multiple of 128, ffn <= 4 * hidden): O projection, RMSNorm + quant, gate|up, act*up + quant, down, and the
        // RMSNorm + quant that opens the next layer (or closes the stack).
        int blk = RVLLM_E_UNSUPPORTED;
        if (c.gemm_impl != 1 && c.fused_block != 0 && s->blk_ws_bytes > 0) {
            const void* next_gamma = l + 1 < c.num_layers ? s->layers[l + 1].attn_norm_gamma : s->head.final_norm_gamma;
            blk = rvllm_fp8_layer_block(B, H, c.ffn, L.q_dim, c.act, c.dtype, c.rms_eps, have16 ? s->attn_out : nullptr,
                                        s->attn_amax, c.kv_heads, have16 ? nullptr : s->attn_fp8, s->attn_scale, W.o_w,
                                        W.o_scale, s->residual, W.mlp_norm_gamma, next_gamma, s->x_fp8, s->x_scale,
                                        W.gateup_w, W.gateup_scale, s->h_fp8, s->h_scale, W.down_w, W.down_scale,
                                        s->blk_ws, s->blk_ws_bytes, RVLLM_BLOCK_ALL, st);
        }
        if (blk == RVLLM_OK) {
            x_ready = true;
            n++;
            continue;
        }
        if (blk != RVLLM_E_UNSUPPORTED) RV_TRY(blk);
        if (!on(8)) {
            n--;
        } else if (have16) {
            RV_TRY(rvllm_fp8_gemm_residual_from16(s->residual, c.dtype, s->attn_out, s->attn_amax, c.kv_heads, W.o_w,
                                                  W.o_scale, s->residual, B, H, L.q_dim, st));
        } else {
            RV_TRY(rvllm_fp8_gemm_channelscale(s->residual, c.dtype, s->attn_fp8, W.o_w, s->attn_scale, W.o_scale,
                                               s->residual, B, H, L.q_dim, c.gemm_impl, s->gemm_ws, s->gemm_ws_bytes, st));
        }
        if (on(16))
            RV_TRY(rvllm_fused_rmsnorm_fp8_quant_launch(B, H, c.rms_eps, s->x_fp8, s->x_scale, s->residual,
                                                        W.mlp_norm_gamma, c.dtype, st));
        if (on(32))
            RV_TRY(rvllm_fp8_gemm_channelscale(s->gateup, c.dtype, s->x_fp8, W.gateup_w, s->x_scale, W.gateup_scale,
                                               nullptr, B, 2 * c.ffn, H, c.gemm_impl, s->gemm_ws, s->gemm_ws_bytes, st));
        if (on(64))
            RV_TRY(rvllm_fused_act_mul_fp8_quant_launch(B, c.ffn, c.act, s->x_fp8, s->x_scale, s->gateup, c.dtype, st));
        if (on(128))
            RV_TRY(rvllm_fp8_gemm_channelscale(s->residual, c.dtype, s->x_fp8, W.down_w, s->x_scale, W.down_scale,
                                               s->residual, B, H, c.ffn, c.gemm_impl, s->gemm_ws, s->gemm_ws_bytes, st));
        n += 5 - !on(16) - !on(32) - !on(64) - !on(128);
    }
    if (!x_ready) {
        RV_TRY(rvllm_fused_rmsnorm_fp8_quant_launch(B, H, c.rms_eps, s->x_fp8, s->x_scale, s->residual,
                                                    s->head.final_norm_gamma, c.dtype, st));
        n++;
    }
    // Greedy tail: the LM head keeps only each weight tile's best (logit, token) and a merge picks the row's winner
    // (no [batch, vocab] f32 logits in HBM); or the LM head into f32 logits, the optional soft cap, argmax.
    int tail = RVLLM_E_UNSUPPORTED;
    if (c.fused_argmax != 0 && c.gemm_impl != 1)
        tail = rvllm_fp8_gemm_lm_head_argmax(s->next_tokens, s->x_fp8, s->head.lm_head_w, s->x_scale, s->head.lm_head_scale,
                                             B, c.vocab, H, c.logit_softcap, s->arg_ws, s->arg_ws_bytes, st);
    if (tail == RVLLM_OK) {
        n += 2;
    } else {
        if (tail != RVLLM_E_UNSUPPORTED) RV_TRY(tail);
        RV_TRY(rvllm_fp8_gemm_channelscale(s->logits, RVLLM_OUT_F32, s->x_fp8, s->head.lm_head_w, s->x_scale,
                                           s->head.lm_head_scale, nullptr, B, c.vocab, H, c.gemm_impl, s->gemm_ws,
                                           s->gemm_ws_bytes, st));
        n++;
        if (c.logit_softcap > 0.0f) {
            RV_TRY(rvllm_logit_softcap_launch(s->logits, B, c.vocab, c.logit_softcap, RVLLM_OUT_F32, st));
            n++;
        }
        RV_TRY(rvllm_argmax_launch(B, c.vocab, s->logits, s->next_tokens, 0, st));
        n++;
    }
    rv_launch(advance_kernel, dim3(1), dim3(256), 0, s->stream, dim3(1, 1, 1), s->tokens, s->next_tokens, s->positions, s->prompt, c.prompt_len,
                                             s->history, s->step_counter, c.max_steps, B, (const int*)s->tables_global,
                                             (const int*)s->tables_sliding, s->slots_global, s->slots_sliding, s->ctx_lens,
                                             c.block_size, s->mb_global, s->mb_sliding);
    RV_TRY(rv_launched("advance"));
    n += 1;
    if (launches) *launches = n;
    return RVLLM_OK;
}

int cuda_ok(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return RVLLM_OK;
    cudaGetLastError();
    return rv_fail(RVLLM_E_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

unsigned long long coprime_multiplier(unsigned long long seed, unsigned long long n) {
    auto gcd = [](unsigned long long a, unsigned long long b) {
        while (b) {
            unsigned long long t = a % b;
            a = b;
            b = t;
        }
        return a;
    };
    if (n <= 2) return 1;
    unsigned long long m = (seed * 6364136223846793005ull + 1442695040888963407ull) % n;
    if (m < 2) m = 2;
    while (gcd(m, n) != 1) m = m + 1 < n ? m + 1 : 2;
    return m;
}


// Deals the global layers' block pool out to the sequences.  need[b] = blocks sequence b may touch (NULL: an
// equal share each).  Physical ids come from a seeded shuffle of the pool; table entries past a sequence's
// share are -1 (no slot: the KV write of such a position is skipped, as for any negative slot).
int assign_pool_blocks(rvllm_stack* s, const int* need) {
    const rvllm_stack_config& c = s->cfg;
    const int B = c.batch, mb = s->mb_global, pool = c.kv_pool_blocks;
    std::vector<int> table((size_t)B * mb, -1), perm((size_t)pool);
    for (int i = 0; i < pool; i++) perm[i] = i;
    unsigned long long x = c.seed * 0x9E3779B97F4A7C15ull + 0xD1B54A32D192ED03ull;
    for (int i = pool - 1; i > 0; i--) {  // Fisher-Yates with a splitmix-style stream
        x += 0x9E3779B97F4A7C15ull;
        unsigned long long z = x;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        const int j = (int)(z % (unsigned long long)(i + 1));
        const int t = perm[i];
        perm[i] = perm[j];
        perm[j] = t;
    }
    long long used = 0;
    for (int b = 0; b < B; b++) {
        int n = need ? need[b] : pool / B;
        if (n > mb) n = mb;
        if (used + n > pool) return rv_fail(RVLLM_E_INVALID, "the KV block pool (%d blocks) is too small for this batch", pool);
        for (int p = 0; p < n; p++) table[(size_t)b * mb + p] = perm[(size_t)used + p];
        used += n;
    }
    RV_TRY(cuda_ok(cudaMemcpyAsync(s->tables_global, table.data(), table.size() * sizeof(int), cudaMemcpyHostToDevice,
                                   s->stream), "upload block tables"));
    return cuda_ok(cudaStreamSynchronize(s->stream), "upload block tables");  // `table` must outlive the copy
}

}  // namespace

extern "C" {

int rvllm_stack_config_validate(const rvllm_stack_config* cfg) { return validate_cfg(cfg); }

uint64_t rvllm_stack_device_bytes(const rvllm_stack_config* cfg) {
    if (validate_cfg(cfg) != RVLLM_OK) return 0;
    rvllm_stack tmp;
    tmp.cfg = *cfg;
    return (uint64_t)layout(&tmp, nullptr);
}

int rvllm_stack_create(rvllm_stack** out, const rvllm_stack_config* cfg, const rvllm_layer_weights* layers,
                       const rvllm_head_weights* head) {
    if (!out || !layers || !head) return rv_fail(RVLLM_E_INVALID, "null argument");
    RV_TRY(validate_cfg(cfg));
    for (int l = 0; l < cfg->num_layers; l++) {
        const rvllm_layer_weights& w = layers[l];
        if (!w.attn_norm_gamma || !w.qkv_w || !w.qkv_scale || !w.o_w || !w.o_scale || !w.mlp_norm_gamma ||
            !w.gateup_w || !w.gateup_scale || !w.down_w || !w.down_scale)
            return rv_fail(RVLLM_E_INVALID, "layer %d has a null weight pointer", l);
    }
    if (!head->embedding || !head->final_norm_gamma || !head->lm_head_w || !head->lm_head_scale)
        return rv_fail(RVLLM_E_INVALID, "head has a null weight pointer");
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        cudaGetLastError();
        return rv_fail(RVLLM_E_NO_DEVICE, "no CUDA device");
    }
    rvllm_stack* s = new rvllm_stack();
    s->cfg = *cfg;
    s->skip_mask = g_skip_mask.load();
    s->layers.assign(layers, layers + cfg->num_layers);
    s->head = *head;
    s->arena_bytes = layout(s, nullptr);
    int rc = cuda_ok(cudaMalloc((void**)&s->arena, s->arena_bytes), "cudaMalloc(stack arena)");
    if (rc == RVLLM_OK) rc = cuda_ok(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking), "cudaStreamCreate");
    if (rc == RVLLM_OK) rc = cuda_ok(cudaMallocHost((void**)&s->pinned, sizeof(int32_t) * 2 * cfg->batch), "cudaMallocHost");
    if (rc != RVLLM_OK) {
        rvllm_stack_destroy(s);
        return rc;
    }
    layout(s, s->arena);
    cudaMemsetAsync(s->arena, 0, s->arena_bytes, s->stream);
    // block tables: shuffled physical order, one table per cache layout
    const unsigned long long ng = (unsigned long long)cfg->batch * s->mb_global;
    int pool_rc = RVLLM_OK;
    if (cfg->kv_pool_blocks > 0) {
        // ragged batch: every sequence gets an equal share of the pool until rvllm_stack_seed_contexts deals
        // the blocks out by need
        pool_rc = assign_pool_blocks(s, nullptr);
    } else {
        fill_tables_kernel<<<64, 256, 0, s->stream>>>(s->tables_global, (int)ng, coprime_multiplier(cfg->seed, ng),
                                                      cfg->seed % ng);
    }
    if (s->mb_sliding > 0) {
        const unsigned long long nsl = (unsigned long long)cfg->batch * s->mb_sliding;
        fill_tables_kernel<<<64, 256, 0, s->stream>>>(s->tables_sliding, (int)nsl,
                                                      coprime_multiplier(cfg->seed + 1, nsl), (cfg->seed / 3) % nsl);
    }
    const int hs = cfg->sliding_head_dim / 2, hg = cfg->global_head_dim / 2, mp = cfg->max_context;
    if (cfg->dtype == RVLLM_F16) {
        rope_table_kernel<__half><<<(mp * hs + 255) / 256, 256, 0, s->stream>>>((__half*)s->cos_s, (__half*)s->sin_s, mp, hs, cfg->rope_theta);
        rope_table_kernel<__half><<<(mp * hg + 255) / 256, 256, 0, s->stream>>>((__half*)s->cos_g, (__half*)s->sin_g, mp, hg, cfg->rope_theta);
    } else {
        rope_table_kernel<__nv_bfloat16><<<(mp * hs + 255) / 256, 256, 0, s->stream>>>((__nv_bfloat16*)s->cos_s, (__nv_bfloat16*)s->sin_s, mp, hs, cfg->rope_theta);
        rope_table_kernel<__nv_bfloat16><<<(mp * hg + 255) / 256, 256, 0, s->stream>>>((__nv_bfloat16*)s->cos_g, (__nv_bfloat16*)s->sin_g, mp, hg, cfg->rope_theta);
    }
    rc = pool_rc != RVLLM_OK ? pool_rc : rv_launched("stack set-up kernels");
    if (rc == RVLLM_OK) rc = cuda_ok(cudaStreamSynchronize(s->stream), "stack set-up");
    // One eager step sets every function attribute and tensor map before capture; its effects
    // are wiped by the reset below.
    if (rc == RVLLM_OK) rc = enqueue_step(s, &s->launches);
    if (rc == RVLLM_OK) rc = cuda_ok(cudaStreamSynchronize(s->stream), "eager warm-up step");
    if (rc == RVLLM_OK) rc = cuda_ok(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal), "begin capture");
    if (rc == RVLLM_OK) {
        s->capturing = true;
        int rc2 = enqueue_step(s, nullptr);
        s->capturing = false;
        cudaError_t e = cudaStreamEndCapture(s->stream, &s->graph);
        rc = rc2 != RVLLM_OK ? rc2 : cuda_ok(e, "end capture");
    }
    if (rc == RVLLM_OK) rc = cuda_ok(cudaGraphInstantiate(&s->exec, s->graph, 0), "graph instantiate");
    if (rc == RVLLM_OK) rc = rvllm_stack_reset(s, nullptr);
    if (rc != RVLLM_OK) {
        rvllm_stack_destroy(s);
        return rc;
    }
    *out = s;
    return RVLLM_OK;
}

void rvllm_stack_destroy(rvllm_stack* s) {
    if (!s) return;
    if (s->stream) cudaStreamSynchronize(s->stream);
    if (s->exec) cudaGraphExecDestroy(s->exec);
    if (s->graph) cudaGraphDestroy(s->graph);
    if (s->pinned) cudaFreeHost(s->pinned);
    if (s->arena) cudaFree(s->arena);
    if (s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

int rvllm_stack_reset(rvllm_stack* s, const int32_t* prompt_tokens) {
    if (!s) return rv_fail(RVLLM_E_INVALID, "stack is null");
    const rvllm_stack_config& c = s->cfg;
    RV_TRY(cuda_ok(cudaStreamSynchronize(s->stream), "sync before reset"));
    // caches and scale caches need no clearing: a position is always written before it is read
    cudaMemsetAsync(s->positions, 0, sizeof(int) * c.batch, s->stream);
    cudaMemsetAsync(s->step_counter, 0, sizeof(int), s->stream);
    cudaMemsetAsync(s->tokens, 0, sizeof(int) * c.batch, s->stream);
    cudaMemsetAsync(s->history, 0, sizeof(int) * (size_t)c.max_steps * c.batch, s->stream);
    if (prompt_tokens && c.prompt_len > 0) {
        RV_TRY(cuda_ok(cudaMemcpyAsync(s->prompt, prompt_tokens, sizeof(int) * (size_t)c.batch * c.prompt_len,
                                       cudaMemcpyHostToDevice, s->stream), "upload prompt"));
        // first input token of every sequence = prompt[b][0]
        RV_TRY(cuda_ok(cudaMemcpy2DAsync(s->tokens, sizeof(int), prompt_tokens, sizeof(int) * c.prompt_len, sizeof(int),
                                         c.batch, cudaMemcpyHostToDevice, s->stream), "upload first tokens"));
    } else if (c.prompt_len > 0) {
        cudaMemsetAsync(s->prompt, 0, sizeof(int) * (size_t)c.batch * c.prompt_len, s->stream);
    }
    s->steps_done = 0;
    s->start_pos = 0;
    RV_TRY(place_first_tokens(s));
    return cuda_ok(cudaStreamSynchronize(s->stream), "reset");
}

static int seed_common(rvllm_stack* s, const int32_t* contexts, int uniform) {
    const rvllm_stack_config& c = s->cfg;
    RV_TRY(rvllm_stack_reset(s, nullptr));
    std::vector<int> pos((size_t)c.batch, uniform), need;
    int most = uniform;
    if (contexts)
        for (int b = 0; b < c.batch; b++) {
            if (contexts[b] < 0 || contexts[b] >= c.max_context) return rv_fail(RVLLM_E_INVALID, "bad seeded context");
            pos[b] = contexts[b];
            most = contexts[b] > most ? contexts[b] : most;
        }
    if (c.kv_pool_blocks > 0) {
        // a sequence may touch positions [0, context + steps still to come): max_steps bounds those
        need.resize(c.batch);
        for (int b = 0; b < c.batch; b++) {
            long long last = (long long)pos[b] + c.max_steps;
            if (last > c.max_context) last = c.max_context;
            need[b] = (int)((last + c.block_size - 1) / c.block_size);
        }
        RV_TRY(assign_pool_blocks(s, need.data()));
    }
    for (const LayerState& L : s->ls) {
        const size_t slots = (size_t)L.num_blocks * c.block_size;
        cudaMemsetAsync(L.k_cache, 0x34, slots * L.kv_dim, s->stream);  // 0.75 in E4M3
        cudaMemsetAsync(L.v_cache, 0xb2, slots * L.kv_dim, s->stream);  // -0.625
        fill_f32_kernel<<<256, 256, 0, s->stream>>>(L.k_scale, slots * c.kv_heads, 0.02f);
        fill_f32_kernel<<<256, 256, 0, s->stream>>>(L.v_scale, slots * c.kv_heads, 0.03f);
    }
    RV_TRY(rv_launched("seed context"));
    RV_TRY(cuda_ok(cudaMemcpyAsync(s->positions, pos.data(), sizeof(int) * c.batch, cudaMemcpyHostToDevice, s->stream),
                   "upload positions"));
    RV_TRY(place_first_tokens(s));
    RV_TRY(cuda_ok(cudaStreamSynchronize(s->stream), "seed context"));
    s->start_pos = most;
    return RVLLM_OK;
}

int rvllm_stack_seed_context(rvllm_stack* s, int context) {
    if (!s || context < 0 || context >= s->cfg.max_context) return rv_fail(RVLLM_E_INVALID, "bad seeded context");
    return seed_common(s, nullptr, context);
}

int rvllm_stack_seed_contexts(rvllm_stack* s, const int32_t* contexts) {
    if (!s || !contexts) return rv_fail(RVLLM_E_INVALID, "bad seeded contexts");
    return seed_common(s, contexts, 0);
}

// A step at position p writes slot p of a global layer's cache: positions must stay below max_context, or the
// write is skipped and attention reads rows that were never written.  Refused before anything is launched.
static int room_for(rvllm_stack* s, int n) {
    if ((long long)s->start_pos + s->steps_done + n > s->cfg.max_context)
        return rv_fail(RVLLM_E_INVALID, "%d more step(s) would pass max_context = %d (position %d now)", n,
                       s->cfg.max_context, s->start_pos + s->steps_done);
    return RVLLM_OK;
}

int rvllm_stack_run(rvllm_stack* s, int n) {
    if (!s || n < 0) return rv_fail(RVLLM_E_INVALID, "bad run arguments");
    RV_TRY(room_for(s, n));
    for (int i = 0; i < n; i++) RV_TRY(cuda_ok(cudaGraphLaunch(s->exec, s->stream), "graph launch"));
    s->steps_done += n;
    return RVLLM_OK;
}

int rvllm_stack_run_eager(rvllm_stack* s, int n) {
    if (!s || n < 0) return rv_fail(RVLLM_E_INVALID, "bad run arguments");
    RV_TRY(room_for(s, n));
    for (int i = 0; i < n; i++) RV_TRY(enqueue_step(s, nullptr));
    s->steps_done += n;
    return RVLLM_OK;
}

int rvllm_stack_sync(rvllm_stack* s) {
    if (!s) return rv_fail(RVLLM_E_INVALID, "stack is null");
    return cuda_ok(cudaStreamSynchronize(s->stream), "stack sync");
}

int rvllm_stack_step_host(rvllm_stack* s, const int32_t* tokens_in, int32_t* tokens_out) {
    if (!s || !tokens_out) return rv_fail(RVLLM_E_INVALID, "bad step arguments");
    RV_TRY(room_for(s, 1));
    const int B = s->cfg.batch;
    if (tokens_in) {
        memcpy(s->pinned, tokens_in, sizeof(int32_t) * B);
        RV_TRY(cuda_ok(cudaMemcpyAsync(s->tokens, s->pinned, sizeof(int32_t) * B, cudaMemcpyHostToDevice, s->stream),
                       "upload tokens"));
    }
    RV_TRY(cuda_ok(cudaGraphLaunch(s->exec, s->stream), "graph launch"));
    RV_TRY(cuda_ok(cudaMemcpyAsync(s->pinned + B, s->next_tokens, sizeof(int32_t) * B, cudaMemcpyDeviceToHost,
                                   s->stream), "download tokens"));
    RV_TRY(cuda_ok(cudaStreamSynchronize(s->stream), "step sync"));
    memcpy(tokens_out, s->pinned + B, sizeof(int32_t) * B);
    s->steps_done += 1;
    return RVLLM_OK;
}

int rvllm_stack_read_tokens(rvllm_stack* s, int first, int count, int32_t* out) {
    if (!s || !out || first < 0 || count < 0) return rv_fail(RVLLM_E_INVALID, "bad read arguments");
    RV_TRY(cuda_ok(cudaStreamSynchronize(s->stream), "sync before read"));
    int avail = s->steps_done < s->cfg.max_steps ? s->steps_done : s->cfg.max_steps;
    if (first >= avail) return 0;
    if (first + count > avail) count = avail - first;
    RV_TRY(cuda_ok(cudaMemcpy(out, s->history + (size_t)first * s->cfg.batch, sizeof(int) * (size_t)count * s->cfg.batch,
                              cudaMemcpyDeviceToHost), "read history"));
    return count;
}

void rvllm_stack_debug_skip(int mask) { g_skip_mask = mask; }

int rvllm_stack_steps_done(rvllm_stack* s) { return s ? s->steps_done : -1; }
int rvllm_stack_launches_per_step(const rvllm_stack* s) { return s ? s->launches : -1; }
void* rvllm_stack_stream(rvllm_stack* s) { return s ? (void*)s->stream : nullptr; }

int rvllm_stack_debug_read(rvllm_stack* s, int what, void* host_out, size_t bytes) {
    if (!s || !host_out) return rv_fail(RVLLM_E_INVALID, "bad debug read");
    const void* src = nullptr;
    size_t have = 0;
    if (what == 0) { src = s->residual; have = (size_t)s->cfg.batch * s->cfg.hidden * 2; }
    else if (what == 1) {
        if (s->cfg.fused_argmax != 0 && s->cfg.gemm_impl != 1)
            return rv_fail(RVLLM_E_INVALID, "logits are not materialised when the argmax is fused into the LM head");
        src = s->logits;
        have = (size_t)s->cfg.batch * s->cfg.vocab * 4;
    }
    else if (what == 2) { src = s->positions; have = (size_t)s->cfg.batch * 4; }
    else return rv_fail(RVLLM_E_INVALID, "unknown buffer");
    if (bytes > have) return rv_fail(RVLLM_E_INVALID, "buffer is smaller than requested");
    RV_TRY(cuda_ok(cudaStreamSynchronize(s->stream), "sync before debug read"));
    return cuda_ok(cudaMemcpy(host_out, src, bytes, cudaMemcpyDeviceToHost), "debug read");
}

}  // extern "C"
