// Host side of the C ABI: argument validation mirroring the reference launch descriptors,
// geometry selection and kernel launches.  No device allocation, no synchronisation; every
// call only enqueues work on the caller's stream.
#include <limits.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>

#include "../../include/rvllm_b200.h"
#include "../../include/rvllm_b200_tuning.h"
#include "host_util.h"
// the PTX-module translation units double as this library's kernels
#include "greedy_argmax.cu"
#include "greedy_argmax_cluster.cuh"
#include "rope_kv_write.cu"
#include "rowq_gelu.cu"
#include "rowq_blockscale.cu"
#include "rowq_gemma.cu"
#include "rowq_rmsnorm.cu"
#include "rowq_silu.cu"

namespace {

thread_local char g_err[512] = "";

}  // namespace

int rv_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}
// The reference launchers pass min(dim, 1024) threads as is; a block that is not a whole
// number of warps would run full-mask shuffles with missing lanes, so it is rounded down
// (identical to the reference geometry for every dimension that is a multiple of 32).
static inline uint32_t round_block(uint32_t b) { return b < 32 ? 32 : b - b % 32; }

int rv_launched(const char* what) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();
        return rv_fail(RVLLM_E_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
    }
    return RVLLM_OK;
}
static std::atomic<bool> g_pdl{true};
bool rv_pdl_enabled() { return g_pdl.load(std::memory_order_relaxed); }
void rv_set_pdl(bool on) { g_pdl.store(on, std::memory_order_relaxed); }

namespace rvhost {
int fail_msg(int code, const char* msg) { return rv_fail(code, "%s", msg); }
}  // namespace rvhost

extern "C" {

int rvllm_b200_abi_version(void) { return 1; }
const char* rvllm_b200_last_error(void) { return g_err; }
const char* rvllm_b200_build_arch(void) { return "sm_100a"; }
void rvllm_b200_set_pdl(int enabled) { rv_set_pdl(enabled != 0); }
int rvllm_b200_get_pdl(void) { return rv_pdl_enabled() ? 1 : 0; }

int rvllm_b200_selftest_device_once(void) {
    RvDeviceOnce once;
    int calls = 0;
    auto ok = [&]() { calls++; return 0; };
    auto bad = [&]() { calls++; return -1; };
    if (once.seen(0) || once.seen(1)) return 1;
    if (once.run(0, ok) != 0 || calls != 1 || !once.seen(0) || once.seen(1)) return 2;   // first use of device 0
    if (once.run(0, ok) != 0 || calls != 1) return 3;                                    // remembered
    if (once.run(1, bad) != -1 || calls != 2 || once.seen(1)) return 4;                  // a failure is not remembered
    if (once.run(1, ok) != 0 || calls != 3 || !once.seen(1)) return 5;                   // device 1 has its own flag
    if (once.run(70, ok) != 0 || calls != 4 || !once.seen(70) || once.seen(6)) return 6; // second word of the table
    if (once.run(-1, ok) != 0 || once.run(-1, ok) != 0 || calls != 6) return 7;          // unknown device: every time
    if (once.run(RvDeviceOnce::MAX_DEVICES, ok) != 0 || calls != 7) return 8;
    return 0;
}

// ---------------------------------------------------------------- stage 1
int rvllm_fused_rmsnorm_fp8_quant_validate(uint32_t num_tokens, uint32_t hidden, float eps) {
    if (hidden == 0 || hidden % 8 != 0) return rv_fail(RVLLM_E_INVALID, "hidden must be a positive multiple of 8");
    if (num_tokens == 0) return rv_fail(RVLLM_E_INVALID, "num_tokens must be > 0");
    if (!isfinite(eps) || eps < 0.0f) return rv_fail(RVLLM_E_INVALID, "eps must be finite and >= 0");
    return RVLLM_OK;
}

int rvllm_fused_rmsnorm_fp8_quant_launch(uint32_t num_tokens, uint32_t hidden, float eps, void* out_fp8,
                                         float* scale, const void* in_hidden, const void* gamma, int dtype,
                                         void* stream) {
    int rc = rvllm_fused_rmsnorm_fp8_quant_validate(num_tokens, hidden, eps);
    if (rc) return rc;
    if (!out_fp8 || !scale || !in_hidden || !gamma) return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    dim3 grid(num_tokens), block(round_block(rv_umin(hidden, 1024)));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RVLLM_F16)
        rv_launch(fused_rmsnorm_fp8_quant_kernel, dim3(grid), dim3(block), 128, s, dim3(1, 1, 1), (uint8_t*)out_fp8, scale, (const __half*)in_hidden,
                                                                (const __half*)gamma, eps, (int)hidden);
    else
        rv_launch(fused_rmsnorm_fp8_quant_bf16_kernel, dim3(grid), dim3(block), 128, s, dim3(1, 1, 1), (uint8_t*)out_fp8, scale,
                                                                     (const __nv_bfloat16*)in_hidden,
                                                                     (const __nv_bfloat16*)gamma, eps, (int)hidden);
    return rv_launched("fused_rmsnorm_fp8_quant");
}

int rvllm_fused_add_rmsnorm_fp8_quant_launch(uint32_t num_tokens, uint32_t hidden, float eps, void* out_fp8,
                                             float* scale, void* residual_out, const void* in_hidden,
                                             const void* residual_in, const void* gamma, int dtype,
                                             void* stream) {
    int rc = rvllm_fused_rmsnorm_fp8_quant_validate(num_tokens, hidden, eps);
    if (rc) return rc;
    if (!out_fp8 || !scale || !residual_out || !in_hidden || !residual_in || !gamma)
        return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    dim3 grid(num_tokens), block(round_block(rv_umin(hidden, 1024)));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RVLLM_F16)
        rv_launch(fused_add_rmsnorm_fp8_quant_kernel, dim3(grid), dim3(block), 128, s, dim3(1, 1, 1), 
            (uint8_t*)out_fp8, scale, (__half*)residual_out, (const __half*)in_hidden, (const __half*)residual_in,
            (const __half*)gamma, eps, (int)hidden);
    else
        rv_launch(fused_add_rmsnorm_fp8_quant_bf16_kernel, dim3(grid), dim3(block), 128, s, dim3(1, 1, 1), 
            (uint8_t*)out_fp8, scale, (__nv_bfloat16*)residual_out, (const __nv_bfloat16*)in_hidden,
            (const __nv_bfloat16*)residual_in, (const __nv_bfloat16*)gamma, eps, (int)hidden);
    return rv_launched("fused_add_rmsnorm_fp8_quant");
}

int rvllm_quantize_fp8_per_token_validate(uint32_t num_tokens, uint32_t dim) {
    if (dim == 0 || dim % 8 != 0) return rv_fail(RVLLM_E_INVALID, "dim must be a positive multiple of 8");
    if (num_tokens == 0) return rv_fail(RVLLM_E_INVALID, "num_tokens must be > 0");
    if (dim > 65536) return rv_fail(RVLLM_E_INVALID, "dim must be <= 65536");
    return RVLLM_OK;
}

int rvllm_quantize_fp8_per_token_launch(uint32_t num_tokens, uint32_t dim, void* out_fp8, float* scale,
                                        const void* in, int dtype, void* stream) {
    int rc = rvllm_quantize_fp8_per_token_validate(num_tokens, dim);
    if (rc) return rc;
    if (!out_fp8 || !scale || !in) return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    dim3 grid(num_tokens), block(round_block(rv_umax(rv_umin(dim, 1024), 256)));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RVLLM_F16)
        rv_launch(quantize_fp8_per_token_kernel, dim3(grid), dim3(block), 128, s, dim3(1, 1, 1), (uint8_t*)out_fp8, scale, (const __half*)in, (int)dim);
    else
        rv_launch(quantize_fp8_per_token_bf16_kernel, dim3(grid), dim3(block), 128, s, dim3(1, 1, 1), (uint8_t*)out_fp8, scale,
                                                                    (const __nv_bfloat16*)in, (int)dim);
    return rv_launched("quantize_fp8_per_token");
}

// ---------------------------------------------------------------- stage 2c
int rvllm_fused_act_mul_fp8_quant_validate(uint32_t num_tokens, uint32_t intermediate) {
    if (intermediate == 0 || intermediate % 8 != 0)
        return rv_fail(RVLLM_E_INVALID, "intermediate must be a positive multiple of 8");
    if (num_tokens == 0) return rv_fail(RVLLM_E_INVALID, "num_tokens must be > 0");
    return RVLLM_OK;
}

int rvllm_fused_act_mul_fp8_quant_launch(uint32_t num_tokens, uint32_t intermediate, int act, void* out_fp8,
                                         float* scale, const void* gate_up, int dtype, void* stream) {
    int rc = rvllm_fused_act_mul_fp8_quant_validate(num_tokens, intermediate);
    if (rc) return rc;
    if (!out_fp8 || !scale || !gate_up) return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (!rv_aligned(gate_up, 16) || !rv_aligned(out_fp8, 8)) return rv_fail(RVLLM_E_INVALID, "gate_up / out misaligned");
    if (act != RVLLM_ACT_SILU && act != RVLLM_ACT_GELU_TANH) return rv_fail(RVLLM_E_INVALID, "unknown activation");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    uint32_t b = rv_umin(intermediate, 1024);
    b = rv_umax(32, b - b % 32);
    dim3 grid(num_tokens), block(b);
    cudaStream_t s = (cudaStream_t)stream;
    uint8_t* o = (uint8_t*)out_fp8;
    int I = (int)intermediate;
    // Few long rows (a decode batch): spread each row over a cluster of CTAs.  Same bytes and scales.
    // The kernel is one latency chain per CTA (load, meet the cluster, store), so what matters is that all
    // CTAs are resident at once: about 512 CTAs at 4 per SM, however many rows share them.  From about
    // 100 rows on, one CTA of 1024 threads per row (one wave up to 148 rows) is as fast or faster.
    const uint32_t cl = num_tokens <= 64 ? 8u : (num_tokens <= 96 ? 4u : 1u);
    if (cl > 1 && intermediate >= 4096) {
        dim3 cgrid(cl, num_tokens), cblock(rvact::CLUSTER_THREADS), cdim(cl, 1, 1);
        const bool roomy = cl * num_tokens <= 3u * 128u;  // resident at 3 CTAs per SM: keep the wider register cache
#define RV_ACT_CLUSTER(ACT, T)                                                                                         \
    do {                                                                                                               \
        if (roomy)                                                                                                     \
            rv_launch(rvact::act_mul_quant_cluster_kernel<ACT, T, 4, 3>, cgrid, cblock, 0, s, cdim, o, scale,          \
                      (const T*)gate_up, I);                                                                           \
        else                                                                                                           \
            rv_launch(rvact::act_mul_quant_cluster_kernel<ACT, T, 3, 4>, cgrid, cblock, 0, s, cdim, o, scale,          \
                      (const T*)gate_up, I);                                                                           \
    } while (0)
        if (act == RVLLM_ACT_SILU && dtype == RVLLM_F16) RV_ACT_CLUSTER(rvact::ACT_SILU, __half);
        else if (act == RVLLM_ACT_SILU) RV_ACT_CLUSTER(rvact::ACT_SILU, __nv_bfloat16);
        else if (dtype == RVLLM_F16) RV_ACT_CLUSTER(rvact::ACT_GELU, __half);
        else RV_ACT_CLUSTER(rvact::ACT_GELU, __nv_bfloat16);
#undef RV_ACT_CLUSTER
        return rv_launched("fused_act_mul_fp8_quant (cluster)");
    }
    if (act == RVLLM_ACT_SILU && dtype == RVLLM_F16)
        rv_launch(fused_silu_mul_fp8_quant_kernel, dim3(grid), dim3(block), 128, s, dim3(1, 1, 1), o, scale, (const __half*)gate_up, I);
    else if (act == RVLLM_ACT_SILU)
        rv_launch(fused_silu_mul_fp8_quant_bf16_kernel, dim3(grid), dim3(block), 128, s, dim3(1, 1, 1), o, scale, (const __nv_bfloat16*)gate_up, I);
    else if (dtype == RVLLM_F16)
        rv_launch(fused_gelu_mul_fp8_quant_kernel, dim3(grid), dim3(block), 128, s, dim3(1, 1, 1), o, scale, (const __half*)gate_up, I);
    else
        rv_launch(fused_gelu_mul_fp8_quant_bf16_kernel, dim3(grid), dim3(block), 128, s, dim3(1, 1, 1), o, scale, (const __nv_bfloat16*)gate_up, I);
    return rv_launched("fused_act_mul_fp8_quant");
}

// ---------------------------------------------------------------- stage 4
int rvllm_argmax_validate(uint32_t num_tokens, uint32_t vocab) {
    if (vocab == 0) return rv_fail(RVLLM_E_INVALID, "vocab must be > 0");
    if (vocab > (uint32_t)INT_MAX) return rv_fail(RVLLM_E_INVALID, "vocab too large");
    if (num_tokens == 0) return rv_fail(RVLLM_E_INVALID, "num_tokens must be > 0");
    return RVLLM_OK;
}

int rvllm_argmax_launch(uint32_t num_tokens, uint32_t vocab, const float* logits, int32_t* out, int use_grid,
                        void* stream) {
    int rc = rvllm_argmax_validate(num_tokens, vocab);
    if (rc) return rc;
    if (!logits || !out) return rv_fail(RVLLM_E_INVALID, "null device pointer");
    cudaStream_t s = (cudaStream_t)stream;
    if (use_grid) {
        if (cudaMemsetAsync(out, 0, sizeof(int32_t) * (size_t)num_tokens, s) != cudaSuccess)
            return rv_fail(RVLLM_E_LAUNCH, "cudaMemsetAsync(out) failed");
        dim3 grid((vocab + 1023) / 1024, num_tokens), block(256);
        rv_launch(argmax_grid_f32_kernel, dim3(grid), dim3(block), 0, s, dim3(1, 1, 1), logits, out, (int)vocab);
    } else if (vocab >= 32768 && num_tokens <= 192) {
        // few long rows: eight CTAs per row (same winner, see greedy_argmax_cluster.cuh); 1024 threads while
        // two such CTAs per SM hold the whole grid, 512 beyond (four per SM)
        dim3 cgrid(8, num_tokens), cblock(num_tokens <= 32 ? rvargmax::ARGMAX_CLUSTER_THREADS : 512), cdim(8, 1, 1);
        rv_launch(rvargmax::argmax_cluster_f32_kernel, cgrid, cblock, 0, s, cdim, logits, out, (int)vocab);
    } else {
        uint32_t b = 1;
        while (b * 2 <= rv_umin(vocab, 1024)) b *= 2;  // min(vocab, 1024) rounded down to a power of two
        rv_launch(argmax_kernel, dim3(dim3(num_tokens)), dim3(dim3(b)), 0, s, dim3(1, 1, 1), logits, out, (int)vocab);
    }
    return rv_launched("argmax");
}

// ---------------------------------------------------------------- neighbours
int rvllm_rope_fp8kv_launch(const void* q_in, const void* k_in, const void* v_in, int in_stride, void* q_fp8,
                            void* k_cache, void* v_cache, float* k_scale_cache, float* v_scale_cache,
                            float* q_scale_cache, const void* cos_table, const void* sin_table,
                            const int32_t* positions, const int32_t* slot_mapping, int num_tokens, int num_heads,
                            int num_kv_heads, int head_dim, int rotary_dim, int max_positions,
                            int num_cache_slots, int dtype, void* stream) {
    if (num_tokens <= 0 || num_heads <= 0 || num_kv_heads <= 0) return rv_fail(RVLLM_E_INVALID, "bad token/head counts");
    if (head_dim < 64 || head_dim % 64 != 0 || head_dim > 512) return rv_fail(RVLLM_E_INVALID, "head_dim must be 64..512, multiple of 64");
    if (rotary_dim < 0 || rotary_dim > head_dim || rotary_dim % 2 != 0) return rv_fail(RVLLM_E_INVALID, "bad rotary_dim");
    if (max_positions <= 0 || num_cache_slots <= 0 || in_stride <= 0) return rv_fail(RVLLM_E_INVALID, "bad sizes");
    if (!q_in || !k_in || !v_in || !q_fp8 || !k_cache || !v_cache || !k_scale_cache || !v_scale_cache ||
        !q_scale_cache || !positions || !slot_mapping || (rotary_dim > 0 && (!cos_table || !sin_table)))
        return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    dim3 grid(num_tokens, num_heads > num_kv_heads ? num_heads : num_kv_heads), block(head_dim / 2);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RVLLM_F16)
        rv_launch(rvllm_rope_fp8kv_kernel, dim3(grid), dim3(block), 0, s, dim3(1, 1, 1), 
            (const __half*)q_in, (const __half*)k_in, (const __half*)v_in, in_stride, (uint8_t*)q_fp8,
            (uint8_t*)k_cache, (uint8_t*)v_cache, k_scale_cache, v_scale_cache, q_scale_cache,
            (const __half*)cos_table, (const __half*)sin_table, positions, slot_mapping, num_tokens, num_heads,
            num_kv_heads, head_dim, rotary_dim, max_positions, num_cache_slots);
    else
        rv_launch(rvllm_rope_fp8kv_bf16_kernel, dim3(grid), dim3(block), 0, s, dim3(1, 1, 1), 
            (const __nv_bfloat16*)q_in, (const __nv_bfloat16*)k_in, (const __nv_bfloat16*)v_in, in_stride,
            (uint8_t*)q_fp8, (uint8_t*)k_cache, (uint8_t*)v_cache, k_scale_cache, v_scale_cache, q_scale_cache,
            (const __nv_bfloat16*)cos_table, (const __nv_bfloat16*)sin_table, positions, slot_mapping, num_tokens,
            num_heads, num_kv_heads, head_dim, rotary_dim, max_positions, num_cache_slots);
    return rv_launched("rope_fp8kv");
}

// ---------------------------------------------------------------- Gemma-4 decorations, greedy tail
static inline uint32_t block_for(uint32_t width) { return round_block(rv_umin(width, 1024)); }

int rvllm_fused_qkv_rmsnorm_launch(const void* q_in, const void* k_in, const void* v_in, void* q_out, void* k_out,
                                   void* v_out, const void* q_gamma, const void* k_gamma, int num_tokens, int num_heads,
                                   int num_kv_heads, int head_dim, float eps, int src_row_stride, int dtype,
                                   void* stream) {
    if (num_tokens <= 0 || num_heads <= 0 || num_kv_heads < 0 || head_dim <= 0)
        return rv_fail(RVLLM_E_INVALID, "bad token / head counts");
    if (!isfinite(eps) || eps <= 0.0f) return rv_fail(RVLLM_E_INVALID, "eps must be finite and > 0");
    if ((long long)src_row_stride < ((long long)num_heads + 2LL * num_kv_heads) * head_dim)
        return rv_fail(RVLLM_E_INVALID, "src_row_stride is shorter than one packed QKV row");
    if (!q_in || !q_out || !q_gamma || (num_kv_heads > 0 && (!k_in || !v_in || !k_out || !v_out || !k_gamma)))
        return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (q_in == q_out || (num_kv_heads > 0 && (k_in == k_out || v_in == v_out)))
        return rv_fail(RVLLM_E_INVALID, "in-place QKV norm is not supported (outputs are compact, inputs packed)");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    dim3 grid(num_tokens, num_heads + 2 * num_kv_heads), block(block_for((uint32_t)head_dim));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RVLLM_F16)
        rv_launch(fused_qkv_rmsnorm_kernel, grid, block, 0, s, dim3(1, 1, 1), (const __half*)q_in, (const __half*)k_in,
                  (const __half*)v_in, (__half*)q_out, (__half*)k_out, (__half*)v_out, (const __half*)q_gamma,
                  (const __half*)k_gamma, num_tokens, num_heads, num_kv_heads, head_dim, eps, src_row_stride);
    else
        rv_launch(fused_qkv_rmsnorm_bf16_kernel, grid, block, 0, s, dim3(1, 1, 1), (const __nv_bfloat16*)q_in,
                  (const __nv_bfloat16*)k_in, (const __nv_bfloat16*)v_in, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out,
                  (__nv_bfloat16*)v_out, (const __nv_bfloat16*)q_gamma, (const __nv_bfloat16*)k_gamma, num_tokens,
                  num_heads, num_kv_heads, head_dim, eps, src_row_stride);
    return rv_launched("fused_qkv_rmsnorm");
}

int rvllm_fused_norm_add_residual_launch(const void* gemm_out, int gemm_out_is_f32, const float* channelscale,
                                         const void* gamma, void* residual, const void* layer_scalar, int num_tokens,
                                         int hidden, float eps, int dtype, void* stream) {
    if (num_tokens <= 0 || hidden <= 0) return rv_fail(RVLLM_E_INVALID, "num_tokens and hidden must be > 0");
    if (!isfinite(eps) || eps <= 0.0f) return rv_fail(RVLLM_E_INVALID, "eps must be finite and > 0");
    if (!gemm_out || !gamma || !residual || (gemm_out_is_f32 && !channelscale))
        return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    dim3 grid(num_tokens), block(block_for((uint32_t)hidden));
    cudaStream_t s = (cudaStream_t)stream;
    if (gemm_out_is_f32) {
        if (dtype == RVLLM_F16)
            rv_launch(fused_norm_add_residual_f16_kernel, grid, block, 0, s, dim3(1, 1, 1), (const float*)gemm_out,
                      channelscale, (const __half*)gamma, (__half*)residual, (const __half*)layer_scalar, hidden, eps);
        else
            rv_launch(fused_norm_add_residual_f16_bf16_kernel, grid, block, 0, s, dim3(1, 1, 1), (const float*)gemm_out,
                      channelscale, (const __nv_bfloat16*)gamma, (__nv_bfloat16*)residual,
                      (const __nv_bfloat16*)layer_scalar, hidden, eps);
    } else {
        if (dtype == RVLLM_F16)
            rv_launch(fused_norm_add_residual_f16in_kernel, grid, block, 0, s, dim3(1, 1, 1), (const __half*)gemm_out,
                      (const __half*)gamma, (__half*)residual, (const __half*)layer_scalar, hidden, eps);
        else
            rv_launch(fused_norm_add_residual_f16in_bf16_kernel, grid, block, 0, s, dim3(1, 1, 1),
                      (const __nv_bfloat16*)gemm_out, (const __nv_bfloat16*)gamma, (__nv_bfloat16*)residual,
                      (const __nv_bfloat16*)layer_scalar, hidden, eps);
    }
    return rv_launched("fused_norm_add_residual");
}

int rvllm_residual_scale_launch(void* residual, const void* scalar, int num_tokens, int hidden, int dtype, void* stream) {
    if (num_tokens <= 0 || hidden <= 0) return rv_fail(RVLLM_E_INVALID, "num_tokens and hidden must be > 0");
    if (!residual || !scalar) return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    dim3 grid(num_tokens), block(block_for((uint32_t)hidden));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RVLLM_F16)
        rv_launch(residual_scale_f16_kernel, grid, block, 0, s, dim3(1, 1, 1), (__half*)residual, (const __half*)scalar, hidden);
    else
        rv_launch(residual_scale_f16_bf16_kernel, grid, block, 0, s, dim3(1, 1, 1), (__nv_bfloat16*)residual,
                  (const __nv_bfloat16*)scalar, hidden);
    return rv_launched("residual_scale");
}

int rvllm_logit_softcap_launch(void* logits, int num_tokens, int vocab, float cap, int dtype, void* stream) {
    if (num_tokens <= 0 || vocab <= 0) return rv_fail(RVLLM_E_INVALID, "zero dim");          // gemma4_launcher.rs:960-963
    if (!isfinite(cap) || cap <= 0.0f) return rv_fail(RVLLM_E_INVALID, "cap must be > 0");   // :964-966
    if (!logits) return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16 && dtype != RVLLM_OUT_F32)
        return rv_fail(RVLLM_E_INVALID, "dtype must be f16, bf16 or f32");
    dim3 grid(num_tokens), block(block_for((uint32_t)vocab));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RVLLM_OUT_F32)
        rv_launch(logit_softcap_f32_kernel, grid, block, 0, s, dim3(1, 1, 1), (float*)logits, vocab, cap);
    else if (dtype == RVLLM_F16)
        rv_launch(logit_softcap_kernel, grid, block, 0, s, dim3(1, 1, 1), (__half*)logits, vocab, cap);
    else
        rv_launch(logit_softcap_bf16_kernel, grid, block, 0, s, dim3(1, 1, 1), (__nv_bfloat16*)logits, vocab, cap);
    return rv_launched("logit_softcap");
}

int rvllm_rope_cache_fp8kv_launch(const void* q_in, const void* k_in, const void* v_in, int in_stride, void* q_fp8,
                                  void* k_cache, void* v_cache, const void* cos_table, const void* sin_table,
                                  const int32_t* positions, const int32_t* slot_mapping, const float* q_scale_ptr,
                                  const float* kv_scale_ptr, int num_tokens, int num_heads, int num_kv_heads, int head_dim,
                                  int max_positions, int num_cache_slots, int dtype, void* stream) {
    if (num_tokens <= 0 || num_heads <= 0 || num_kv_heads < 0) return rv_fail(RVLLM_E_INVALID, "bad token / head counts");
    if (head_dim != 128 && head_dim != 256 && head_dim != 512)                                  // launcher.rs:598-603
        return rv_fail(RVLLM_E_INVALID, "head_dim must be 128, 256 or 512");
    if (num_kv_heads > 0 && num_heads % num_kv_heads != 0)
        return rv_fail(RVLLM_E_INVALID, "num_heads must be a multiple of num_kv_heads");
    if (max_positions <= 0 || (num_kv_heads > 0 && num_cache_slots <= 0) || in_stride <= 0) return rv_fail(RVLLM_E_INVALID, "bad sizes");
    if (!q_in || !q_fp8 || !cos_table || !sin_table || !positions || !q_scale_ptr ||
        (num_kv_heads > 0 && (!k_in || !v_in || !k_cache || !v_cache || !slot_mapping || !kv_scale_ptr)))
        return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (!rv_aligned(q_in, 4) || (num_kv_heads > 0 && (!rv_aligned(k_in, 4) || !rv_aligned(v_in, 4))) || (in_stride & 1))
        return rv_fail(RVLLM_E_INVALID, "q / k / v rows must be 4-byte aligned");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    dim3 grid(num_tokens, num_heads > num_kv_heads ? num_heads : num_kv_heads), block(rv_umax(head_dim / 2, 32));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RVLLM_F16)
        rv_launch(rvllm_rope_cache_fp8kv_strided_kernel, grid, block, 0, s, dim3(1, 1, 1), (const __half*)q_in,
                  (const __half*)k_in, (const __half*)v_in, in_stride, (uint8_t*)q_fp8, (uint8_t*)k_cache,
                  (uint8_t*)v_cache, (const __half*)cos_table, (const __half*)sin_table, positions, slot_mapping,
                  q_scale_ptr, kv_scale_ptr, num_tokens, num_heads, num_kv_heads, head_dim, max_positions, num_cache_slots);
    else
        rv_launch(rvllm_rope_cache_fp8kv_strided_bf16_kernel, grid, block, 0, s, dim3(1, 1, 1), (const __nv_bfloat16*)q_in,
                  (const __nv_bfloat16*)k_in, (const __nv_bfloat16*)v_in, in_stride, (uint8_t*)q_fp8, (uint8_t*)k_cache,
                  (uint8_t*)v_cache, (const __nv_bfloat16*)cos_table, (const __nv_bfloat16*)sin_table, positions,
                  slot_mapping, q_scale_ptr, kv_scale_ptr, num_tokens, num_heads, num_kv_heads, head_dim, max_positions,
                  num_cache_slots);
    return rv_launched("rope_cache_fp8kv");
}

int rvllm_fp8_gemv_blockscale_launch(void* out, const void* w_fp8, const float* block_scale, const void* x16, int M, int N,
                                     int K, int dtype, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return rv_fail(RVLLM_E_INVALID, "M, N, K must be > 0");
    if (!out || !w_fp8 || !block_scale || !x16) return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (K % 8 != 0 || !rv_aligned(w_fp8, 8) || !rv_aligned(x16, 8))
        return rv_fail(RVLLM_E_INVALID, "K must be a multiple of 8 and W / x 8-byte aligned");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    dim3 grid((N + 7) / 8, M), block(256);
    const int ncb = (K + 127) / 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RVLLM_F16)
        rv_launch(fp8_gemv_blockwise_wpr_native_f16in_kernel, grid, block, 0, s, dim3(1, 1, 1), (__half*)out,
                  (const unsigned char*)w_fp8, block_scale, (const __half*)x16, M, N, K, ncb);
    else
        rv_launch(fp8_gemv_blockwise_wpr_native_bf16in_kernel, grid, block, 0, s, dim3(1, 1, 1), (__nv_bfloat16*)out,
                  (const unsigned char*)w_fp8, block_scale, (const __nv_bfloat16*)x16, M, N, K, ncb);
    return rv_launched("fp8_gemv_blockscale");
}

int rvllm_embedding_gather_launch(void* out, const void* table, const int32_t* token_ids, int num_tokens,
                                  int hidden, int vocab, void* stream) {
    if (num_tokens <= 0 || hidden <= 0 || vocab <= 0) return rv_fail(RVLLM_E_INVALID, "bad embedding shapes");
    if (!out || !table || !token_ids) return rv_fail(RVLLM_E_INVALID, "null device pointer");
    int b = hidden / 8 < 256 ? (hidden / 8 < 32 ? 32 : ((hidden / 8 + 31) / 32) * 32) : 256;
    rv_launch(embedding_gather_f16_kernel, dim3(num_tokens), dim3(b), 0, (cudaStream_t)stream, dim3(1, 1, 1), (__half*)out, (const __half*)table,
                                                                           token_ids, hidden, vocab);
    return rv_launched("embedding_gather");
}

}  // extern "C"

namespace {
__global__ void e4m3_encode_kernel(uint8_t* out, const float* in, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = rv::f32_to_e4m3(in[i]);
}
__global__ void e4m3_decode_kernel(float* out, const uint8_t* in, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        // convert through the pair instruction with the byte in the low half
        float2 f = rv::e4m3x2_to_f32x2((uint32_t)in[i]);
        out[i] = f.x;
    }
}
}  // namespace

extern "C" {
int rvllm_e4m3_encode_f32(void* out_u8, const float* in, size_t n, void* stream) {
    if (!out_u8 || !in || n == 0) return rv_fail(RVLLM_E_INVALID, "bad encode arguments");
    e4m3_encode_kernel<<<296, 256, 0, (cudaStream_t)stream>>>((uint8_t*)out_u8, in, n);
    return rv_launched("e4m3_encode");
}
int rvllm_e4m3_decode_f32(float* out, const void* in_u8, size_t n, void* stream) {
    if (!out || !in_u8 || n == 0) return rv_fail(RVLLM_E_INVALID, "bad decode arguments");
    e4m3_decode_kernel<<<296, 256, 0, (cudaStream_t)stream>>>(out, (const uint8_t*)in_u8, n);
    return rv_launched("e4m3_decode");
}
}
