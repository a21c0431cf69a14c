/*
 * rvllm_b200 — C ABI of the B200 (sm_100a) FP8 decode hot path.
 *
 * Plain pointers and sizes only.  Every pointer named "device" is CUDA device memory
 * owned by the caller; the library never allocates or frees device memory on these
 * paths (the decode-stack object in section 7 is the one exception and says so).
 * `stream` is a cudaStream_t / CUstream passed as void*.  All launches are
 * asynchronous on that stream and safe to record into a CUDA graph.
 *
 * Return value: 0 on success; a negative RVLLM_E_* code otherwise.  After a failure
 * rvllm_b200_last_error() returns a thread-local, human-readable reason.  Functions that
 * carry a reference entry-point name (cutlass_*, fa_sm89_*) keep the reference's own
 * convention (0 ok, non-zero error).
 *
 * "Reference" below is solidsf-inc/rvLLM v0.3.0; each entry cites the reference
 * interface it replaces as file:line within that project.
 */
#ifndef RVLLM_B200_H
#define RVLLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RVLLM_OK 0
#define RVLLM_E_INVALID (-1)     /* argument failed validation; nothing was launched */
#define RVLLM_E_LAUNCH (-2)      /* CUDA refused the launch */
#define RVLLM_E_UNSUPPORTED (-3) /* shape outside what the kernels implement */
#define RVLLM_E_WORKSPACE (-4)   /* workspace missing, misaligned or too small */
#define RVLLM_E_ARTIFACT (-5)    /* manifest / artifact verification failed */
#define RVLLM_E_NO_DEVICE (-6)   /* no usable CUDA device / driver */

/* 16-bit activation types */
#define RVLLM_F16 0
#define RVLLM_BF16 1
/* GEMM output kinds */
#define RVLLM_OUT_F16 0
#define RVLLM_OUT_BF16 1
#define RVLLM_OUT_F32 2
/* MLP activations */
#define RVLLM_ACT_SILU 0
#define RVLLM_ACT_GELU_TANH 1

/* ---- 0. library ------------------------------------------------------------------- */
int rvllm_b200_abi_version(void);          /* = 1 */
const char* rvllm_b200_last_error(void);   /* thread-local; "" when no error */
const char* rvllm_b200_build_arch(void);   /* "sm_100a" */

/* ---- 1. fused RMSNorm + per-token FP8 quantisation ----------------------------------
 * Replaces FusedRmsnormFp8QuantLaunch / FusedAddRmsnormFp8QuantLaunch /
 * QuantizeFp8PerTokenLaunch (v3/crates/rvllm-fused/src/launcher.rs:96-274) and the kernels
 * they launch (kernels/fused_rmsnorm_fp8_quant.cu:52,108,166).  Same validation: hidden /
 * dim a multiple of 8, num_tokens > 0, dim <= 65536 for the plain quantiser; same launch
 * geometry (grid = tokens, block = min(hidden, 1024), quantiser block >= 256).
 * out_fp8 [T, H] u8, scale [T] f32, in / gamma / residual 16-bit of `dtype`. */
int rvllm_fused_rmsnorm_fp8_quant_validate(uint32_t num_tokens, uint32_t hidden, float eps);
int rvllm_fused_rmsnorm_fp8_quant_launch(uint32_t num_tokens, uint32_t hidden, float eps, void* out_fp8,
                                         float* scale, const void* in_hidden, const void* gamma, int dtype,
                                         void* stream);
int rvllm_fused_add_rmsnorm_fp8_quant_launch(uint32_t num_tokens, uint32_t hidden, float eps, void* out_fp8,
                                             float* scale, void* residual_out, const void* in_hidden,
                                             const void* residual_in, const void* gamma, int dtype,
                                             void* stream);
int rvllm_quantize_fp8_per_token_validate(uint32_t num_tokens, uint32_t dim);
int rvllm_quantize_fp8_per_token_launch(uint32_t num_tokens, uint32_t dim, void* out_fp8, float* scale,
                                        const void* in, int dtype, void* stream);

/* ---- 2. act(gate) * up + per-token FP8 quantisation ---------------------------------
 * Replaces FusedSiluMulFp8QuantLaunch (launcher.rs:280-323; kernels
 * kernels/fused_silu_fp8_quant.cu:42, v3/kernels/fused_gelu_mul_fp8_quant.cu:53).
 * gate_up [T, 2*I] 16-bit laid out [gate | up]; out_fp8 [T, I]; scale [T]. */
int rvllm_fused_act_mul_fp8_quant_validate(uint32_t num_tokens, uint32_t intermediate);
int rvllm_fused_act_mul_fp8_quant_launch(uint32_t num_tokens, uint32_t intermediate, int act, void* out_fp8,
                                         float* scale, const void* gate_up, int dtype, void* stream);

/* ---- 3. greedy argmax ---------------------------------------------------------------
 * Replaces ArgmaxLaunch (launcher.rs:329-399; kernels/argmax.cu:81,132).  logits [T, V]
 * f32, out [T] i32.  use_grid != 0 selects the multi-CTA-per-row variant, which first
 * clears `out` with an async memset exactly as the reference launcher does. */
int rvllm_argmax_validate(uint32_t num_tokens, uint32_t vocab);
int rvllm_argmax_launch(uint32_t num_tokens, uint32_t vocab, const float* logits, int32_t* out, int use_grid,
                        void* stream);

/* ---- 4. FP8 E4M3 GEMMs --------------------------------------------------------------
 * A [M, K] u8 row-major, per-token scale a_scale[M]; W [N, K] u8 row-major, per-output-
 * channel scale w_scale[N]; f32 accumulation; deterministic (no float atomics).
 *
 * cutlass_fp8_gemm_channelscale / _workspace: the reference's exported pair
 * (kernels/cutlass_fp8_gemm_channelscale.cu:98,163; loaded by
 * v3/crates/rvllm-cutlass/src/lib_so.rs:403-415): D_f16 = f16(row_scale[m] * (col_scale[n] * acc)).
 * cutlass_fp8_gemm_v0 / cutlass_fp8_gemm_residual_v0 (+ _workspace_size): scalar weight
 * scale `b_scale` (device pointer to one f32), optional f16 residual
 * (kernels/cutlass_fp8_gemm_residual.cu:252-287, lib_so.rs:1486-1500). */
int cutlass_fp8_gemm_channelscale(void* out_f16, const void* a_fp8, const void* b_fp8, const void* row_scale,
                                  const void* col_scale, int M, int N, int K, void* workspace,
                                  size_t workspace_size, void* stream);
size_t cutlass_fp8_gemm_channelscale_workspace(int M, int N, int K);
int cutlass_fp8_gemm_v0(void* out_f16, const void* a_fp8, const void* b_fp8, const void* a_scales,
                        const void* b_scale, int M, int N, int K, void* workspace, size_t workspace_size,
                        void* stream);
size_t cutlass_fp8_gemm_v0_workspace_size(int M, int N, int K);
int cutlass_fp8_gemm_residual_v0(void* out_f16, const void* a_fp8, const void* b_fp8, const void* a_scales,
                                 const void* b_scale, const void* residual_f16, int M, int N, int K,
                                 void* workspace, size_t workspace_size, void* stream);
size_t cutlass_fp8_gemm_residual_v0_workspace_size(int M, int N, int K);

/* New exports in the same style.  The reference has no single kernel that applies a
 * per-channel weight scale and a residual (kernels/cutlass_fp8_gemm_channelscale.cu:3 vs
 * kernels/cutlass_fp8_gemm_residual.cu:3); its executor composes them
 * (v3/crates/rvllm-runtime/src/layer_exec.rs:439-450,523-534).
 * out_kind: RVLLM_OUT_*; residual (may be NULL, may alias out) has the output's 16-bit type.
 * impl: 0 = pick by shape, 1 = weight-streaming mma.sync kernel, 2 = tcgen05/TMEM kernel. */
int rvllm_fp8_gemm_channelscale(void* out, int out_kind, const void* a_fp8, const void* w_fp8,
                                const float* a_scale, const float* w_scale, const void* residual, int M, int N,
                                int K, int impl, void* workspace, size_t workspace_size, void* stream);
size_t rvllm_fp8_gemm_workspace(int M, int N, int K);
/* Status word of the tcgen05 kernel's bounded waits: 0 = every wait completed; otherwise
 * (site << 16 | CTA) of the first wait that ran out.  Synchronous (copies from the device);
 * for tests and diagnosis, not for the decode loop.  reset != 0 clears it. */
int rvllm_fp8_gemm_tc_status(int* status, int reset);
/* QKV projection with RoPE, per-(token, head) Q quantisation and the paged FP8 K/V write (per-(slot,
 * kv_head) scales) done in the GEMM's epilogue: the result of rvllm_fp8_gemm_channelscale into a
 * [M, (heads + 2*kv_heads)*128] 16-bit buffer followed by rvllm_rope_fp8kv_launch with rotary_dim =
 * head_dim, bit for bit, without the buffer and without the second launch.  head_dim must be 128 (one
 * 128-row weight tile is one head) and M <= 128; returns RVLLM_E_UNSUPPORTED for shapes it does not
 * take (use the two calls).  dtype: the 16-bit type of the implied intermediate and of the tables. */
int rvllm_fp8_gemm_qkv_rope_fp8kv(const void* a_fp8, const void* w_fp8, const float* a_scale, const float* w_scale, int M,
                                  int K, int heads, int kv_heads, int head_dim, int dtype, void* q_fp8, float* q_scale,
                                  void* k_cache, void* v_cache, float* k_scale_cache, float* v_scale_cache,
                                  const void* cos_table, const void* sin_table, const int32_t* positions,
                                  const int32_t* slot_mapping, int max_positions, int num_cache_slots, void* stream);
/* out = residual + (quantise_per_token(a16) @ W^T) with the per-token quantiser folded into the GEMM:
 * a16 [M, K] 16-bit activations (the attention output), amax_partials [M, amax_parts] partial maxima
 * of |a16| per row (their maximum is the row's absmax; rvllm_paged_decode_fp8_amax leaves one per KV
 * head).  Same bytes as rvllm_quantize_fp8_per_token_launch followed by rvllm_fp8_gemm_channelscale
 * with a residual, without the FP8 copy of the activations and without the quantiser launch.  M <= 32;
 * RVLLM_E_UNSUPPORTED otherwise (use the two calls).  out may alias residual. */
int rvllm_fp8_gemm_residual_from16(void* out, int dtype, const void* a16, const float* amax_partials, int amax_parts,
                                   const void* w_fp8, const float* w_scale, const void* residual, int M, int N, int K,
                                   void* stream);

/* gate|up projection + act(gate)*up + per-token FP8 re-quantisation behind one call
 * (reference: GEMM at layer_exec.rs:484-494 followed by FusedSiluMulFp8QuantLaunch :509).
 * W [2*I, K] rows [gate(0..I) | up(I..2I)]; out_fp8 [M, I]; out_scale [M].
 * impl 0: one launch where the shape allows (M <= 32, K a multiple of 128 up to 6144, I a multiple of 64 up to
 * 4 * K, every CTA of the launch resident at once): the gate|up stage of the layer-block kernel — gate and up
 * rows of the same 64 columns form one 128-row tensor-core operand, the epilogue multiplies act(gate) by up on
 * chip, the grid meets once for the row maxima and quantises; the [M, 2*I] intermediate never reaches HBM
 * (preceded by a 256-byte memset of the barrier words at the front of the workspace).  Otherwise, and with
 * impl 1 (streaming GEMM) / 2 (tcgen05 GEMM), two launches: the GEMM writes its [M, 2*I] 16-bit result into the
 * workspace and the act-mul-quant row kernel reads it back.  impl 3: the single launch or RVLLM_E_UNSUPPORTED.
 * Same bytes and scales in every form.  Needs rvllm_fp8_gemm_gateup_workspace(M, I, K) bytes of workspace. */
int rvllm_fp8_gemm_gateup_act_quant(void* out_fp8, float* out_scale, const void* a_fp8, const void* w_fp8,
                                    const float* a_scale, const float* w_scale, int M, int I, int K, int act,
                                    int dtype, int impl, void* workspace, size_t workspace_size, void* stream);
size_t rvllm_fp8_gemm_gateup_workspace(int M, int I, int K);

/* The greedy tail in two launches and without materialised logits: LM-head GEMM whose epilogue keeps, per 128-channel
 * weight tile and batch row, only the best (logit, token id) — logit = a_scale[m] * (w_scale[n] * acc), the f32 value
 * rvllm_fp8_gemm_channelscale would have stored, soft-capped first as cap * tanh(logit / cap) when softcap > 0 — and a
 * merge over the tiles.  Ordering rule of the reference's argmax kernels (kernels/argmax.cu:16-25): greater value
 * wins, the lower token id on ties, NaN is never a candidate, a row without candidates gives -1.  Same token as
 * rvllm_fp8_gemm_channelscale (f32 out) -> [soft cap] -> rvllm_argmax_launch; the reference composes
 * cublaslt.fp8_gemm -> logit_softcap -> ArgmaxLaunch (v3/crates/rvllm-runtime/src/gemma4_bring_up.rs:2119-2161) and has
 * no fused counterpart.  A [M, K] FP8, W [vocab, K] FP8, out_tokens [M] i32.  The workspace
 * (rvllm_fp8_gemm_lm_head_argmax_workspace bytes, 256-byte aligned) holds the per-tile winners. */
size_t rvllm_fp8_gemm_lm_head_argmax_workspace(int M, int vocab);
int rvllm_fp8_gemm_lm_head_argmax(int32_t* out_tokens, const void* a_fp8, const void* w_fp8, const float* a_scale,
                                  const float* w_scale, int M, int vocab, int K, float softcap, void* workspace,
                                  size_t workspace_bytes, void* stream);

/* Everything between two attention calls of a decoder layer in ONE launch, for decode batches of at most 32
 * rows: O projection (+residual) -> RMSNorm + FP8 quant -> gate|up projection -> act(gate)*up + FP8 quant ->
 * down projection (+residual) -> RMSNorm + FP8 quant with the next layer's gain.  Reference: the six launches of
 * v3/crates/rvllm-runtime/src/layer_exec.rs:425-541 (quantize_fp8_per_token, cuBLASLt O GEMM + residual,
 * fused_rmsnorm_fp8_quant, gate|up GEMM, fused_silu_mul_fp8_quant, down GEMM + residual) and the
 * fused_rmsnorm_fp8_quant that opens the next layer (:205-222); there is no single reference entry point.  Every
 * stage is the arithmetic of this library's stand-alone calls (rvllm_fp8_gemm_residual_from16 or
 * rvllm_fp8_gemm_channelscale, rvllm_fused_rmsnorm_fp8_quant_launch, rvllm_fp8_gemm_channelscale,
 * rvllm_fused_act_mul_fp8_quant_launch), bit for bit; the CTAs stay resident across the stages and meet at
 * grid-wide barriers while their TMA producers already stream the next stage's weights.
 *
 * attention output: 16-bit [M, o_k] + attn_amax [M, amax_parts] (as left by rvllm_paged_decode_fp8_amax), or, with
 * attn_out16 NULL, FP8 rows attn_fp8 [M, o_k] + attn_scale [M].  residual [M, hidden] 16-bit is updated in place.
 * x_fp8 [M, hidden] / x_scale [M]: the RMSNorm output feeding gate|up; on return they hold the closing norm's
 * output (RMSNorm of the final residual with next_norm_gamma), the next layer's QKV input.  h_fp8 [M, ffn] /
 * h_scale [M]: act(gate)*up.  gateup_w [2*ffn, hidden] rows [gate | up]; o_w [hidden, o_k]; down_w [hidden, ffn].
 * stages: mask of RVLLM_BLOCK_* (all of them in production; a subset runs only those stages on the buffers given,
 * which is how each stage is tested against the stand-alone kernels).
 * workspace: rvllm_fp8_layer_block_workspace(hidden, ffn) bytes (a few MB: split-K partial tiles and partial row
 * maxima), 256-byte aligned.  Its first 256 bytes are the grid barrier's counters: they must be zero before the first launch (one cudaMemsetAsync at set-up) and every launch
 * leaves them zero; calls that share a workspace must not overlap on the GPU.
 * Returns RVLLM_E_UNSUPPORTED for shapes it does not take (M > 32, hidden not a multiple of 128 or above 6144,
 * ffn not a multiple of 64 or above 4 * hidden, or a device on which the grid cannot be resident at once):
 * issue the stand-alone calls then. */
#define RVLLM_BLOCK_O 1
#define RVLLM_BLOCK_NORM_MLP 2
#define RVLLM_BLOCK_GATEUP_ACT 4
#define RVLLM_BLOCK_DOWN 8
#define RVLLM_BLOCK_NORM_NEXT 16
#define RVLLM_BLOCK_ALL 31
size_t rvllm_fp8_layer_block_workspace(int hidden, int ffn);
int rvllm_fp8_layer_block(int M, int hidden, int ffn, int o_k, int act, int dtype, float eps, const void* attn_out16,
                          const float* attn_amax, int amax_parts, const void* attn_fp8, const float* attn_scale,
                          const void* o_w, const float* o_scale, void* residual, const void* mlp_norm_gamma,
                          const void* next_norm_gamma, void* x_fp8, float* x_scale, const void* gateup_w,
                          const float* gateup_scale, void* h_fp8, float* h_scale, const void* down_w,
                          const float* down_scale, void* workspace, size_t workspace_bytes, int stages, void* stream);

/* ---- 5. FP8-KV paged GQA decode attention -------------------------------------------
 * The fa_sm89_* family the reference loads from libfa_sm89_kernels.so
 * (v3/kernels/fp8_decode_v2.cu:939-1112; loader v3/crates/rvllm-attention/src/lib.rs:353-493).
 * Output f16 [batch, heads, head_dim]; head_dim in {128, 256, 512}. */
int rvllm_fa_sm89_abi_version(void);          /* 2 */
int fa_sm89_fp8_output_dtype(void);           /* 1 = f16 */
int fa_sm89_fp8_output_element_size(void);    /* 2 */
uint64_t fa_sm89_decode_workspace_size(int batch_size, int num_heads, int num_kv_heads, int head_dim);
int fa_sm89_paged_decode_fp8(void* q_fp8, void* k_cache_fp8, void* v_cache_fp8, void* output,
                             void* block_tables, void* context_lens, void* workspace, size_t workspace_bytes,
                             void* k_scale_cache, void* v_scale_cache, void* q_scale_cache, float* q_descale,
                             float* k_descale, float* v_descale, float scale, int batch_size, int num_heads,
                             int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                             int num_blocks_total, int window_size_left, void* stream);
/* Present because the reference loader requires the symbols; f16-KV decode and FP8 prefill
 * are outside this path and return -1. */
int fa_sm89_paged_decode(void* q, void* k_cache, void* v_cache, void* output, void* block_tables,
                         void* context_lens, void* workspace, size_t workspace_bytes, float scale,
                         int batch_size, int num_heads, int num_kv_heads, int head_dim, int block_size,
                         int max_blocks_per_seq, int num_blocks_total, int window_size_left, void* stream);
int fa_sm89_paged_prefill_fp8(void* q_fp8, void* k_cache_fp8, void* v_cache_fp8, void* output,
                              void* block_tables, void* context_lens, void* cu_seqlens_q, void* workspace,
                              size_t workspace_bytes, void* k_scale_cache, void* v_scale_cache,
                              void* q_scale_cache, float* q_descale, float* k_descale, float* v_descale,
                              float scale, int total_q, int max_seqlen_q, int batch_size, int num_heads,
                              int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                              int num_blocks_total, int window_size_left, void* stream);
/* Same kernel with the output type selectable and head_dim 64 allowed
 * (PagedDecodeParams, v3/crates/rvllm-attention/src/decode.rs:14-102). */
int rvllm_paged_decode_fp8_validate(int batch_size, int num_heads, int num_kv_heads, int head_dim,
                                    int block_size, int max_blocks_per_seq, int num_blocks_total,
                                    int window_size_left, float scale);
uint64_t rvllm_paged_decode_workspace_size(int batch_size, int num_heads, int num_kv_heads, int head_dim);
int rvllm_paged_decode_max_chunks(int batch_size, int num_kv_heads);
/* Variant 4 is the tcgen05 / TMA main kernel (head_dim 128 or 256, at most 8 query heads per KV
 * head, pages of 8..128 tokens that divide 128).  Its waits on mbarriers are bounded; this reads
 * (and optionally clears) the word that records the first wait that gave up: 0 = none. */
int rvllm_paged_decode_tc_status(int* status, int reset);
/* Which main kernel a launch of this shape runs (1 = both products on the FP32 pipes, 2 = scores on
 * mma.sync FP8 tensor cores and P.V on the FP32 pipes, 3 = both products on mma.sync, 4 = tcgen05 /
 * TMEM / TMA: 4 where the shape allows it, else 3, else 2); negative on bad arguments. */
int rvllm_paged_decode_kernel_for(int num_heads, int num_kv_heads, int head_dim, int block_size, int num_blocks_total);
int rvllm_paged_decode_fp8(const void* q_fp8, const void* k_cache_fp8, const void* v_cache_fp8, void* output,
                           int out_dtype, const int32_t* block_tables, const int32_t* context_lens,
                           void* workspace, size_t workspace_bytes, const float* k_scale_cache,
                           const float* v_scale_cache, const float* q_scale_cache, const float* q_descale,
                           const float* k_descale, const float* v_descale, float scale, int batch_size,
                           int num_heads, int num_kv_heads, int head_dim, int block_size,
                           int max_blocks_per_seq, int num_blocks_total, int window_size_left, void* stream);

/* Attention with its epilogue fused: the chunk partials are combined per token, rounded to the
 * 16-bit type `round_dtype` exactly as the plain call would store them, and quantised per token
 * over the whole [heads * head_dim] row — the bytes and scales equal those of
 * rvllm_paged_decode_fp8 followed by rvllm_quantize_fp8_per_token_launch
 * (v3/crates/rvllm-runtime/src/layer_exec.rs:326-362,425), with one launch and one 16-bit
 * round trip less.  out_fp8 [batch, heads*head_dim] u8, out_scale [batch] f32.  The workspace is
 * always needed: rvllm_paged_decode_quant_workspace_size bytes. */
uint64_t rvllm_paged_decode_quant_workspace_size(int batch_size, int num_heads, int num_kv_heads, int head_dim);
/* rvllm_paged_decode_fp8 that also leaves, per (sequence, kv_head), the maximum of |output as stored|
 * in amax_out [batch, num_kv_heads] (input of rvllm_fp8_gemm_residual_from16).  Only where the tcgen05
 * kernel runs with a single chunk per sequence; RVLLM_E_UNSUPPORTED otherwise. */
int rvllm_paged_decode_fp8_amax(const void* q_fp8, const void* k_cache_fp8, const void* v_cache_fp8, void* output,
                                int out_dtype, float* amax_out, const int32_t* block_tables, const int32_t* context_lens,
                                void* workspace, size_t workspace_bytes, const float* k_scale_cache,
                                const float* v_scale_cache, const float* q_scale_cache, const float* q_descale,
                                const float* k_descale, const float* v_descale, float scale, int batch_size,
                                int num_heads, int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                                int num_blocks_total, int window_size_left, void* stream);
int rvllm_paged_decode_fp8_quant(const void* q_fp8, const void* k_cache_fp8, const void* v_cache_fp8, void* out_fp8,
                                 float* out_scale, int round_dtype, const int32_t* block_tables,
                                 const int32_t* context_lens, void* workspace, size_t workspace_bytes,
                                 const float* k_scale_cache, const float* v_scale_cache, const float* q_scale_cache,
                                 const float* q_descale, const float* k_descale, const float* v_descale, float scale,
                                 int batch_size, int num_heads, int num_kv_heads, int head_dim, int block_size,
                                 int max_blocks_per_seq, int num_blocks_total, int window_size_left, void* stream);

/* Decode attention without a caller workspace.  No counterpart in the reference: its callers
 * always own an arena to cut a workspace from.  This entry point is for callers that cannot
 * allocate device memory at all — a runtime whose memory was split into fixed regions at start-up,
 * or a plug-in whose host does not let it call the CUDA allocator.  The split-KV partials go into
 * an 8 MiB scratch array compiled into the library (rvllm_paged_decode_static_scratch_bytes();
 * every GPU that loads the library holds it until the process exits).  Same arguments, results and
 * errors as rvllm_paged_decode_fp8 minus workspace / workspace_bytes; a launch whose partials need
 * more than the built-in scratch is refused with RVLLM_E_WORKSPACE and nothing is launched.  It
 * calls no allocating routine.  The first call on each device looks up the scratch's device
 * address (once, with that device current), so make that first call before any stream capture
 * begins; no call after that first one touches anything but the launch.  (cudaDeviceReset destroys the
 * context the address belongs to: a process that resets a device must not use this entry point on it
 * afterwards.)  All calls on a device share the one array and it keeps the last call's contents
 * (nothing in it needs clearing between calls): two calls whose kernels overlap on the GPU — on
 * different streams — race on it; keep them on one stream or order them with events. */
size_t rvllm_paged_decode_static_scratch_bytes(void);
int rvllm_paged_decode_fp8_static_scratch(const void* q_fp8, const void* k_cache_fp8, const void* v_cache_fp8,
                                          void* output, int out_dtype, const int32_t* block_tables,
                                          const int32_t* context_lens, const float* k_scale_cache,
                                          const float* v_scale_cache, const float* q_scale_cache,
                                          const float* q_descale, const float* k_descale, const float* v_descale,
                                          float scale, int batch_size, int num_heads, int num_kv_heads, int head_dim,
                                          int block_size, int max_blocks_per_seq, int num_blocks_total,
                                          int window_size_left, void* stream);

/* ---- 6. neighbours of the path ------------------------------------------------------
 * RoPE + Q quantisation + paged FP8 KV write with per-(slot, head) scales
 * (v3/kernels/fused_rope_partial_fp8kv.cu:54; launcher
 * v3/crates/rvllm-fused/src/gemma4_launcher.rs:248-400) with an explicit input row
 * stride, and the token embedding gather (kernels/embedding_gather_f16.cu). */
int rvllm_rope_fp8kv_launch(const void* q_in, const void* k_in, const void* v_in, int in_stride, void* q_fp8,
                            void* k_cache, void* v_cache, float* k_scale_cache, float* v_scale_cache,
                            float* q_scale_cache, const void* cos_table, const void* sin_table,
                            const int32_t* positions, const int32_t* slot_mapping, int num_tokens, int num_heads,
                            int num_kv_heads, int head_dim, int rotary_dim, int max_positions,
                            int num_cache_slots, int dtype, void* stream);
int rvllm_embedding_gather_launch(void* out, const void* table, const int32_t* token_ids, int num_tokens,
                                  int hidden, int vocab, void* stream);

/* Llama-form RoPE (interleaved pairs 2t, 2t+1 over the whole head) + FP8 Q + paged FP8 K/V write with the
 * static per-tensor scales *q_scale_ptr / *kv_scale_ptr: FusedRopeCacheFp8KvLaunch
 * (v3/crates/rvllm-fused/src/launcher.rs:577-712; kernel v3/kernels/fused_rope_cache_fp8kv.cu:20-101; call
 * site v3/crates/rvllm-runtime/src/layer_exec.rs:297).  Same validation (head_dim 128/256/512, heads a
 * multiple of kv_heads) and geometry (grid tokens x max(heads, kv_heads), block max(head_dim/2, 32)); the
 * inputs carry a row stride in elements so the packed QKV output is consumed in place.  A position outside
 * [0, max_positions) or a non-positive scale writes nothing; a slot outside [0, num_cache_slots) skips the
 * cache write, as in the reference kernel. */
int rvllm_rope_cache_fp8kv_launch(const void* q_in, const void* k_in, const void* v_in, int in_stride, void* q_fp8,
                                  void* k_cache, void* v_cache, const void* cos_table, const void* sin_table,
                                  const int32_t* positions, const int32_t* slot_mapping, const float* q_scale_ptr,
                                  const float* kv_scale_ptr, int num_tokens, int num_heads, int num_kv_heads, int head_dim,
                                  int max_positions, int num_cache_slots, int dtype, void* stream);

/* ---- 6b. Gemma-4 layer decorations and the greedy tail's soft cap --------------------------------
 * Per-head RMSNorm of the packed QKV projection output into compact Q / K / V buffers (learned gain on Q
 * and K, none on V): FusedQkvRmsnormLaunch (v3/crates/rvllm-fused/src/gemma4_launcher.rs:178-246; kernel
 * v3/kernels/fused_qkv_rmsnorm.cu:28-130; call site v3/crates/rvllm-runtime/src/gemma4_layer_exec.rs:754-789).
 * grid (tokens, heads + 2*kv_heads), block min(head_dim, 1024). */
int rvllm_fused_qkv_rmsnorm_launch(const void* q_in, const void* k_in, const void* v_in, void* q_out, void* k_out,
                                   void* v_out, const void* q_gamma, const void* k_gamma, int num_tokens, int num_heads,
                                   int num_kv_heads, int head_dim, float eps, int src_row_stride, int dtype,
                                   void* stream);
/* Post-norm folded into the residual update: residual = (residual + rmsnorm(x) * gamma) * layer_scalar, x
 * being the GEMM's f32 output times its per-channel scales (gemm_out_is_f32 != 0: FusedNormAddResidualF16Launch,
 * gemma4_launcher.rs:784-822, kernel v3/kernels/fused_norm_add_residual_f16.cu:8-58) or its 16-bit output
 * (gemm_out_is_f32 == 0, channelscale ignored: FusedNormAddResidualF16InLaunch :888-923, kernel :67-116).
 * layer_scalar may be NULL (= 1).  Call sites gemma4_layer_exec.rs:1200-1235.  grid tokens, block min(hidden, 1024). */
int rvllm_fused_norm_add_residual_launch(const void* gemm_out, int gemm_out_is_f32, const float* channelscale,
                                         const void* gamma, void* residual, const void* layer_scalar, int num_tokens,
                                         int hidden, float eps, int dtype, void* stream);
/* residual *= *scalar (ResidualScaleF16Launch, gemma4_launcher.rs:572-616; v3/kernels/residual_scale_f16.cu:13-27). */
int rvllm_residual_scale_launch(void* residual, const void* scalar, int num_tokens, int hidden, int dtype, void* stream);
/* logits = cap * tanh(logits / cap) in place (LogitSoftcapLaunch, gemma4_launcher.rs:953-996;
 * v3/kernels/logit_softcap.cu:12-31; call site v3/crates/rvllm-runtime/src/gemma4_bring_up.rs:2144-2151).  dtype
 * RVLLM_F16 / RVLLM_BF16 as the reference kernel (16-bit logits), or RVLLM_OUT_F32 for f32 logits. */
int rvllm_logit_softcap_launch(void* logits, int num_tokens, int vocab, float cap, int dtype, void* stream);

/* FP8 weights with 128 x 128 block scales (scale f32 [ceil(N/128), ceil(K/128)]) times 16-bit activations, 16-bit out:
 * the alternative weight-scale layout of the Gemma-4 executor.  Fp8GemvF16InLaunch (gemma4_launcher.rs:839-886; kernel
 * fp8_gemv_blockwise_wpr_native_f16in_kernel, kernels/fp8_gemv.cu:811-891): grid (ceil(N/8), M), block 256, one warp per
 * output row; M is a handful of rows (decode).  K a multiple of 8. */
int rvllm_fp8_gemv_blockscale_launch(void* out, const void* w_fp8, const float* block_scale, const void* x16, int M, int N,
                                     int K, int dtype, void* stream);

/* FP8 encode / decode of a flat array with the kernels' own convert instructions
 * (used by the bit-exactness tests; not on the decode path). */
int rvllm_e4m3_encode_f32(void* out_u8, const float* in, size_t n, void* stream);
int rvllm_e4m3_decode_f32(float* out, const void* in_u8, size_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RVLLM_B200_H */
