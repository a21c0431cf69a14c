/*
 * rvllm_b200 decode stack — the per-step chain of the hot path for a whole decoder stack,
 * recorded once into a CUDA graph and replayed per token.
 *
 * One step, per layer (the chain of v3/crates/rvllm-runtime/src/layer_exec.rs:163-541 of the
 * reference): RMSNorm+FP8 quant -> QKV GEMM -> RoPE + Q quant + paged FP8 KV write ->
 * split-KV decode attention -> per-token quant -> O GEMM (+residual, in place) ->
 * RMSNorm+FP8 quant -> gate|up GEMM -> act*up+quant -> down GEMM (+residual); then final
 * RMSNorm+quant -> LM-head GEMM (f32 logits) -> [soft cap] -> argmax -> token feedback and position /
 * slot bookkeeping on the device (what the reference does with three small host uploads
 * per step, v3/crates/rvllm-runtime/src/gemma4_serve.rs:884-901).  Sliding layers keep a
 * ring cache (page % table length) and attend the last `sliding_window` tokens.
 *
 * Weights are caller-owned device memory (pointers are only read).  The stack object owns
 * its scratch buffers and KV caches: rvllm_stack_create is the one place in this library
 * that allocates device memory, and it does so once, outside the step.
 */
#ifndef RVLLM_B200_STACK_H
#define RVLLM_B200_STACK_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rvllm_stack rvllm_stack;

typedef struct {
    int hidden, ffn, vocab, num_layers;
    int heads, kv_heads;
    int sliding_head_dim, global_head_dim;
    int sliding_window;  /* tokens attended by a sliding layer (>= 1) */
    int global_every;    /* layer i is global when (i + 1) % global_every == 0; 0 = all sliding, 1 = all global */
    int act;             /* RVLLM_ACT_* */
    int dtype;           /* RVLLM_F16 / RVLLM_BF16: residual stream and GEMM outputs */
    int batch;           /* sequences decoded per step */
    int block_size;      /* KV page size in tokens */
    int max_context;     /* capacity per sequence of a global layer's cache, in tokens */
    int max_steps;       /* capacity of the emitted-token history */
    int prompt_len;      /* tokens per sequence fed from the prompt buffer before feedback starts */
    int gemm_impl;       /* 0 auto, 1 streaming, 2 tcgen05 */
    float rms_eps;
    float rope_theta;
    uint64_t seed;       /* shuffles the physical block order of the block tables */
    int kv_pool_blocks;  /* 0: every sequence owns max_context tokens of every global layer's cache.  > 0: the
                            global layers share a pool of this many blocks per layer, dealt out per sequence by
                            need (a ragged batch: rvllm_stack_seed_contexts); sliding layers always keep their
                            fixed ring of sliding_window tokens per sequence */
    int fused_block;     /* 1: where the shape allows (batch <= 32), everything between two attention calls is one
                            launch (rvllm_fp8_layer_block); 0: always the stand-alone kernels.  Same bytes either way. */
    int fused_argmax;    /* 1: the LM head keeps per-tile argmax winners and a merge picks the token
                            (rvllm_fp8_gemm_lm_head_argmax; no f32 logits are written, debug read 1 is refused);
                            0: f32 logits, then argmax.  Same tokens either way. */
    float logit_softcap; /* > 0: logits pass through cap * tanh(x / cap) before the argmax; 0 = none */
} rvllm_stack_config;

typedef struct {
    const void* attn_norm_gamma; /* [hidden] 16-bit */
    const void* qkv_w;           /* [(heads + 2*kv_heads) * head_dim, hidden] fp8 */
    const float* qkv_scale;      /* per output channel */
    const void* o_w;             /* [hidden, heads * head_dim] fp8 */
    const float* o_scale;
    const void* mlp_norm_gamma;  /* [hidden] 16-bit */
    const void* gateup_w;        /* [2 * ffn, hidden] fp8, rows [gate | up] */
    const float* gateup_scale;
    const void* down_w;          /* [hidden, ffn] fp8 */
    const float* down_scale;
} rvllm_layer_weights;

typedef struct {
    const void* embedding;        /* [vocab, hidden] 16-bit */
    const void* final_norm_gamma; /* [hidden] 16-bit */
    const void* lm_head_w;        /* [vocab, hidden] fp8 */
    const float* lm_head_scale;   /* [vocab] */
} rvllm_head_weights;

/* Validates the configuration without touching a device (0 or RVLLM_E_INVALID). */
int rvllm_stack_config_validate(const rvllm_stack_config* cfg);
/* Device bytes rvllm_stack_create will allocate (scratch + KV caches + bookkeeping). */
uint64_t rvllm_stack_device_bytes(const rvllm_stack_config* cfg);

/* layers[num_layers]; all pointers must stay valid for the life of the stack.  The stack launches on a stream of
 * its own and does not wait for any other: the weights must be completely written (synchronise the stream that
 * produced them) before this call. */
int rvllm_stack_create(rvllm_stack** out, const rvllm_stack_config* cfg, const rvllm_layer_weights* layers,
                       const rvllm_head_weights* head);
void rvllm_stack_destroy(rvllm_stack* s);

/* Restart every sequence at position 0.  prompt_tokens: host [batch, prompt_len] int32. */
int rvllm_stack_reset(rvllm_stack* s, const int32_t* prompt_tokens);

/* Profiling aid: restart with every sequence already at position `context`, the caches filled
 * with constant bytes and scales instead of being produced by `context` decode steps.  The
 * kernels then do the work of a step at that context length without the prefill run. */
int rvllm_stack_seed_context(rvllm_stack* s, int context);
/* The same with one context length per sequence (host [batch] int32, each in [0, max_context)): a ragged
 * batch.  With kv_pool_blocks > 0 the pool is dealt out so that sequence b can reach position
 * contexts[b] + max_steps; RVLLM_E_INVALID if the pool is too small. */
int rvllm_stack_seed_contexts(rvllm_stack* s, const int32_t* contexts);

/* Enqueue `n` decode steps (graph replays) on the stack's stream; returns without waiting.
 * rvllm_stack_sync waits for them.  A run that would take any sequence past max_context is refused
 * with RVLLM_E_INVALID before anything is launched (so are the eager and the host-buffer forms); the
 * emitted-token history keeps the first max_steps steps after a reset and drops later ones. */
int rvllm_stack_run(rvllm_stack* s, int n);
int rvllm_stack_sync(rvllm_stack* s);
/* Same steps launched kernel by kernel without the graph (for debugging and as a check that
 * the graph reproduces the eager result). */
int rvllm_stack_run_eager(rvllm_stack* s, int n);

/* One step through host buffers: copies tokens_in (host [batch] int32; NULL = keep the
 * device-side feedback) to the device, replays one step, copies the batch's next tokens to
 * tokens_out (host [batch]) and waits.  This is the end-to-end call a serving loop makes. */
int rvllm_stack_step_host(rvllm_stack* s, const int32_t* tokens_in, int32_t* tokens_out);

/* Emitted-token history since the last reset: host out [count][batch] int32 starting at
 * step `first`.  Returns the number of steps copied or a negative error. */
int rvllm_stack_read_tokens(rvllm_stack* s, int first, int count, int32_t* out);
int rvllm_stack_steps_done(rvllm_stack* s);
/* Number of kernel launches recorded in one step's graph. */
int rvllm_stack_launches_per_step(const rvllm_stack* s);
/* Stream the stack launches on (cudaStream_t), e.g. to bracket replays with events. */
void* rvllm_stack_stream(rvllm_stack* s);
/* Copy a scratch buffer to the host for step-by-step parity checks.  what: 0 residual
 * [batch, hidden] 16-bit, 1 logits [batch, vocab] f32, 2 positions [batch] i32. */
int rvllm_stack_debug_read(rvllm_stack* s, int what, void* host_out, size_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* RVLLM_B200_STACK_H */
