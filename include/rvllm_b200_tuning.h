/*
 * rvllm_b200 — tuning and diagnostic hooks.  NOT part of the drop-in ABI.
 *
 * The reference boundary allows no mutable process state behind the kernel entry points
 * (v3/crates/rvllm-cutlass/src/lib_so.rs:139-191 binds plain functions).  Everything in
 * rvllm_b200.h honours that: with the hooks below left alone, a launch depends on its arguments
 * only.  The hooks exist for sweeps and for tests that force one kernel form against another.
 * They set process-wide atomics: a launch running on another thread sees the old or the new value.
 * A workspace query and the launch it sizes must not straddle a change, and graphs record the
 * choice in force at capture time.  A production host never calls them.
 */
#ifndef RVLLM_B200_TUNING_H
#define RVLLM_B200_TUNING_H

#ifdef __cplusplus
extern "C" {
#endif

/* Programmatic dependent launch: when enabled (the default) every kernel is launched with the
 * programmatic-stream-serialization attribute, so the next kernel on the stream may start its
 * prologue and weight prefetch while the current one drains; every kernel waits for its
 * predecessor before touching dependent data.  Process-wide; set it before recording graphs. */
void rvllm_b200_set_pdl(int enabled);
int rvllm_b200_get_pdl(void);

/* Overrides of the tcgen05 kernel's automatic choices, for tuning runs: TMA ring depth
 * (2..8) and split-K factor (1..8); 0 restores the automatic choice.  Process-wide. */
void rvllm_fp8_gemm_tc_tune(int stages, int splits);
/* Form of the split-K reduction inside a cluster: 0 automatic (batch tiles up to 32 rows: partials are pushed into
 * the finishing CTA's receive buffer and every sender arrives on the owner's mbarrier; 64- and 128-row tiles: pushed
 * into the peers' idle rings between two cluster barriers; 256-row tiles: pulled out of the peers' rings), 1 always
 * pull, 2 the same as 0, 3 the small-tile push completed by one cluster barrier instead of the mbarrier arrivals
 * (1.3 us per layer slower in the decode graph; kept as a cross-check).  All forms sum in cluster-rank order, so their
 * results are bitwise equal (tested). */
void rvllm_fp8_gemm_tc_reduce(int mode);
/* CTAs a split-K launch aims for (splits = round(target / weight tiles), at most 8, at least 4 K blocks each);
 * 0 restores the built-in 360.  Process-wide. */
void rvllm_fp8_gemm_tc_split_target(int ctas);
/* Timing aid of the tcgen05 GEMM: while a device buffer of `slots` x 16 u64 is set, every launch takes the next row
 * (launch order, modulo `slots`; the count restarts with this call) and leaves, for each of 8 points, the
 * %globaltimer stamp of the earliest and of the latest CTA to pass it: 0 CTA runs, 1 the kernel ahead in the stream
 * is complete, 2 operands of the first K block in shared memory, 3 last MMA issued, 4 accumulator complete,
 * 5 split-K partials exchanged (push forms), 6 outputs stored.  Even entries must be preset to all ones (they take a
 * minimum), odd entries to 0.  A launch recorded into a CUDA graph keeps its row.  slots 0 or a null buffer: off.
 * The stamps exist only in a library built with RVLLM_TC_TRACE=1 (they cost the decode step 1.2 % even when off);
 * otherwise setting a buffer returns RVLLM_E_UNSUPPORTED. */
int rvllm_fp8_gemm_tc_trace(void* device_u64_buffer, int slots);
/* Split-K factor of one weight shape [N, K] (batch tiles up to 128 rows), four slots; splits 0 clears the slot. */
void rvllm_fp8_gemm_tc_split_for(int slot, int N, int K, int splits);

/* Overrides for tuning runs (0 restores the default): CTAs the grid aims for, the fewest tokens
 * worth a chunk of their own, and the main-kernel variant (1 = both products on the FP32 pipes,
 * 2 = scores on mma.sync FP8 tensor cores and P.V on the FP32 pipes, 3 = both products on mma.sync,
 * 4 = tcgen05 / TMEM / TMA; 0 picks 4 where the shape allows it, else 3, else 2).
 * Process-wide; the workspace query and the launch always use the same values. */
void rvllm_paged_decode_tune(int target_ctas, int min_chunk_tokens, int variant);
/* Split-KV on the tcgen05 kernel with a 16-bit output: 1 (default) = the chunks of a (sequence, KV head) form one
 * thread-block cluster (at most 8 chunks, each at least one 128-token tile) and the chunk-0 CTA merges the partials
 * out of its own shared memory — no workspace traffic, no combine launch; 0 = partials through the workspace and the
 * combine kernel, as the other variants do.  Process-wide. */
void rvllm_paged_decode_cluster_combine(int enabled);
/* Early metadata: the tcgen05 attention kernel reads context lengths and block tables, and fetches every K / V tile but
 * the last of a sequence, without waiting for the kernel before it in the stream (programmatic dependent launch); only
 * Q, the last tile and the scales wait.  Legal only for a caller whose context lengths, block tables and older cache
 * rows were complete before that kernel could start — the decode stack's graph qualifies: its bookkeeping for a step is
 * written by the last kernel of the step before, and consecutive graph launches do not overlap.
 * `rvllm_paged_decode_hint_early_meta()`: one-shot, calling thread only — the next decode-attention launch made from
 * this thread runs in that mode.  `rvllm_paged_decode_early_meta(mode)`: process-wide override, 0 = as hinted
 * (default), 1 = always, -1 = never.  Same bytes either way. */
void rvllm_paged_decode_hint_early_meta(void);
void rvllm_paged_decode_early_meta(int mode);
/* The cluster-merged form's own plan: CTAs aimed for (chunks per sequence = ceil(target / (batch * KV heads)), at most
 * 8) and the smallest chunk in tokens; 0 restores the defaults.  Process-wide. */
void rvllm_paged_decode_cluster_tune(int target_ctas, int min_chunk_tokens);
/* Depth of the tcgen05 kernel's K/V ring in 16 KB units (2..8 for head_dim 128, 3..8 for 256);
 * 0 restores the automatic choice.  Tuning aid, process-wide. */
void rvllm_paged_decode_ring(int units);

/* Timing aid: decode stacks created while a mask is set leave the marked launches out of every layer of their step
 * (1 attention-block RMSNorm, 2 QKV GEMM (+RoPE / KV write), 4 attention, 8 O projection, 16 MLP RMSNorm, 32 gate|up,
 * 64 act-mul-quant, 128 down projection).  The tokens such a stack emits mean nothing; step time with a launch left
 * out, against the full step, is what that launch costs inside the graph (its kernel time less whatever overlapped
 * with its neighbours).  0 = off, the default; process-wide. */
void rvllm_stack_debug_skip(int mask);

/* What the layer-block kernel's residency check sees on the current device: CTAs of the kernel one SM holds and the
 * number of SMs (their product must cover the grid of 8 * hidden / 128 CTAs), from the device's per-SM limits.  The
 * last argument is ignored.  Diagnostic. */
int rvllm_fp8_layer_block_capacity(int* ctas_per_sm, int* sms, int carveout_percent);

/* Stage timing of the layer-block kernel: while a device buffer of (8 * hidden / 128) x 16 u64 is set, every launch
 * writes %globaltimer stamps of its stage boundaries into it, one row per CTA (0 start, 1 predecessor done, 2/7/12
 * accumulator of the O / gate|up / down stage complete, 3-4, 5-6, 8-9, 10-11, 13-14 before / after the five grid
 * barriers, 15 end).  NULL switches it off (the default). */
void rvllm_fp8_layer_block_trace(void* device_u64_buffer);

/* Host-only self-test of the per-device "set up once" bookkeeping that guards cudaFuncSetAttribute
 * (the attribute belongs to a device, not to the process).  Touches no CUDA API; 0 = pass. */
int rvllm_b200_selftest_device_once(void);

#ifdef __cplusplus
}
#endif
#endif /* RVLLM_B200_TUNING_H */
