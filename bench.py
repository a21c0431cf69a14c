#!/usr/bin/env python
"""Decode-throughput benchmark of the FP8 decode hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --gpus N --steps K ...  # the path on the host CPU (oracle port)

Workload (N = 1): the 31B-class decode shape — 62 layers (5 sliding : 1 global), hidden 5376,
ffn 21504, vocab 262144, 32 query / 16 KV heads, head_dim 128 (window 1024) / 256, random-init
FP8 E4M3 weights with per-output-channel scales, block_size 16, shuffled block tables — a
512-token random prompt is run through the decode path, then K greedy decode steps are timed
at batch 32 (contexts 512+).  One step = one token for every sequence of the batch through all
layers, the LM head and argmax.  N > 1 runs one independent replica per GPU (no collective on
the data path); the timed region is bracketed by a barrier and the max over ranks is taken.
Prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tok/s, Gemma-4-31B shape, batch 32"


def metric_name(batch):
    """The headline label at the headline batch; another --batch names itself."""
    return METRIC if batch == HEADLINE_BATCH else METRIC.replace("batch 32", "batch %d" % batch)
UNIT = "tok/s"
HEADLINE_BATCH = 32


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs, device copy)"
    return 6650.0, "fallback (earlier measurement on this pool)"


# ----------------------------------------------------------------------------- byte model
def layer_shapes(cfg, is_global):
    hd = cfg["global_head_dim"] if is_global else cfg["sliding_head_dim"]
    q_dim, kv_dim = cfg["heads"] * hd, cfg["kv_heads"] * hd
    H, F = cfg["hidden"], cfg["ffn"]
    return dict(hd=hd, q_dim=q_dim, kv_dim=kv_dim,
                gemms=[("qkv", q_dim + 2 * kv_dim, H, False), ("o", H, q_dim, True),
                       ("gateup", 2 * F, H, False), ("down", H, F, True)])


def gemm_bytes(M, N, K, residual, out_bytes=2):
    """Algorithmic bytes of one GEMM launch: weights + activations + output (+ residual read) + scales."""
    return N * K + M * K + out_bytes * M * N + (2 * M * N if residual else 0) + 4 * M + 4 * N


def step_bytes(cfg, B, ctx):
    """Algorithmic HBM bytes of one decode step at context length `ctx` (every sequence)."""
    H, F, V = cfg["hidden"], cfg["ffn"], cfg["vocab"]
    total = 0
    for l in range(cfg["num_layers"]):
        g = cfg["global_every"] != 0 and (l + 1) % cfg["global_every"] == 0
        s = layer_shapes(cfg, g)
        for _, N, K, res in s["gemms"]:
            total += gemm_bytes(B, N, K, res)
        total += 2 * (B * H * 2 + B * H + B * 4 + H * 2)                      # two norm+quant
        total += B * s["q_dim"] * 3 + B * 4                                     # attention-output quant
        total += B * 2 * F * 2 + B * F + B * 4                                  # act*up + quant
        ctx_eff = min(ctx, cfg["sliding_window"]) if not g else ctx
        total += B * ctx_eff * cfg["kv_heads"] * (2 * s["hd"] + 8)              # K/V rows + their scales
        total += B * cfg["heads"] * s["hd"] * 3 + B * cfg["heads"] * 4          # Q in, O out, Q scales
    total += gemm_bytes(B, V, H, False, out_bytes=4)                           # LM head, f32 logits
    total += B * V * 4 + B * 4                                                  # argmax
    return total


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc, self.first = index, [], None, 0

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def mark(self):
        """Samples from here on count: nvidia-smi was started earlier only so that its start-up
        time does not eat the timed region."""
        self.first = len(self.rows)

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.rows = self.rows[self.first:]
        sm = sorted(float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit())
        out = {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": None, "reasons": [], "samples": len(sm)}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) >= 7:
                try:
                    out["sm_max_mhz"] = float(r[1])
                except ValueError:
                    pass
                for n, v in zip(names, r[3:7]):
                    if v.lower().startswith("active") and n not in out["reasons"]:
                        out["reasons"].append(n)
        return out


# ----------------------------------------------------------------------------- CPU arm (oracle port)
def cpu_step_sample(cfg, B, ctx, seed=0, min_seconds=0.0):
    """Times the path on the host cores with the CPU oracle, on a bounded sample of one decode
    step: one sliding and one global layer's full chain (norm+quant, QKV, attention at context
    `ctx`, quant, O+residual, norm+quant, gate|up, act+quant, down+residual) at batch B, and the
    LM head + argmax on 1/16 of the vocabulary.  The sample is repeated (same buffers) until
    `min_seconds` of timed work have been done.  Returns (estimated seconds for a whole step,
    seconds actually spent, description).  Random bytes stand in for weights: timing does not
    depend on values."""
    import numpy as np
    import oracle as orc

    H, F, V = cfg["hidden"], cfg["ffn"], cfg["vocab"]
    dt = cfg["dtype"]
    key = (B, ctx, cfg["num_layers"], H, F, V, dt)
    if key in _SAMPLE_CACHE:  # the buffers of an earlier step of the same run: timing does not depend on values
        chains, n_sliding, n_global, vs = _SAMPLE_CACHE[key]
        return _run_sample(chains, n_sliding, n_global, V, vs, B, ctx, min_seconds)
    g = np.random.default_rng(seed)

    def rbytes(*shape):
        b = g.integers(0, 256, shape, dtype=np.uint8)
        b[(b & 0x7F) == 0x7F] ^= 1
        return b

    n_global = sum(1 for l in range(cfg["num_layers"]) if cfg["global_every"] and (l + 1) % cfg["global_every"] == 0)
    n_sliding = cfg["num_layers"] - n_global
    resid = orc.to_bits16(g.standard_normal((B, H)).astype(np.float32), dt)
    gamma = orc.to_bits16(np.ones(H, np.float32), dt)
    chains = {}
    for kind, is_global in (("sliding", False), ("global", True)):
        if (n_global if is_global else n_sliding) == 0:
            continue
        s = layer_shapes(cfg, is_global)
        hd, q_dim = s["hd"], s["q_dim"]
        w = {name: (rbytes(N, K), np.full(N, 1e-3, np.float32)) for name, N, K, _ in s["gemms"]}
        ctx_eff = ctx if is_global else min(ctx, cfg["sliding_window"])
        bs = cfg["block_size"]
        mb = (ctx_eff + bs - 1) // bs + 1
        nblk = B * mb
        kc, vc = rbytes(nblk * bs * cfg["kv_heads"], hd), rbytes(nblk * bs * cfg["kv_heads"], hd)
        ksc = np.full(nblk * bs * cfg["kv_heads"], 0.01, np.float32)
        tables = g.permutation(nblk).astype(np.int32).reshape(B, mb)
        ctxs = np.full(B, ctx_eff, np.int32)

        def chain(w=w, hd=hd, q_dim=q_dim, kc=kc, vc=vc, ksc=ksc, tables=tables, ctxs=ctxs, bs=bs, nblk=nblk):
            t0 = time.perf_counter()
            x8, xs = orc.rmsnorm_fp8_quant(resid, gamma, cfg["rms_eps"], dt)
            qkv = orc.fp8_gemm(x8, w["qkv"][0], xs, w["qkv"][1], out_kind=dt)
            q8, qs = orc.quantize_fp8_per_token(np.ascontiguousarray(qkv[:, :q_dim]).reshape(B * cfg["heads"], hd), dt)
            att = orc.paged_decode_fp8(q8.reshape(B, cfg["heads"], hd), kc, vc, tables, ctxs, hd ** -0.5, cfg["heads"],
                                       cfg["kv_heads"], hd, bs, k_scale_cache=ksc, v_scale_cache=ksc, q_scale_cache=qs,
                                       dtype=dt, num_blocks_total=nblk)
            a8, a_s = orc.quantize_fp8_per_token(att.reshape(B, q_dim), dt)
            r2 = orc.fp8_gemm(a8, w["o"][0], a_s, w["o"][1], residual=resid, out_kind=dt)
            x8, xs = orc.rmsnorm_fp8_quant(r2, gamma, cfg["rms_eps"], dt)
            gu = orc.fp8_gemm(x8, w["gateup"][0], xs, w["gateup"][1], out_kind=dt)
            h8, hs = orc.act_mul_fp8_quant(gu, cfg["act"], dt)
            orc.fp8_gemm(h8, w["down"][0], hs, w["down"][1], residual=r2, out_kind=dt)
            return time.perf_counter() - t0
        chains[kind] = chain
    vs = max(V // 16, 1)
    wl = rbytes(vs, H)
    x8h, xsh = orc.rmsnorm_fp8_quant(resid, gamma, cfg["rms_eps"], dt)

    def head():
        t0 = time.perf_counter()
        logits = orc.fp8_gemm(x8h, wl, xsh, np.full(vs, 1e-3, np.float32), out_kind=2)
        orc.argmax_f32(logits)
        return time.perf_counter() - t0
    chains["head"] = head
    _SAMPLE_CACHE[key] = (chains, n_sliding, n_global, vs)
    return _run_sample(chains, n_sliding, n_global, V, vs, B, ctx, min_seconds)


_SAMPLE_CACHE = {}


def _run_sample(chains, n_sliding, n_global, V, vs, B, ctx, min_seconds):
    spent = {k: 0.0 for k in chains}
    passes = 0
    while True:
        for k, fn in chains.items():
            spent[k] += fn()
        passes += 1
        if sum(spent.values()) >= min_seconds or passes >= 200:
            break
    mean = {k: v / passes for k, v in spent.items()}
    est = mean.get("sliding", 0.0) * n_sliding + mean.get("global", 0.0) * n_global + mean["head"] * (V / vs)
    desc = (f"{passes} passes over: 1 sliding + 1 global layer chain at batch {B}, context {ctx}, and LM head + argmax on "
            f"1/16 of the vocabulary; step time = {n_sliding} x sliding + {n_global} x global + 16 x head slice")
    return est, sum(spent.values()), desc


def run_reference_arm(args, cfg):
    """The path on the host CPU: the oracle's C restatement of the reference's arithmetic with
    every host thread (the reference has no CPU executor for GEMM / attention; its Rust per-op
    references cannot be built here)."""
    import oracle as orc

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    orc.build()
    orc.use_all_host_threads()  # a torchrun worker inherits OMP_NUM_THREADS=1
    B = args.batch
    times = []
    per_step = max(0.3, min(4.0, 150.0 / (args.warmup + args.steps)))  # the whole run stays within a few minutes
    for i in range(args.warmup + args.steps):
        est, spent, desc = cpu_step_sample(cfg, B, ctx=cfg["prompt_len"], seed=i, min_seconds=per_step)
        if i >= args.warmup:
            times.append(est)
    est = sum(times) / len(times)
    value = B / est
    line = {
        "impl": "reference", "metric": metric_name(args.batch), "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": est * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32", "data": "synthetic",
        "config": workload_config(cfg, B),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": orc.num_threads(), "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(cfg, B):
    return {"workload": "31B-class FP8 decode: 62 layers (5 sliding:1 global), hidden 5376, ffn 21504, vocab 262144, "
                        "32q/16kv heads, head_dim 128 (window 1024) / 256; 512-token random prompt then greedy decode",
            "batch_per_gpu": B, "prompt_len": cfg["prompt_len"], "block_size": cfg["block_size"],
            "layers": cfg["num_layers"], "parallelism": "independent replicas",
            "l2": "per-step weight stream (28 GB) is far larger than the 126 MB L2, no flush needed"}


# ----------------------------------------------------------------------------- GPU arm
def time_steps(torch, stack, n):
    """Device time of n graph replays, CUDA events on the stack's own stream."""
    ext = torch.cuda.ExternalStream(stack.stream())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(ext):
        e0.record()
        stack.run(n)
        e1.record()
    stack.sync()
    return e0.elapsed_time(e1) / 1e3


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the gate|up GEMM, from the ncu capture
# summarised in profiles/fp8_gemm_tc_gateup_m32.md, keyed by (N, K, M); other shapes were not captured
NCU_TRAFFIC_BYTES = {(43008, 5376, 32): 236.3e6}


def dominant_kernel_roofline(torch, cfg, weights, B, peak, peak_src):
    """The gate|up projection is the largest stream of a step (56 % of a layer's weight bytes).
    It is launched alone through the C ABI, cycling over the layers' different weight matrices
    (231 MB each, larger than L2, so every launch streams from HBM), and timed with CUDA events on
    the launching stream."""
    from rvllm_b200 import gemm
    H, F = cfg["hidden"], cfg["ffn"]
    tdt = torch.float16 if cfg["dtype"] == 0 else torch.bfloat16
    a = torch.randint(0, 120, (B, H), dtype=torch.uint8, device="cuda")
    a_s = torch.full((B,), 0.01, dtype=torch.float32, device="cuda")
    out = torch.empty((B, 2 * F), dtype=tdt, device="cuda")
    layers = weights.layers
    for i in range(8):
        gemm.fp8_gemm_channelscale(out, a, layers[i % len(layers)]["gateup_w"], a_s,
                                   layers[i % len(layers)]["gateup_scale"], impl=cfg["gemm_impl"])
    torch.cuda.synchronize()
    n = 4 * len(layers)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        lw = layers[i % len(layers)]
        gemm.fp8_gemm_channelscale(out, a, lw["gateup_w"], a_s, lw["gateup_scale"], impl=cfg["gemm_impl"])
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / 1e3 / n
    algo = gemm_bytes(B, 2 * F, H, False)
    achieved = algo / sec / 1e9
    return {"bound": "hbm", "kernel": "fp8 GEMM, gate|up shape [%d x %d] x M=%d" % (2 * F, H, B),
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
            "us_per_launch": sec * 1e6, "algorithmic_bytes_per_launch": algo,
            "traffic": NCU_TRAFFIC_BYTES.get((2 * F, H, B))}


def attention_case(torch, cfg, B, ctx, peak, peak_src):
    """The decode-attention kernel alone at the bench's two layer shapes (sliding: head_dim 128,
    window 1024; global: head_dim 256), batch B, context ctx, seeded random cache bytes and shuffled
    block tables, through the C ABI.  Cycles over enough cache copies to exceed L2; timed with CUDA
    events on the launching stream.  A small case for ncu, and a kernel-level roofline line."""
    from rvllm_b200.attention import PagedDecodeFp8Launcher, PagedDecodeParams
    H, KVH, bs = cfg["heads"], cfg["kv_heads"], cfg["block_size"]
    tdt = torch.float16 if cfg["dtype"] == 0 else torch.bfloat16
    gen = torch.Generator(device="cuda")
    gen.manual_seed(11)
    out = []
    for tag, HD, window in (("sliding", cfg["sliding_head_dim"], cfg["sliding_window"] - 1),
                            ("global", cfg["global_head_dim"], -1)):
        att = min(ctx, window + 1) if window >= 0 else ctx
        mb = (window + 1 + bs - 1) // bs + 1 if window >= 0 else (ctx + bs - 1) // bs + 1
        nblk = B * mb
        per_copy = 2 * B * att * KVH * HD
        copies = min(6, max(2, int(300e6 // per_copy) + 1))
        ks = [torch.randint(0, 120, (nblk, bs, KVH, HD), dtype=torch.uint8, device="cuda", generator=gen) for _ in range(copies)]
        vs = [torch.randint(0, 120, (nblk, bs, KVH, HD), dtype=torch.uint8, device="cuda", generator=gen) for _ in range(copies)]
        sc = torch.full((nblk * bs * KVH,), 0.01, dtype=torch.float32, device="cuda")
        q = torch.randint(0, 120, (B, H, HD), dtype=torch.uint8, device="cuda", generator=gen)
        qs = torch.full((B * H,), 0.01, dtype=torch.float32, device="cuda")
        tables = torch.randperm(nblk, device="cuda", generator=gen).to(torch.int32).reshape(B, mb).contiguous()
        ctxs = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        o = torch.empty((B, H, HD), dtype=tdt, device="cuda")
        p = PagedDecodeParams(B, H, KVH, HD, bs, mb, nblk, HD ** -0.5, window)
        ws = torch.empty(max(p.workspace_bytes(), 16), dtype=torch.uint8, device="cuda")
        la = PagedDecodeFp8Launcher(p)

        def launch(i):
            la.launch(q, ks[i % copies], vs[i % copies], o, tables, ctxs, workspace=ws, k_scale_cache=sc,
                      v_scale_cache=sc, q_scale_cache=qs)
        for i in range(4):
            launch(i)
        torch.cuda.synchronize()
        n = 8 * copies
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            launch(i)
        e1.record()
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) / 1e3 / n
        algo = B * att * KVH * (2 * HD + 8)  # K and V rows plus their two f32 scales, per attended token and KV head
        out.append({"kernel": "paged decode attention, %s layer shape (head_dim %d)" % (tag, HD), "batch": B, "context": ctx,
                    "attended": att, "bound": "hbm", "achieved": algo / sec / 1e9, "peak": peak, "unit": "GB/s",
                    "frac": algo / sec / 1e9 / peak, "peak_source": peak_src, "us_per_launch": sec * 1e6,
                    "algorithmic_bytes_per_launch": algo, "max_chunks": p.max_chunks()})
        del ks, vs
    return out


def run_batch(torch, cfg, weights, B, steps, warmup, e2e_steps, sampler=None, barrier=None, profiler_range=False, seeded=False):
    import numpy as np
    from rvllm_b200.stack import DecodeStack

    c = dict(cfg, batch=B)
    if sampler:
        sampler.start()   # started early (it needs a few hundred ms to produce its first line); counted from mark()
    stack = DecodeStack(c, weights)
    g = np.random.default_rng(3)
    prompt = g.integers(0, c["vocab"], (B, c["prompt_len"]), dtype=np.int32)
    if seeded:
        stack.seed_context(c["prompt_len"] - 1)   # profiling runs: skip the prefill steps
    else:
        stack.reset(prompt)
        stack.run(c["prompt_len"] - 1)   # prompt through the decode path; the next step emits token 1
    stack.run(max(warmup, 3))
    stack.sync()
    if barrier:
        barrier()
    if sampler:
        sampler.mark()
    if profiler_range:
        torch.cuda.profiler.start()
    sec = time_steps(torch, stack, steps)
    if profiler_range:
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    clocks = sampler.stop() if sampler else None
    if barrier:
        barrier()
    ctx_mid = c["prompt_len"] + max(warmup, 3) + steps // 2
    res = {"batch": B, "ms_per_step": sec / steps * 1e3, "tok_s": B * steps / sec, "seconds": sec,
           "launches_per_step": stack.launches_per_step(), "context_mid": ctx_mid,
           "step_bytes": step_bytes(c, B, ctx_mid), "clocks": clocks}
    # end to end: host token buffer in, host token buffer out, every step
    if e2e_steps > 0:
        tok_in = stack.tokens()[-1].copy()
        tok_out = np.zeros(B, np.int32)
        stack.step_host(tok_in, tok_out)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            tok_in, tok_out = tok_out, tok_in
            stack.step_host(tok_in, tok_out)
        dt = time.perf_counter() - t0
        res["e2e"] = {"value": B * e2e_steps / dt, "unit": UNIT, "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
                      "ms_per_step": dt / e2e_steps * 1e3, "steps": e2e_steps}
    res["greedy_tokens_tail"] = stack.tokens()[-1][:4].tolist()
    stack.close()
    return res


def run_gpu_arm(args, cfg):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA path has no CPU fallback")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        torch.cuda.synchronize()
        if dist:
            dist.barrier(device_ids=[local])

    from rvllm_b200 import build, _lib
    from rvllm_b200.stack import random_weights
    if not os.path.exists(_lib.LIB_PATH):
        build.build_all()
    peak, peak_src = measured_peaks()
    t0 = time.perf_counter()
    weights = random_weights(cfg, seed=3)
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t0

    B = args.batch
    main = run_batch(torch, cfg, weights, B, args.steps, args.warmup, args.e2e_steps, ClockSampler(local), barrier,
                     profiler_range=args.profiler_range, seeded=args.seeded_context)
    from rvllm_b200 import replicas
    sec = replicas.job_seconds(dist, main["seconds"], device="cuda")            # slowest replica
    e2e_ms_max = replicas.job_seconds(dist, main["e2e"]["ms_per_step"] if "e2e" in main else 0.0, device="cuda")
    value = world * B * args.steps / sec
    line = {
        "metric": metric_name(args.batch), "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3 x fp8_e4m3 -> f32 (bf16 activations)" if cfg["dtype"] == 1 else "fp8_e4m3 x fp8_e4m3 -> f32 (f16 activations)",
        "data": "synthetic", "config": workload_config(cfg, B),
        "gpu_launches": main["launches_per_step"] * args.steps, "clocks": main["clocks"],
        "weights_gb": weights.nbytes() / 1e9, "setup_s": setup_s,
    }
    if "e2e" in main:
        e = dict(main["e2e"])
        e["value"] = world * B / (e2e_ms_max / 1e3)
        e["ms_per_step"] = e2e_ms_max
        line["e2e"] = e
    step_frac = main["step_bytes"] / (main["seconds"] / args.steps) / 1e9 / peak
    line["step_roofline"] = {"algorithmic_bytes_per_step": main["step_bytes"], "context": main["context_mid"],
                             "achieved_gbs": main["step_bytes"] / (main["seconds"] / args.steps) / 1e9,
                             "frac_of_hbm_peak": step_frac}
    if rank == 0:
        if not args.no_roofline:
            line["roofline"] = dominant_kernel_roofline(torch, cfg, weights, B, peak, peak_src)
        if world == 1 and not args.no_cpu_baseline:
            import oracle as orc
            orc.build()
            orc.use_all_host_threads()
            est, spent, desc = cpu_step_sample(cfg, B, ctx=cfg["prompt_len"], min_seconds=12.0)
            line["cpu_baseline"] = {"value": B / est, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
                                    "sample": desc, "sample_seconds": spent}
        if world == 1 and args.all_batches:
            line["by_batch"] = {}
            for b in (1, 128):
                r = run_batch(torch, cfg, weights, b, args.steps, args.warmup, 0)
                line["by_batch"][str(b)] = {"tok_s": r["tok_s"], "ms_per_step": r["ms_per_step"],
                                            "frac_of_hbm_peak": r["step_bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / peak}
            line["by_batch"][str(B)] = {"tok_s": main["tok_s"], "ms_per_step": main["ms_per_step"],
                                        "frac_of_hbm_peak": step_frac}
        print(json.dumps(line))
    if dist:
        dist.barrier(device_ids=[local])
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=HEADLINE_BATCH)
    ap.add_argument("--e2e-steps", type=int, default=32)
    ap.add_argument("--layers", type=int, default=62, help="reduce only for quick functional checks")
    ap.add_argument("--gemm-impl", type=int, default=0)
    ap.add_argument("--all-batches", action="store_true", help="also time batch 1 and 128")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-roofline", action="store_true")
    ap.add_argument("--roofline-only", action="store_true",
                    help="small case for ncu: only the dominant kernel over 4 gate|up weight matrices (0.9 GB)")
    ap.add_argument("--attention-only", action="store_true",
                    help="small case for ncu: only the decode-attention kernel at the two layer shapes")
    ap.add_argument("--context", type=int, default=576, help="context length of --attention-only")
    ap.add_argument("--attention-variant", type=int, default=0,
                    help="decode-attention main kernel: 0 automatic, 1 FP32 pipes, 2/3 mma.sync, 4 tcgen05")
    ap.add_argument("--seeded-context", action="store_true",
                    help="profiling aid: fill the KV caches synthetically instead of running the 512 prefill steps")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed region with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    args = ap.parse_args()
    from rvllm_b200.stack import gemma31b_shape
    need = 512 + max(args.warmup, 3) + args.steps + args.e2e_steps + 8
    cfg = gemma31b_shape(args.batch, num_layers=args.layers, gemm_impl=args.gemm_impl,
                         max_context=(need + 255) // 256 * 256, max_steps=need)
    if args.roofline_only:
        import torch
        from rvllm_b200.stack import Weights, _quant_weight
        gen = torch.Generator(device="cuda")
        gen.manual_seed(3)
        w = Weights()
        for _ in range(4):
            gw, gs = _quant_weight(2 * cfg["ffn"], cfg["hidden"], gen, 0.02)
            w.layers.append({"gateup_w": gw, "gateup_scale": gs})
        peak, src = measured_peaks()
        print(json.dumps({"roofline": dominant_kernel_roofline(torch, cfg, w, args.batch, peak, src)}))
        return
    if args.impl != "reference" and args.attention_variant != 0:
        from rvllm_b200 import _lib
        _lib.lib().rvllm_paged_decode_tune(0, 0, args.attention_variant)
    if args.attention_only:
        import torch
        peak, src = measured_peaks()
        print(json.dumps({"attention": attention_case(torch, cfg, args.batch, args.context, peak, src)}))
        return
    if args.impl == "reference":
        run_reference_arm(args, cfg)
    else:
        run_gpu_arm(args, cfg)


if __name__ == "__main__":
    main()
