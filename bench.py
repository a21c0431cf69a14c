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
    return 6650.0, "fallback (no MEASURED_PEAKS.json: an earlier device-copy measurement of the same part)"


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
    t_run0 = time.perf_counter()
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
        # every "step" is an estimate from a timed sample of the step's work (the description is in
        # cpu_baseline.sample), not a full step: steps x ms_per_step is not the wall time of this run
        "sampled": True, "sample_seconds_per_step": per_step, "wall_seconds": time.perf_counter() - t_run0,
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


def ncu_traffic_bytes(kernel, N, K, M):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of a kernel as captured under ncu: read from
    the table kept beside the capture summaries, so a re-captured kernel updates the figure in one place and a
    shape that was never captured reports null."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            rows = json.load(f)["captures"]
    except (OSError, ValueError, KeyError):
        return None
    for r in rows:
        if r.get("kernel") == kernel and (r.get("N"), r.get("K"), r.get("M")) == (N, K, M):
            return r.get("dram_bytes_per_launch")
    return None


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
            "traffic": ncu_traffic_bytes("fp8_gemm_tc_kernel", 2 * F, H, B)}


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


# ----------------------------------------------------------------------------- config 2: the GEMM sweep
PROJECTIONS = [("qkv", 8192, 5376, False), ("o", 5376, 4096, True), ("gateup", 43008, 5376, False),
               ("down", 5376, 21504, True)]
SWEEP_M = [1, 8, 32, 128, 512, 2048]


def time_launches(torch, launch, n, warm=3):
    """Mean device time of n launches (CUDA events on the launching stream, after warm-up)."""
    for i in range(warm):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        launch(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3 / n


def fp8_tensor_peak(torch, seconds=2.0):
    """Dense FP8 throughput of this repository's own tcgen05 kernel on an 8192^3 problem (2 * N^3 flops):
    best single launch (burst) and a back-to-back loop of about `seconds` (sustained, under the power cap).
    No FP8 peak is published for this part; 2 x the measured bf16 cuBLAS figure is printed beside it."""
    from rvllm_b200 import gemm
    n = 8192
    a = torch.randint(0, 120, (n, n), dtype=torch.uint8, device="cuda")
    w = torch.randint(0, 120, (n, n), dtype=torch.uint8, device="cuda")
    a_s = torch.full((n,), 0.01, dtype=torch.float32, device="cuda")
    w_s = torch.full((n,), 0.01, dtype=torch.float32, device="cuda")
    out = torch.empty((n, n), dtype=torch.bfloat16, device="cuda")
    run = lambda i=0: gemm.fp8_gemm_channelscale(out, a, w, a_s, w_s, impl=gemm.IMPL_TCGEN05)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(10):
        best = min(best, time_launches(torch, run, 1, warm=0))
    reps = max(8, int(seconds / best))
    sustained = time_launches(torch, run, reps, warm=0)
    flops = 2.0 * n ** 3
    out_d = {"shape": "8192^3", "burst_tflops": flops / best / 1e12, "sustained_tflops": flops / sustained / 1e12,
             "sustained_launches": reps}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        out_d["twice_measured_bf16_tflops"] = {"burst": 2 * d["bf16_tflops"], "sustained": 2 * d["bf16_tflops_sustained"]}
    except (OSError, ValueError, KeyError):
        pass
    del a, w, out
    return out_d


def gemm_sweep(torch, cfg, shapes=None, ms=None, with_peak=True):
    """Four projection shapes x M in {1, 8, 32, 128, 512, 2048} through the C ABI: per-token activation scales,
    per-channel weight scales, 16-bit output (the O and down shapes with the fused residual).  Each launch of a
    row cycles to another copy of the weights so that the stream comes from HBM (copies x bytes > L2)."""
    from rvllm_b200 import gemm
    peak, peak_src = measured_peaks()
    fp8 = fp8_tensor_peak(torch) if with_peak else None
    rows = []
    tdt = torch.float16 if cfg["dtype"] == 0 else torch.bfloat16
    for name, N, K, residual in PROJECTIONS:
        if shapes and name not in shapes:
            continue
        copies = max(2, int(300e6 // (N * K)) + 1)
        ws = [torch.randint(0, 120, (N, K), dtype=torch.uint8, device="cuda") for _ in range(copies)]
        w_s = torch.full((N,), 0.001, dtype=torch.float32, device="cuda")
        for M in (ms or SWEEP_M):
            a = torch.randint(0, 120, (M, K), dtype=torch.uint8, device="cuda")
            a_s = torch.full((M,), 0.01, dtype=torch.float32, device="cuda")
            out = torch.zeros((M, N), dtype=tdt, device="cuda")
            res = out if residual else None

            def launch(i, a=a, a_s=a_s, out=out, res=res):
                gemm.fp8_gemm_channelscale(out, a, ws[i % copies], a_s, w_s, residual=res, impl=gemm.IMPL_TCGEN05)
            sec = time_launches(torch, launch, max(4 * copies, 12))
            algo = gemm_bytes(M, N, K, residual)
            flops = 2.0 * M * N * K
            rows.append({"shape": name, "N": N, "K": K, "M": M, "us": sec * 1e6, "gbs": algo / sec / 1e9,
                         "frac_hbm": algo / sec / 1e9 / peak, "tflops": flops / sec / 1e12,
                         "frac_fp8": flops / sec / 1e12 / fp8["burst_tflops"] if fp8 else None, "weight_copies": copies})
            del a, out
        del ws
    assert gemm.tc_status() == 0, "a bounded wait in the tcgen05 GEMM ran out"
    return {"gemm_sweep": rows, "fp8_peak": fp8, "hbm_peak_gbs": peak, "hbm_peak_source": peak_src,
            "note": "frac_fp8 is against the burst figure of this repository's own kernel at 8192^3"}


# ----------------------------------------------------------------------------- config 3: ragged attention
def ragged_attention(torch, cfg, batch=64, lo=512, hi=32768, seed=2, with_reference=False, reps=6):
    """The decode-attention launch of the ragged configuration: `batch` sequences with context lengths drawn
    uniformly from [lo, hi], 32 query / 16 KV heads, both layer kinds (sliding: head_dim 128, window 1024, ring
    of pages; global: head_dim 256), block_size 16, shuffled physical blocks, random cache bytes with
    per-(slot, head) scales.  with_reference also times the reference's two kernels on the same buffers."""
    import numpy as np
    from rvllm_b200.attention import PagedDecodeFp8Launcher, PagedDecodeParams
    peak, peak_src = measured_peaks()
    H_, KVH, bs = cfg["heads"], cfg["kv_heads"], cfg["block_size"]
    tdt = torch.float16   # the reference entry points write f16
    ctx_np = np.random.default_rng(seed).integers(lo, hi + 1, batch).astype(np.int32)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    out = []
    for tag, HD, window in (("sliding", cfg["sliding_head_dim"], cfg["sliding_window"] - 1),
                            ("global", cfg["global_head_dim"], -1)):
        att = np.minimum(ctx_np, window + 1) if window >= 0 else ctx_np
        mb = (window + 1 + bs - 1) // bs + 1 if window >= 0 else int((ctx_np.max() + bs - 1) // bs)
        need = np.full(batch, mb) if window >= 0 else (ctx_np + bs - 1) // bs
        nblk = int(need.sum())
        perm = torch.randperm(nblk, device="cuda", generator=gen).to(torch.int32)
        tables = torch.full((batch, mb), -1, dtype=torch.int32, device="cuda")
        o = 0
        for b in range(batch):
            tables[b, :int(need[b])] = perm[o:o + int(need[b])]
            o += int(need[b])
        k = torch.randint(0, 120, (nblk, bs, KVH, HD), dtype=torch.uint8, device="cuda", generator=gen)
        v = torch.randint(0, 120, (nblk, bs, KVH, HD), dtype=torch.uint8, device="cuda", generator=gen)
        sc = torch.full((nblk * bs * KVH,), 0.01, dtype=torch.float32, device="cuda")
        q = torch.randint(0, 120, (batch, H_, HD), dtype=torch.uint8, device="cuda", generator=gen)
        qs = torch.full((batch * H_,), 0.01, dtype=torch.float32, device="cuda")
        ctxs = torch.from_numpy(ctx_np).cuda()
        res = torch.empty((batch, H_, HD), dtype=tdt, device="cuda")
        p = PagedDecodeParams(batch, H_, KVH, HD, bs, mb, nblk, HD ** -0.5, window)
        ws = torch.empty(max(p.workspace_bytes(), 16), dtype=torch.uint8, device="cuda")
        la = PagedDecodeFp8Launcher(p)
        sec = time_launches(torch, lambda i: la.launch(q, k, v, res, tables, ctxs, workspace=ws, k_scale_cache=sc,
                                                       v_scale_cache=sc, q_scale_cache=qs), reps, warm=2)
        algo = int(att.sum()) * KVH * (2 * HD + 8)
        row = {"kernel": "paged decode attention, %s layer shape (head_dim %d)" % (tag, HD), "batch": batch,
               "contexts": "uniform in [%d, %d], seed %d" % (lo, hi, seed), "attended_tokens": int(att.sum()),
               "us_per_launch": sec * 1e6, "achieved": algo / sec / 1e9, "peak": peak, "unit": "GB/s",
               "frac": algo / sec / 1e9 / peak, "peak_source": peak_src, "algorithmic_bytes_per_launch": algo,
               "cache_bytes_touched_exceed_l2": bool(algo > 126e6)}
        if with_reference:
            row["reference"] = reference_attention_times(torch, dict(q=q, k=k, v=v, sc=sc, qs=qs, tables=tables, ctx=ctxs,
                                                                     batch=batch, heads=H_, kv_heads=KVH, hd=HD, bs=bs, mb=mb,
                                                                     nblk=nblk, window=window), sec)
        out.append(row)
        del k, v
    return out


# ----------------------------------------------------------------------------- the reference's kernels, same GPU
def _ref_dir():
    return os.path.join(ROOT, "oracle", "_ref")


def reference_attention_times(torch, c, ours_sec):
    """fa_sm89_paged_decode_fp8 (the reference's split-KV kernel, compiled from v3/kernels/fp8_decode_v2.cu with
    its own flags) and flash_attention_2_decode_fp8kv_kernel (what its Gemma bring-up launches on this
    architecture; it has no ring paging, so it is given the global-layer case only), on the buffers of `c`."""
    import ctypes as C
    from tests import ptx_harness as H
    out = {}
    so = os.path.join(_ref_dir(), "libfa_sm89_ref.so")
    o16 = torch.empty((c["batch"], c["heads"], c["hd"]), dtype=torch.float16, device="cuda")
    if os.path.exists(so):
        ref = C.CDLL(so)
        ref.fa_sm89_decode_workspace_size.restype = C.c_uint64
        vp, f32, i32 = C.c_void_p, C.c_float, C.c_int
        ref.fa_sm89_paged_decode_fp8.argtypes = [vp] * 7 + [C.c_size_t] + [vp] * 6 + [f32] + [i32] * 8 + [vp]
        need = int(ref.fa_sm89_decode_workspace_size(c["batch"], c["heads"], c["kv_heads"], c["hd"]))
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        st = torch.cuda.current_stream().cuda_stream

        def run(i):
            rc = ref.fa_sm89_paged_decode_fp8(c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), o16.data_ptr(),
                                              c["tables"].data_ptr(), c["ctx"].data_ptr(), ws.data_ptr(), need,
                                              c["sc"].data_ptr(), c["sc"].data_ptr(), c["qs"].data_ptr(), None, None, None,
                                              c["hd"] ** -0.5, c["batch"], c["heads"], c["kv_heads"], c["hd"], c["bs"],
                                              c["mb"], c["nblk"], c["window"], st)
            assert rc == 0
        sec = time_launches(torch, run, 2, warm=1)
        out["fa_sm89_paged_decode_fp8"] = {"us_per_launch": sec * 1e6, "ours_speedup": sec / ours_sec}
    if c["window"] < 0 and os.path.exists(os.path.join(_ref_dir(), "flash_attention.ptx")):
        mod = H.reference("flash_attention")
        hd = c["hd"]
        smem = (2 * 16 * hd + 16 + 4) * 4          # v3/crates/rvllm-attention/src/decode.rs:572-630
        if smem > 48 * 1024:
            mod.set_max_dynamic_smem("flash_attention_2_decode_fp8kv_kernel", smem)

        def run2(i):
            mod.launch("flash_attention_2_decode_fp8kv_kernel", (c["batch"], c["heads"]), (128,), smem,
                       [H.P(o16), H.P(c["q"]), H.P(c["k"]), H.P(c["v"]), H.P(c["sc"]), H.P(c["sc"]), H.P(c["qs"]), H.NULL(),
                        H.NULL(), H.P(c["tables"]), H.P(c["ctx"]), H.NULL(), H.F(hd ** -0.5), H.I(c["heads"]),
                        H.I(c["kv_heads"]), H.I(hd), H.I(c["bs"]), H.I(c["mb"]), H.I(c["window"]), H.I(c["nblk"])])
        sec = time_launches(torch, run2, 2, warm=1)
        out["flash_attention_2_decode_fp8kv_kernel"] = {"us_per_launch": sec * 1e6, "ours_speedup": sec / ours_sec}
    return out


def reference_kernel_table(torch, cfg):
    """ours / theirs device time per kernel, same GPU, same run: the reference's own CUDA kernels for this path
    (compiled from its sources with its flags into oracle/_ref) at the Rust launchers' geometry, next to this
    repository's C-ABI calls on the same buffers.  Test-side tooling: the decode path never loads oracle/_ref."""
    import numpy as np
    from tests import ptx_harness as H
    from rvllm_b200 import gemm, launchers
    if not H.have_reference():
        return {"unavailable": "oracle/_ref is not built (the reference checkout was not present at build time)"}
    rows = []
    B, Hd, F, V = 32, cfg["hidden"], cfg["ffn"], cfg["vocab"]
    f16 = torch.float16

    def add(name, ours, theirs, n=20):
        to = time_launches(torch, ours, n)
        tt = time_launches(torch, theirs, n)
        rows.append({"kernel": name, "ours_us": to * 1e6, "reference_us": tt * 1e6, "speedup": tt / to})

    # row kernels at the decode shapes
    x = torch.randn((B, Hd), device="cuda").to(f16)
    gamma = torch.ones(Hd, dtype=f16, device="cuda")
    o8 = torch.empty((B, Hd), dtype=torch.uint8, device="cuda")
    sc = torch.empty(B, dtype=torch.float32, device="cuda")
    rn = H.reference("fused_rmsnorm_fp8_quant")
    add("fused_rmsnorm_fp8_quant [32 x 5376]",
        lambda i: launchers.FusedRmsnormFp8QuantLaunch(B, Hd, 1e-6).launch(o8, sc, x, gamma),
        lambda i: rn.launch("fused_rmsnorm_fp8_quant_kernel", (B,), (1024,), 128,
                            [H.P(o8), H.P(sc), H.P(x), H.P(gamma), H.F(1e-6), H.I(Hd)]))
    xq = torch.randn((B, 4096), device="cuda").to(f16)
    oq = torch.empty((B, 4096), dtype=torch.uint8, device="cuda")
    add("quantize_fp8_per_token [32 x 4096]",
        lambda i: launchers.QuantizeFp8PerTokenLaunch(B, 4096).launch(oq, sc, xq),
        lambda i: rn.launch("quantize_fp8_per_token_kernel", (B,), (1024,), 128, [H.P(oq), H.P(sc), H.P(xq), H.I(4096)]))
    gu = torch.randn((B, 2 * F), device="cuda").to(f16)
    oa = torch.empty((B, F), dtype=torch.uint8, device="cuda")
    sl = H.reference("fused_silu_fp8_quant")
    add("fused_silu_mul_fp8_quant [32 x 21504]",
        lambda i: launchers.FusedSiluMulFp8QuantLaunch(B, F).launch(oa, sc, gu),
        lambda i: sl.launch("fused_silu_mul_fp8_quant_kernel", (B,), (1024,), 128, [H.P(oa), H.P(sc), H.P(gu), H.I(F)]))
    lg = torch.randn((B, V), device="cuda")
    am = torch.zeros(B, dtype=torch.int32, device="cuda")
    ar = H.reference("argmax")
    add("argmax [32 x 262144]", lambda i: launchers.ArgmaxLaunch(B, V).launch(lg, am),
        lambda i: ar.launch("argmax_kernel", (B,), (1024,), 0, [H.P(lg), H.P(am), H.I(V)]), n=10)
    # M = 1 GEMV: the reference's two kernels + its f32 -> f16 pass, against one call of ours
    kt, sk, cv = H.reference("fp8_channelscale_gemv_ktiled"), H.reference("fp8_channelscale_gemv_splitk"), H.reference("f32_to_f16_sat")
    for name, N, K, _ in PROJECTIONS:
        copies = max(2, int(300e6 // (N * K)) + 1)
        ws = [torch.randint(0, 120, (N, K), dtype=torch.uint8, device="cuda") for _ in range(copies)]
        w_s = torch.full((N,), 0.001, dtype=torch.float32, device="cuda")
        a = torch.randint(0, 120, (1, K), dtype=torch.uint8, device="cuda")
        a_s = torch.full((1,), 0.01, dtype=torch.float32, device="cuda")
        o16 = torch.empty((1, N), dtype=f16, device="cuda")
        o32 = torch.zeros(N, dtype=torch.float32, device="cuda")
        gx = (N + 7) // 8

        def theirs(i, N=N, K=K, ws=ws, copies=copies, w_s=w_s, a=a, a_s=a_s, o16=o16, o32=o32, gx=gx):
            w = ws[i % copies]
            if N <= 8192 and K >= 8192:   # gemma4_layer_exec.rs:2379: split-K 8 into a zeroed f32 buffer
                o32.zero_()
                sk.launch("fp8_channelscale_gemv_splitk_kernel", (gx, 8), (256,), 0,
                          [H.P(o32), H.P(w), H.P(w_s), H.P(a), H.P(a_s), H.I(N), H.I(K), H.I(8)])
            else:
                tile = min(8192, K)
                kt.launch("fp8_channelscale_gemv_ktiled_kernel", (gx,), (256,), tile * 2,
                          [H.P(o32), H.P(w), H.P(w_s), H.P(a), H.P(a_s), H.I(N), H.I(K), H.I(tile)])
            cv.launch("f32_to_f16_sat_kernel", ((N + 255) // 256,), (256,), 0, [H.P(o16), H.P(o32), H.I(N)])
        add("fp8 GEMM M=1, %s [%d x %d]" % (name, N, K),
            lambda i, ws=ws, copies=copies, w_s=w_s, a=a, a_s=a_s, o16=o16: gemm.fp8_gemm_channelscale(
                o16, a, ws[i % copies], a_s, w_s, impl=gemm.IMPL_TCGEN05), theirs, n=max(12, 3 * copies))
        del ws
    att = ragged_attention(torch, cfg, batch=64, with_reference=True, reps=4)
    return {"kernels": rows, "attention_ragged_batch64": att,
            "note": "reference kernels: the reference's sources compiled for sm_100 with its own flags; M > 1 FP8 GEMMs "
                    "have no reference-side kernel that compiles here (CUTLASS sm_90a / cuBLASLt are not linked)"}


# ----------------------------------------------------------------------------- config 5: ragged replicas
def ragged_replica_run(torch, cfg, weights, per_gpu_batch, steps, lo=1024, hi=16384, seed=4, barrier=None):
    """One replica's share of the ragged serving configuration: `per_gpu_batch` sequences whose contexts are
    drawn uniformly from [lo, hi] (seeded per rank), KV caches seeded synthetically at those lengths, global
    layers sharing one block pool sized by need, then `steps` decode steps timed on the device."""
    import numpy as np
    from rvllm_b200.stack import DecodeStack
    rank = int(os.environ.get("RANK", "0"))
    ctx = np.random.default_rng(seed * 1000 + rank).integers(lo, hi + 1, per_gpu_batch).astype(np.int32)
    reserve = steps + 8
    bs = cfg["block_size"]
    pool = int(((ctx + reserve + bs - 1) // bs).sum())
    c = dict(cfg, batch=per_gpu_batch, prompt_len=0, max_context=(hi + reserve + 255) // 256 * 256, max_steps=reserve,
             kv_pool_blocks=pool)
    stack = DecodeStack(c, weights)
    stack.seed_contexts(ctx)
    stack.run(4)
    stack.sync()
    if barrier:
        barrier()
    sec = time_steps(torch, stack, steps)
    if barrier:
        barrier()
    # bytes: the step model with every sequence at its own mid-run context
    mid = ctx.astype(np.int64) + 4 + steps // 2
    b_step = step_bytes(c, per_gpu_batch, 0)
    for l in range(c["num_layers"]):
        g = c["global_every"] != 0 and (l + 1) % c["global_every"] == 0
        hd = c["global_head_dim"] if g else c["sliding_head_dim"]
        eff = mid if g else np.minimum(mid, c["sliding_window"])
        b_step += int(eff.sum()) * c["kv_heads"] * (2 * hd + 8)
    res = {"batch_per_gpu": per_gpu_batch, "steps": steps, "seconds": sec, "ms_per_step": sec / steps * 1e3,
           "tok_s": per_gpu_batch * steps / sec, "contexts": "uniform in [%d, %d], seed %d + rank" % (lo, hi, seed),
           "mean_context": float(ctx.mean()), "kv_pool_blocks_per_global_layer": pool,
           "device_bytes": stack.device_bytes(), "step_bytes": b_step}
    stack.close()
    return res


# ----------------------------------------------------------------------------- the one-launch layer block, stage by stage
def layer_block_trace(torch, cfg, batch, reps=5):
    """The layer-block kernel (O projection .. next RMSNorm in one launch, CTAs resident behind grid-wide barriers)
    alone at the benchmark's layer dimensions, cycling over three weight sets (1.1 GB, larger than L2): device time
    per launch, and the kernel's own %globaltimer stamps of its stage boundaries, reduced over the CTAs."""
    import numpy as np
    from rvllm_b200 import _lib
    from rvllm_b200.stack import _quant_weight
    L = _lib.lib()
    M, H, F, KO = batch, cfg["hidden"], cfg["ffn"], cfg["heads"] * cfg["sliding_head_dim"]
    tdt = torch.float16 if cfg["dtype"] == 0 else torch.bfloat16
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    sets = []
    for _ in range(3):
        o_w, o_s = _quant_weight(H, KO, gen, 0.02)
        gu_w, gu_s = _quant_weight(2 * F, H, gen, 0.02)
        d_w, d_s = _quant_weight(H, F, gen, 0.02)
        sets.append((o_w, o_s, gu_w, gu_s, d_w, d_s))
    attn = (torch.randn((M, KO), generator=gen, device="cuda") * 0.5).to(tdt)
    amax = attn.float().abs().reshape(M, 16, KO // 16).amax(dim=2).contiguous()
    res = torch.randn((M, H), generator=gen, device="cuda").to(tdt)
    g1 = torch.ones(H, dtype=tdt, device="cuda")
    x8 = torch.empty((M, H), dtype=torch.uint8, device="cuda")
    xs = torch.empty(M, dtype=torch.float32, device="cuda")
    h8 = torch.empty((M, F), dtype=torch.uint8, device="cuda")
    hs = torch.empty(M, dtype=torch.float32, device="cuda")
    wsb = int(L.rvllm_fp8_layer_block_workspace(H, F))
    ws = torch.zeros(wsb, dtype=torch.uint8, device="cuda")
    st = _lib.current_stream()

    def launch(i):
        o_w, o_s, gu_w, gu_s, d_w, d_s = sets[i % 3]
        _lib.check(L.rvllm_fp8_layer_block(M, H, F, KO, cfg["act"], cfg["dtype"], cfg["rms_eps"], attn.data_ptr(), amax.data_ptr(),
                                           16, None, None, o_w.data_ptr(), o_s.data_ptr(), res.data_ptr(), g1.data_ptr(),
                                           g1.data_ptr(), x8.data_ptr(), xs.data_ptr(), gu_w.data_ptr(), gu_s.data_ptr(),
                                           h8.data_ptr(), hs.data_ptr(), d_w.data_ptr(), d_s.data_ptr(), ws.data_ptr(), wsb, 31,
                                           st), "fp8_layer_block")
    sec = time_launches(torch, launch, 30, warm=6)
    G = H // 128 * 8
    tr = torch.zeros((G, 16), dtype=torch.int64, device="cuda")
    L.rvllm_fp8_layer_block_trace(tr.data_ptr())
    names = ["start", "predecessor done", "O accumulator complete", "O partials stored", "after barrier 1",
             "rows: O finished + RMSNorm", "after barrier 2", "gate|up accumulator complete", "act*up partial maxima stored",
             "after barrier 3", "act*up quantised", "after barrier 4", "down accumulator complete", "down partials stored",
             "after barrier 5", "rows: down finished + RMSNorm (end)"]
    acc = np.zeros((reps, 16, 3))
    try:
        for r in range(reps):
            launch(r)
            torch.cuda.synchronize()
            t = tr.cpu().numpy().astype(np.float64)
            t = (t - t[:, 0].min()) / 1e3
            acc[r, :, 0], acc[r, :, 1], acc[r, :, 2] = t.min(axis=0), t.mean(axis=0), t.max(axis=0)
    finally:
        L.rvllm_fp8_layer_block_trace(None)
    m = acc.mean(axis=0)
    weights = sum(t.numel() for t in (sets[0][0], sets[0][2], sets[0][4]))
    peak, _ = measured_peaks()
    return {"kernel": "fp8_layer_block_kernel", "batch": M, "hidden": H, "ffn": F, "o_k": KO, "us_per_launch": sec * 1e6,
            "weight_bytes_per_launch": weights, "frac_of_hbm_peak": weights / sec / 1e9 / peak,
            "stamps_us": [{"point": n, "first_cta": m[k, 0], "mean": m[k, 1], "last_cta": m[k, 2]} for k, n in enumerate(names)],
            "note": "globaltimer stamps, 0.26 us resolution; first / mean / last over the %d CTAs, mean of %d launches" % (G, reps)}


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


ABLATE_BITS = [(1, "RMSNorm + quant (attention block)"), (2, "QKV GEMM + RoPE / KV write"), (4, "decode attention"),
               (8, "O projection + residual"), (16, "RMSNorm + quant (MLP block)"), (32, "gate|up GEMM"),
               (64, "act-mul-quant"), (128, "down projection + residual")]


def ablation(torch, cfg, weights, batches, steps):
    """What each launch of a layer costs inside the decode graph: the step timed in full and with that launch left
    out of every layer (the tokens of such a step mean nothing; its neighbours' work does not depend on the data).
    Kernel time that overlaps with a neighbour under programmatic dependent launch does not show up here, time the
    chain loses around the launch does."""
    from rvllm_b200 import _lib
    L = _lib.lib()
    out = {}
    for B in batches:
        def timed(mask):
            L.rvllm_stack_debug_skip(mask)
            try:
                r = run_batch(torch, cfg, weights, B, steps, 3, 0, seeded=True)
            finally:
                L.rvllm_stack_debug_skip(0)
            return r
        full = timed(0)
        rows = []
        for bit, name in ABLATE_BITS:
            r = timed(bit)
            rows.append({"launch": name, "ms_per_step_without": r["ms_per_step"],
                         "us_per_layer": (full["ms_per_step"] - r["ms_per_step"]) * 1e3 / cfg["num_layers"]})
        tail = timed(255)
        out[str(B)] = {"ms_per_step": full["ms_per_step"], "layers": cfg["num_layers"], "per_launch": rows,
                       "sum_us_per_layer": sum(x["us_per_layer"] for x in rows),
                       "step_us_per_layer": (full["ms_per_step"] - tail["ms_per_step"]) * 1e3 / cfg["num_layers"],
                       "ms_per_step_tail_only": tail["ms_per_step"]}
    return out


GEMM_TRACE_POINTS = ["CTA runs", "predecessor complete", "first K block in shared memory", "last MMA issued",
                     "accumulator complete", "partials exchanged", "outputs stored"]


def gemm_trace(torch, cfg, weights, B, reps=5):
    """Timeline of the tcgen05 GEMM launches of one decode step inside the CUDA graph: the kernel's own %globaltimer
    stamps (earliest and latest CTA per point, rvllm_fp8_gemm_tc_trace), read after single graph replays.  Launch
    order per layer: QKV, O, gate|up, down; the LM head closes the step.  Reported per kind, averaged over the
    sliding layers: how long before its predecessor's completion the launch was resident, and the phases after it;
    and the time between a launch's last store and the next launch's "predecessor complete" (the row kernel or the
    attention in between, with both hand-offs)."""
    import numpy as np
    from rvllm_b200 import _lib
    from rvllm_b200.stack import DecodeStack
    L = _lib.lib()
    c = dict(cfg, batch=B)
    G = 4 * c["num_layers"] + 1
    tr = torch.zeros((G, 16), dtype=torch.int64, device="cuda")
    _lib.check(L.rvllm_fp8_gemm_tc_trace(tr.data_ptr(), G), "fp8_gemm_tc_trace")
    try:
        stack = DecodeStack(c, weights)      # the graph is recorded with the rows in place
    finally:
        L.rvllm_fp8_gemm_tc_trace(None, 0)
    stack.seed_context(c["prompt_len"] - 1)
    stack.run(4)
    stack.sync()
    acc = []
    for _ in range(reps):
        tr[:, 0::2] = -1                     # all ones: the even entries take a minimum
        tr[:, 1::2] = 0
        torch.cuda.synchronize()
        stack.run(1)
        stack.sync()
        t = tr.cpu().numpy().view(np.uint64).astype(np.float64)
        acc.append((t - t[0, 0]) / 1e3)      # us from the first CTA of the first GEMM
    stack.close()
    t = np.mean(acc, axis=0)                 # [G][16]
    kinds = ["QKV (+RoPE / KV write)", "O projection", "gate|up", "down projection"]
    global_every = c["global_every"]
    rows = []
    for k, kind in enumerate(kinds):
        sel = [4 * l + k for l in range(1, c["num_layers"]) if not (global_every and (l + 1) % global_every == 0)]
        first = lambda pt: t[sel, 2 * pt].mean()
        last = lambda pt: t[sel, 2 * pt + 1].mean()
        prev_end = np.mean([t[i - 1, 13] for i in sel])
        rows.append({"launch": kind, "launches_averaged": len(sel),
                     "resident_before_predecessor_done_us": last(1) - first(0),
                     "previous_gemm_end_to_predecessor_done_us": first(1) - prev_end,
                     "predecessor_done_to_first_k_block_us": last(2) - last(1),
                     "first_k_block_to_last_mma_us": last(3) - last(2),
                     "last_mma_to_accumulator_us": last(4) - last(3),
                     "accumulator_to_exchange_us": (last(5) - last(4)) if t[sel[0], 11] > 0 else None,
                     "to_outputs_stored_us": last(6) - (last(5) if t[sel[0], 11] > 0 else last(4)),
                     "predecessor_done_to_end_us": last(6) - first(1)})
    head = {"predecessor_done_to_end_us": t[G - 1, 13] - t[G - 1, 2], "start_to_end_us": t[G - 1, 13] - t[G - 1, 0]}
    return {"batch": B, "layers": c["num_layers"], "points": GEMM_TRACE_POINTS, "per_kind": rows, "lm_head": head,
            "step_span_us": float(t[:, 13].max()),
            "note": "globaltimer stamps, mean of %d single graph replays; sliding layers 1.. averaged" % reps}


def greedy_parity_block(steps):
    """The composition the headline number times (fused QKV+RoPE epilogue, tcgen05 attention leaving per-row
    maxima, O projection quantising its own A tiles, fused gate|up activation, cluster argmax) decoded greedily at
    a width the CPU oracle can chain — 3 layers (2 sliding head_dim 128 + 1 global head_dim 256), hidden 1024,
    32q/16kv heads, batch 32 — and replayed teacher-forced through the oracle.  The oracle is the checker here,
    nothing measured."""
    import numpy as np
    import oracle as orc
    from oracle.chain import greedy_parity
    from rvllm_b200.stack import DecodeStack, random_weights, tiny_shape
    cfg = tiny_shape(hidden=1024, ffn=2048, vocab=2048, num_layers=3, heads=32, kv_heads=16, sliding_head_dim=128,
                     global_head_dim=256, sliding_window=32, global_every=3, dtype=1, batch=32, prompt_len=8,
                     max_context=8 + steps, max_steps=8 + steps)
    w = random_weights(cfg, seed=0)
    stack = DecodeStack(cfg, w)
    prompt = np.random.default_rng(32).integers(0, cfg["vocab"], (32, 8), dtype=np.int32)
    stats = greedy_parity(orc, stack, cfg, w, prompt, steps)
    stats["launches_per_step"] = stack.launches_per_step()
    stats["shape"] = "3 layers (2 sliding hd128 + 1 global hd256), hidden 1024, ffn 2048, vocab 2048, 32q/16kv, batch 32"
    stack.close()
    return stats


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
        "weights_gb": weights.nbytes() / 1e9, "setup_s": setup_s, "fused_block": cfg["fused_block"],
        "collective": "none on the data path (independent replicas); NCCL only for the barrier around the timed "
                      "region and the max-over-ranks of the device times" if world > 1 else "none (one GPU)",
        "greedy_tokens_tail": main["greedy_tokens_tail"],
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
    if rank == 0 and not args.no_roofline:
        # (before the long ragged run: after seconds of sustained load the part sits at its power cap and a lower SM
        # clock, which this HBM-bound kernel follows; the headline region above ran at the clocks it reports)
        line["roofline"] = dominant_kernel_roofline(torch, cfg, weights, B, peak, peak_src)
    if args.ragged_batch > 0 and cfg["num_layers"] > 0:
        # the ragged serving configuration, every rank: aggregate batch = ragged_batch x N (1024 at N = 8),
        # contexts uniform in [1024, 16384], 128 steps; weak scaling like the headline line
        rg = ragged_replica_run(torch, cfg, weights, args.ragged_batch, args.ragged_steps, barrier=barrier)
        rg_sec = replicas.job_seconds(dist, rg["seconds"], device="cuda")
        line["ragged_replicas"] = {
            "workload": "aggregate batch %d split evenly over %d GPU(s), contexts uniform in [1024, 16384], %d decode "
                        "steps, KV caches seeded synthetically at those lengths" % (args.ragged_batch * world, world,
                                                                                     args.ragged_steps),
            "value": world * args.ragged_batch * args.ragged_steps / rg_sec, "unit": UNIT, "scaling": "weak",
            "ms_per_step": rg_sec / args.ragged_steps * 1e3, "batch_per_gpu": args.ragged_batch,
            "aggregate_batch": args.ragged_batch * world, "mean_context_rank0": rg["mean_context"],
            "frac_of_hbm_peak_rank0": rg["step_bytes"] / (rg["seconds"] / args.ragged_steps) / 1e9 / peak,
            "kv_pool_blocks_per_global_layer": rg["kv_pool_blocks_per_global_layer"],
            "stack_device_gb_rank0": rg["device_bytes"] / 1e9,
            "note": "per-GPU batch is fixed at the share of the 8-GPU configuration (1024 / 8); a single GPU cannot "
                    "hold 1024 such sequences (about 0.9 GB of KV each)"}
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            import oracle as orc
            orc.build()
            orc.use_all_host_threads()
            est, spent, desc = cpu_step_sample(cfg, B, ctx=cfg["prompt_len"], min_seconds=12.0)
            line["cpu_baseline"] = {"value": B / est, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
                                    "sample": desc, "sample_seconds": spent}
        if world == 1 and not args.no_by_batch:
            # the metric names three batch sizes: the headline one above, the other two here
            line["by_batch"] = {str(B): {"tok_s": main["tok_s"], "ms_per_step": main["ms_per_step"],
                                         "frac_of_hbm_peak": step_frac}}
            for b in (1, 128):
                if b == B:
                    continue
                r = run_batch(torch, cfg, weights, b, args.steps, args.warmup, 0)
                line["by_batch"][str(b)] = {"tok_s": r["tok_s"], "ms_per_step": r["ms_per_step"],
                                            "frac_of_hbm_peak": r["step_bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / peak}
        if world == 1 and not args.no_cpu_baseline and not args.no_parity:
            line["parity"] = greedy_parity_block(args.parity_steps)
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
    ap.add_argument("--no-by-batch", action="store_true", help="skip the batch 1 and batch 128 runs of the metric")
    ap.add_argument("--no-parity", action="store_true", help="skip the greedy-token check against the oracle chain")
    ap.add_argument("--parity-steps", type=int, default=64)
    ap.add_argument("--ragged-batch", type=int, default=128,
                    help="per-GPU batch of the ragged serving configuration (0 = skip it)")
    ap.add_argument("--ragged-steps", type=int, default=128)
    ap.add_argument("--gemm-sweep", action="store_true",
                    help="only the GEMM sweep: four projection shapes x M in {1, 8, 32, 128, 512, 2048}, and the FP8 peak")
    ap.add_argument("--sweep-shapes", default="", help="--gemm-sweep: only these projections (comma list of qkv,o,gateup,down)")
    ap.add_argument("--sweep-m", default="", help="--gemm-sweep: only these batch sizes (comma list)")
    ap.add_argument("--no-fp8-peak", action="store_true", help="--gemm-sweep: skip the 8192^3 peak measurement (small case for ncu)")
    ap.add_argument("--ragged-attention", action="store_true",
                    help="only the decode attention at batch 64 with contexts uniform in [512, 32768]")
    ap.add_argument("--fused-block", type=int, default=0, choices=[0, 1],
                    help="1: run the step with the one-launch layer block (O projection .. next RMSNorm) instead of the chain")
    ap.add_argument("--gemm-trace", action="store_true",
                    help="only the in-graph timeline of the GEMM launches of a step (the kernels' own time stamps)")
    ap.add_argument("--ablate", default="", help="only the in-graph cost of each launch of a layer, for these batches (comma list)")
    ap.add_argument("--layer-block-trace", action="store_true",
                    help="only the layer-block kernel alone at the layer dimensions, with its stage-boundary time stamps")
    ap.add_argument("--vs-ref-kernels", action="store_true",
                    help="only the ours / reference kernel table (needs oracle/_ref)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-roofline", action="store_true")
    ap.add_argument("--roofline-only", action="store_true",
                    help="small case for ncu: only the dominant kernel over 4 gate|up weight matrices (0.9 GB)")
    ap.add_argument("--attention-only", action="store_true",
                    help="small case for ncu: only the decode-attention kernel at the two layer shapes")
    ap.add_argument("--context", type=int, default=576, help="context length of --attention-only")
    ap.add_argument("--seeded-context", action="store_true",
                    help="profiling aid: fill the KV caches synthetically instead of running the 512 prefill steps")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed region with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    args = ap.parse_args()
    from rvllm_b200.stack import gemma31b_shape
    need = 512 + max(args.warmup, 3) + args.steps + args.e2e_steps + 8
    cfg = gemma31b_shape(args.batch, num_layers=args.layers, max_context=(need + 255) // 256 * 256, max_steps=need,
                         fused_block=args.fused_block)
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
    if args.gemm_sweep or args.ragged_attention or args.vs_ref_kernels or args.layer_block_trace or args.ablate or args.gemm_trace:
        import torch
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the CUDA path has no CPU fallback")
        if args.gemm_sweep:
            print(json.dumps(gemm_sweep(torch, cfg, [x for x in args.sweep_shapes.split(",") if x],
                                        [int(x) for x in args.sweep_m.split(",") if x], not args.no_fp8_peak)))
        if args.ragged_attention:
            print(json.dumps({"attention_ragged": ragged_attention(torch, cfg)}))
        if args.vs_ref_kernels:
            print(json.dumps({"ref_kernels": reference_kernel_table(torch, cfg)}))
        if args.layer_block_trace:
            print(json.dumps({"layer_block": layer_block_trace(torch, cfg, args.batch)}))
        if args.gemm_trace:
            from rvllm_b200.stack import random_weights
            w = random_weights(cfg, seed=3)
            print(json.dumps({"gemm_trace": gemm_trace(torch, cfg, w, args.batch)}))
        if args.ablate:
            from rvllm_b200.stack import random_weights
            w = random_weights(cfg, seed=3)
            print(json.dumps({"ablation": ablation(torch, cfg, w, [int(x) for x in args.ablate.split(",")], args.steps)}))
        return
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
