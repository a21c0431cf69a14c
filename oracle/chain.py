"""The decode chain restated on the CPU oracle, stage by stage: norm+quant -> QKV -> RoPE + Q quant +
paged KV write -> attention -> per-token quant -> O (+residual) -> norm+quant -> gate|up -> act*up+quant
-> down (+residual), then final norm -> LM head (the chain of
v3/crates/rvllm-runtime/src/layer_exec.rs:163-541 of the reference).

Test infrastructure, like everything under oracle/: the checker that the GPU decode stack is compared
with.  Weights arrive as the torch tensors the stack was built from and are copied to the host once.
"""
from __future__ import annotations

import numpy as np


def _host(t):
    import torch

    if t.dtype in (torch.float16, torch.bfloat16):
        return np.ascontiguousarray(t.cpu().view(torch.int16).numpy().view(np.uint16))
    return np.ascontiguousarray(t.cpu().numpy())


class OracleChain:
    def __init__(self, orc, cfg, weights):
        self.o, self.c = orc, cfg
        self.dt = cfg["dtype"]
        h = _host
        self.layers = [{k: h(v) for k, v in l.items()} for l in weights.layers]
        self.head = {k: h(v) for k, v in weights.head.items()}
        B, bs = cfg["batch"], cfg["block_size"]
        self.state = []
        for l in range(cfg["num_layers"]):
            g = cfg["global_every"] != 0 and (l + 1) % cfg["global_every"] == 0
            hd = cfg["global_head_dim"] if g else cfg["sliding_head_dim"]
            mb = (cfg["max_context"] + bs - 1) // bs if g else (cfg["sliding_window"] + bs - 1) // bs + 1
            nblk = B * mb
            slots = nblk * bs
            half = hd // 2
            inv = np.float32(cfg["rope_theta"]) ** (-np.arange(half, dtype=np.float32) / np.float32(half))
            ang = np.arange(cfg["max_context"], dtype=np.float32)[:, None] * inv[None, :].astype(np.float32)
            self.state.append(dict(
                g=g, hd=hd, mb=mb, nblk=nblk, window=-1 if g else cfg["sliding_window"] - 1,
                kc=np.zeros((slots, cfg["kv_heads"], hd), np.uint8), vc=np.zeros((slots, cfg["kv_heads"], hd), np.uint8),
                ks=np.zeros(slots * cfg["kv_heads"], np.float32), vs=np.zeros(slots * cfg["kv_heads"], np.float32),
                tables=np.arange(nblk, dtype=np.int32).reshape(B, mb),
                cos=orc.to_bits16(np.cos(ang).astype(np.float32), self.dt),
                sin=orc.to_bits16(np.sin(ang).astype(np.float32), self.dt)))
        self.pos = 0

    def step(self, tokens):
        o, c, dt = self.o, self.c, self.dt
        B, bs = c["batch"], c["block_size"]
        resid = o.embedding_gather(self.head["embedding"], tokens)
        positions = np.full(B, self.pos, np.int32)
        ctx = np.full(B, self.pos + 1, np.int32)
        for L, S in zip(self.layers, self.state):
            x8, xs = o.rmsnorm_fp8_quant(resid, L["attn_norm_gamma"], c["rms_eps"], dt)
            qkv = o.fp8_gemm(x8, L["qkv_w"], xs, L["qkv_scale"], out_kind=dt)
            page = self.pos // bs
            tp = page % S["mb"] if S["window"] >= 0 else page
            slot = (S["tables"][:, tp] * bs + self.pos % bs).astype(np.int32)
            q8, qs = o.rope_fp8kv(qkv, c["heads"], c["kv_heads"], S["hd"], S["hd"], S["cos"], S["sin"], positions,
                                  slot, S["kc"], S["vc"], S["ks"], S["vs"], dt)
            att = o.paged_decode_fp8(q8, S["kc"], S["vc"], S["tables"], ctx, S["hd"] ** -0.5, c["heads"],
                                     c["kv_heads"], S["hd"], bs, window_size_left=S["window"], k_scale_cache=S["ks"],
                                     v_scale_cache=S["vs"], q_scale_cache=qs.reshape(-1), dtype=dt,
                                     num_blocks_total=S["nblk"])
            a8, a_s = o.quantize_fp8_per_token(att.reshape(B, -1), dt)
            resid = o.fp8_gemm(a8, L["o_w"], a_s, L["o_scale"], residual=resid, out_kind=dt)
            x8, xs = o.rmsnorm_fp8_quant(resid, L["mlp_norm_gamma"], c["rms_eps"], dt)
            gu = o.fp8_gemm(x8, L["gateup_w"], xs, L["gateup_scale"], out_kind=dt)
            h8, hs = o.act_mul_fp8_quant(gu, c["act"], dt)
            resid = o.fp8_gemm(h8, L["down_w"], hs, L["down_scale"], residual=resid, out_kind=dt)
        x8, xs = o.rmsnorm_fp8_quant(resid, self.head["final_norm_gamma"], c["rms_eps"], dt)
        logits = o.fp8_gemm(x8, self.head["lm_head_w"], xs, self.head["lm_head_scale"], out_kind=2)
        cap = np.float32(c.get("logit_softcap", 0.0))
        if cap > 0:  # logit_softcap_kernel's arithmetic on f32 logits: cap * tanhf(x * (1 / cap))
            logits = (cap * np.tanh(logits * (np.float32(1.0) / cap))).astype(np.float32)
        self.pos += 1
        return logits


def greedy_parity(orc, stack, cfg, weights, prompt, steps, logit_tol=2e-2):
    """Runs `prompt` and then `steps` greedy decode steps through `stack` (the GPU decode stack, already
    built from `weights`) and replays them teacher-forced through the oracle chain: at every step the
    oracle is fed the token the GPU was fed, so one near-tie does not derail the rest of the comparison.

    Returns the figures a reader needs to judge "greedy tokens identical": the share of emitted tokens equal
    to the oracle's argmax, the first step where any sequence differs (None = never), the worst gap between
    the oracle's top logit and its logit for the GPU's token relative to the row's largest |logit|, and the
    share of tokens whose gap exceeds `logit_tol` (the GEMM tolerance)."""
    B, P = cfg["batch"], cfg["prompt_len"]
    stack.reset(prompt)
    stack.run(P - 1 + steps)
    stack.sync()
    emitted = stack.tokens()            # emitted[t] = token produced at position t
    chain = OracleChain(orc, cfg, weights)
    exact = total = over = 0
    worst = 0.0
    first_div = None
    rows = np.arange(B)
    for t in range(P - 1 + steps):
        tok_in = prompt[:, t] if t < P else emitted[t - 1]
        logits = chain.step(np.ascontiguousarray(tok_in, np.int32))
        if t < P - 1:
            continue                    # prompt phase: emitted tokens are not fed back
        want = orc.argmax_f32(logits)
        got = emitted[t]
        rel = (logits[rows, want] - logits[rows, got]) / np.abs(logits).max(axis=1)
        over += int((rel > logit_tol).sum())
        worst = max(worst, float(rel.max()))
        same = got == want
        exact += int(same.sum())
        total += B
        if first_div is None and not same.all():
            first_div = t - (P - 1)
    return {"steps": steps, "batch": B, "tokens": total, "exact_match_rate": exact / total,
            "first_divergence_step": first_div, "worst_rel_gap": worst, "share_over_tol": over / total,
            "logit_tol": logit_tol, "teacher_forced": True}
