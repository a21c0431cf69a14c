"""Whole-chain parity: greedy decode through the CUDA-graph decode stack against the CPU oracle
chained stage by stage (norm+quant -> QKV -> RoPE/KV write -> attention -> quant -> O+residual
-> norm+quant -> gate|up -> act+quant -> down+residual -> final norm -> LM head -> argmax).

Identity of greedy tokens between two different GEMM implementations is only well defined when
the top two logits are further apart than the arithmetic noise, so the check is teacher-forced:
the oracle is fed the same input token as the GPU at every step, and the GPU's token must be
the oracle's argmax or have an oracle logit within LOGIT_TOL of it; the fraction of exact
argmax agreement is asserted separately.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

LOGIT_TOL = 2e-2   # relative to the largest |logit| of the row: the GEMM tolerance
LOGIT_TOL_MAX = 6e-2  # no step may be further off than this
# Two correct implementations do not stay bit-identical over hundreds of steps: an activation that
# lands on the other side of an FP8 rounding boundary changes a cached K/V byte by one code (6 %),
# and the caches then differ slightly for the rest of the run.  So a small share of steps may
# exceed LOGIT_TOL; none may exceed LOGIT_TOL_MAX.
MAX_SHARE_OVER_TOL = 0.02


class OracleChain:
    def __init__(self, orc, cfg, weights):
        self.o, self.c = orc, cfg
        self.dt = cfg["dtype"]
        h = lambda t: np.ascontiguousarray(t.cpu().view(torch.int16).numpy().view(np.uint16)) \
            if t.dtype in (torch.float16, torch.bfloat16) else np.ascontiguousarray(t.cpu().numpy())
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
        self.pos += 1
        return logits


def make(cfg, seed=0):
    from rvllm_b200.stack import DecodeStack, random_weights
    w = random_weights(cfg, seed=seed)
    return DecodeStack(cfg, w), w


@pytest.mark.parametrize("dtype,impl", [(0, 1), (1, 2), (1, 0)])
def test_greedy_decode_256_steps_against_oracle_chain(orc, dtype, impl):
    from rvllm_b200.stack import tiny_shape
    steps, P = 256, 16
    cfg = tiny_shape(batch=4, num_layers=2, global_every=2, sliding_window=32, prompt_len=P, max_context=P + steps,
                     max_steps=P + steps, dtype=dtype, gemm_impl=impl)
    stack, w = make(cfg)
    g = np.random.default_rng(0)
    prompt = g.integers(0, cfg["vocab"], (4, P), dtype=np.int32)
    stack.reset(prompt)
    stack.run(P - 1 + steps)
    stack.sync()
    emitted = stack.tokens()            # emitted[t] = token produced at position t
    chain = OracleChain(orc, cfg, w)
    exact = total = over = 0
    worst = 0.0
    for t in range(P - 1 + steps):
        tok_in = prompt[:, t] if t < P else emitted[t - 1]
        logits = chain.step(np.ascontiguousarray(tok_in, np.int32))
        if t < P - 1:
            continue                    # prompt phase: emitted tokens are not fed back
        want = orc.argmax_f32(logits)
        got = emitted[t]
        top = logits[np.arange(4), want]
        mine = logits[np.arange(4), got]
        rel = (top - mine) / np.abs(logits).max(axis=1)
        assert (rel <= LOGIT_TOL_MAX).all(), f"step {t}: token {got} vs oracle {want}, relative gap {rel.max():.4f}"
        over += int((rel > LOGIT_TOL).sum())
        worst = max(worst, float(rel.max()))
        exact += int((got == want).sum())
        total += 4
    assert over / total <= MAX_SHARE_OVER_TOL, f"{over}/{total} tokens beyond the logit tolerance (worst {worst:.4f})"
    # the assertions above force equality wherever the oracle's top-2 gap exceeds the
    # tolerance; with random-init weights the logits are flat, so a few percent of steps are near-ties
    assert exact / total >= 0.9, f"only {exact}/{total} greedy tokens equal the oracle's argmax"
    stack.close()


def test_graph_eager_and_pdl_variants_agree_bitwise(orc):
    """The same 48 steps through (graph, PDL on), (eager, PDL on) and (graph, PDL off): identical
    tokens and bit-identical final logits.  A kernel that read its input before its predecessor
    finished would show up here."""
    from rvllm_b200 import _lib
    from rvllm_b200.stack import tiny_shape
    cfg = tiny_shape(batch=8, num_layers=3, global_every=3, sliding_window=24, prompt_len=8, max_context=64,
                     max_steps=64, dtype=1)
    g = np.random.default_rng(1)
    prompt = g.integers(0, cfg["vocab"], (8, 8), dtype=np.int32)
    L = _lib.lib()
    results = []
    w = None
    try:
        for pdl, eager in ((1, False), (1, True), (0, False)):
            L.rvllm_b200_set_pdl(pdl)
            from rvllm_b200.stack import DecodeStack, random_weights
            w = w or random_weights(cfg, seed=5)
            st = DecodeStack(cfg, w)
            st.reset(prompt)
            st.run(48, eager=eager)
            st.sync()
            results.append((st.tokens().copy(), st.debug_read(1).copy(), st.debug_read(0).copy()))
            st.close()
    finally:
        L.rvllm_b200_set_pdl(1)
    for toks, logits, resid in results[1:]:
        assert np.array_equal(toks, results[0][0])
        assert np.array_equal(logits.view(np.uint32), results[0][1].view(np.uint32))
        assert np.array_equal(resid, results[0][2])


def test_step_host_matches_device_feedback(orc):
    from rvllm_b200.stack import tiny_shape
    cfg = tiny_shape(batch=4, prompt_len=4, max_context=64, max_steps=64)
    stack, w = make(cfg, seed=2)
    prompt = np.random.default_rng(2).integers(0, cfg["vocab"], (4, 4), dtype=np.int32)
    stack.reset(prompt)
    stack.run(20)
    stack.sync()
    a = stack.tokens()
    stack.reset(prompt)
    stack.run(4)                         # through the prompt; history[3] is the first fed-back token
    stack.sync()
    tok_in = stack.tokens()[-1].copy()
    out = np.zeros(4, np.int32)
    got = []
    for _ in range(16):
        stack.step_host(tok_in, out)
        got.append(out.copy())
        tok_in = out.copy()
    assert np.array_equal(np.stack(got), a[4:20])
    stack.close()


def test_stack_config_validation():
    from rvllm_b200 import InvalidArgument
    from rvllm_b200.stack import DecodeStack, Weights, tiny_shape
    for bad in (dict(hidden=500), dict(heads=7), dict(sliding_head_dim=96), dict(batch=0), dict(prompt_len=4096),
                dict(gemm_impl=5), dict(rope_theta=0.5)):
        with pytest.raises(InvalidArgument):
            DecodeStack(tiny_shape(**bad), Weights())
