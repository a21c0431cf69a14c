"""GPU parity of the FP8 GEMM family through the C ABI against the CPU oracle.

Tolerance (stated by the benchmark contract): every element within 2e-2 relative of the
fp32-accumulated oracle, with an absolute floor of 2e-2 x rms(row of the oracle) so that
elements that cancel to ~0 are judged against the scale of their row.  In practice the
error is the 16-bit output rounding (2^-11 for f16, 2^-8 for bf16).
Both kernel families are exercised explicitly: IMPL_STREAM (mma.sync weight streaming) and
IMPL_TCGEN05 (TMA + tcgen05 + TMEM).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from tests import datagen  # noqa: E402

STREAM, TC = 1, 2
RTOL = 2e-2

_wcache = {}
_cache = {}


def case(orc, M, N, K, seed, n_cols=None):
    """Inputs plus the oracle on all (or a seeded subset of) output channels.  Weights are
    generated once per (N, K, seed) and shared by every M."""
    wkey = (N, K, seed)
    if wkey not in _wcache:
        g = np.random.default_rng(seed)
        _wcache.clear()  # keep one weight matrix alive at a time
        _wcache[wkey] = datagen.quant_rows(orc, g.standard_normal((N, K), dtype=np.float32) * 0.02)
    w, w_s = _wcache[wkey]
    key = (M, N, K, seed, n_cols)
    if key not in _cache:
        g = np.random.default_rng(seed * 1000 + M)
        a, a_s = datagen.quant_rows(orc, g.standard_normal((M, K), dtype=np.float32))
        cols = np.arange(N) if n_cols is None or n_cols >= N else np.sort(
            np.random.default_rng(seed).choice(N, n_cols, replace=False))
        want = orc.fp8_gemm(a, np.ascontiguousarray(w[cols]), a_s, np.ascontiguousarray(w_s[cols]), out_kind=2)
        _cache.clear()
        _cache[key] = (a, a_s, w, w_s, cols, want)
    return _cache[key]


def close(got, want, rtol=RTOL, pure_rtol=None):
    """Two checks: every element within rtol * (|want| + rms of its row) — and, without any floor, the pure relative
    error of every element above 1e-3 of its row's rms within rtol (printed: pytest -s shows the figure)."""
    rms = np.sqrt((want.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    floor = rtol * rms
    err = np.abs(got.astype(np.float64) - want)
    bad = err > rtol * np.abs(want) + floor
    assert not bad.any(), f"{bad.sum()} elements off; worst abs err {err.max():.3e}"
    big = np.abs(want) > 1e-3 * rms
    pure = float((err[big] / np.abs(want[big])).max()) if big.any() else 0.0
    print(f"pure max rel err {pure:.2e} over {int(big.sum())} of {want.size} elements above 1e-3 rms")
    pure_rtol = rtol if pure_rtol is None else pure_rtol
    assert pure <= pure_rtol, f"pure relative error {pure:.3e} above {pure_rtol}"
    return float((err / (np.abs(want) + floor)).max())


def run(impl, a, a_s, w, w_s, out_dtype, residual=None):
    from rvllm_b200 import gemm
    M, N = a.shape[0], w.shape[0]
    d = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    out = torch.empty((M, N), dtype=out_dtype, device="cuda")
    res = None
    if residual is not None:
        out.copy_(residual)  # in place on the residual stream, as the reference does
        res = out
    gemm.fp8_gemm_channelscale(out, d(a), d(w), d(a_s), d(w_s), residual=res, impl=impl)
    torch.cuda.synchronize()
    if impl == TC:
        assert gemm.tc_status() == 0, "a bounded wait in the tcgen05 kernel ran out"
    return out


# config 1 (hidden 512, ffn 2048, batch 4) and ragged shapes
SMALL = [(4, 1024, 512), (4, 512, 512), (4, 4096, 512), (4, 512, 2048), (1, 200, 512), (7, 136, 576),
         (33, 72, 1024), (70, 264, 640), (130, 320, 512)]


@pytest.mark.parametrize("impl", [STREAM, TC], ids=["stream", "tc"])
@pytest.mark.parametrize("M,N,K", SMALL)
@pytest.mark.parametrize("out_dtype", ["float16", "bfloat16", "float32"])
def test_gemm_small_shapes(orc, impl, M, N, K, out_dtype):
    a, a_s, w, w_s, cols, want = case(orc, M, N, K, seed=1)
    out = run(impl, a, a_s, w, w_s, getattr(torch, out_dtype))
    close(out.float().cpu().numpy(), want)


@pytest.mark.parametrize("impl", [STREAM, TC], ids=["stream", "tc"])
@pytest.mark.parametrize("out_dtype", ["float16", "bfloat16"])
def test_gemm_residual_in_place(orc, impl, out_dtype):
    M, N, K = 32, 768, 1024
    a, a_s, w, w_s, cols, want = case(orc, M, N, K, seed=2)
    dt = getattr(torch, out_dtype)
    g = np.random.default_rng(5)
    res = torch.from_numpy(g.standard_normal((M, N)).astype(np.float32)).to(dt).cuda()
    out = run(impl, a, a_s, w, w_s, dt, residual=res)
    close(out.float().cpu().numpy(), want + res.float().cpu().numpy())


# the four projection shapes of the benchmark (QKV, O, gate|up, down) at decode batch sizes;
# the oracle is evaluated on 512 seeded output channels of each
PROJ = [("qkv", 8192, 5376), ("o", 5376, 4096), ("gateup", 43008, 5376), ("down", 5376, 21504)]


@pytest.mark.parametrize("impl", [STREAM, TC], ids=["stream", "tc"])
@pytest.mark.parametrize("M", [1, 8, 32, 128])
@pytest.mark.parametrize("name,N,K", PROJ)
def test_gemm_projection_shapes(orc, impl, name, N, K, M):
    a, a_s, w, w_s, cols, want = case(orc, M, N, K, seed=1, n_cols=512)
    out = run(impl, a, a_s, w, w_s, torch.bfloat16)
    close(out.float().cpu().numpy()[:, cols], want)


@pytest.mark.parametrize("impl", [STREAM, TC], ids=["stream", "tc"])
@pytest.mark.parametrize("M", [512, 2048])
@pytest.mark.parametrize("name,N,K", PROJ)
def test_gemm_large_m(orc, impl, name, N, K, M):
    """The large-M half of the sweep on all four projection shapes (96 seeded output channels against the oracle)."""
    if impl == STREAM and name != "qkv":
        pytest.skip("the streaming cross-check runs the QKV shape only at these sizes")
    a, a_s, w, w_s, cols, want = case(orc, M, N, K, seed=1, n_cols=96)
    out = run(impl, a, a_s, w, w_s, torch.float16)
    close(out.float().cpu().numpy()[:, cols], want)


def test_lm_head_full_vocabulary_against_oracle(orc):
    """The LM head at its real size, N = 262144 x K = 5376, batch 32: f32 logits on 512 seeded token ids against the
    oracle, and the argmax epilogue against argmax over those f32 logits."""
    from rvllm_b200 import _lib, gemm
    from rvllm_b200.launchers import ArgmaxLaunch
    L = _lib.lib()
    M, V, K = 32, 262144, 5376
    gen = torch.Generator(device="cuda")
    gen.manual_seed(17)
    W = torch.empty((V, K), dtype=torch.uint8, device="cuda")
    for lo in range(0, V, 32768):     # E4M3 codes of N(0, 1) * 64 values, slab by slab (no NaN codes)
        W[lo:lo + 32768] = (torch.randn((32768, K), device="cuda", generator=gen) * 64.0).clamp(-448, 448) \
            .to(torch.float8_e4m3fn).view(torch.uint8)
    WS = torch.rand(V, dtype=torch.float32, device="cuda", generator=gen) * 2e-4 + 1e-4
    g = np.random.default_rng(17)
    a, a_s = datagen.quant_rows(orc, g.standard_normal((M, K), dtype=np.float32))
    A, AS = torch.from_numpy(a).cuda(), torch.from_numpy(a_s).cuda()
    logits = torch.empty((M, V), dtype=torch.float32, device="cuda")
    gemm.fp8_gemm_channelscale(logits, A, W, AS, WS, impl=TC)
    cols = np.sort(g.choice(V, 512, replace=False))
    ct = torch.from_numpy(cols).cuda()
    want = orc.fp8_gemm(a, np.ascontiguousarray(W[ct].cpu().numpy()), a_s, np.ascontiguousarray(WS[ct].cpu().numpy()), out_kind=2)
    close(logits[:, ct].cpu().numpy(), want)
    toks = torch.empty(M, dtype=torch.int32, device="cuda")
    ArgmaxLaunch(M, V).launch(logits, toks)
    n = int(L.rvllm_fp8_gemm_lm_head_argmax_workspace(M, V))
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    got = torch.full((M,), -5, dtype=torch.int32, device="cuda")
    _lib.check(L.rvllm_fp8_gemm_lm_head_argmax(got.data_ptr(), A.data_ptr(), W.data_ptr(), AS.data_ptr(), WS.data_ptr(), M, V, K,
                                               0.0, ws.data_ptr(), n, _lib.current_stream()), "lm_head_argmax")
    torch.cuda.synchronize()
    assert gemm.tc_status() == 0
    assert got.tolist() == toks.tolist()


@pytest.mark.parametrize("impl", [STREAM, TC], ids=["stream", "tc"])
def test_gemm_is_deterministic_and_linear_in_scales(orc, impl):
    M, N, K = 32, 5376, 4096
    a, a_s, w, w_s, cols, want = case(orc, M, N, K, seed=3, n_cols=64)
    o1 = run(impl, a, a_s, w, w_s, torch.float32)
    o2 = run(impl, a, a_s, w, w_s, torch.float32)
    assert torch.equal(o1, o2)  # split-K reduces in a fixed order: bitwise reproducible
    o3 = run(impl, a, a_s * 4.0, w, w_s * 0.5, torch.float32)
    assert torch.equal(o3, o1 * 2.0)  # power-of-two rescaling commutes with rounding


@pytest.mark.parametrize("M", [1, 7, 32, 50, 64, 100, 128])
@pytest.mark.parametrize("splits", [2, 3, 5, 7, 8])
@pytest.mark.parametrize("mode", ["scale", "residual", "f32"])
def test_split_k_push_and_pull_reductions_are_bitwise_equal(orc, M, splits, mode):
    """Inside a split-K cluster the partial tiles are either pushed into the finishing CTA's
    receive buffer (behind its ring for batch tiles up to 32 rows; the idle ring itself, after one more
    cluster meeting, for 64- and 128-row tiles) or pulled out of the peers' rings.  All sum in
    cluster-rank order, so every output bit must agree, and all must match the oracle."""
    from rvllm_b200 import _lib
    N, K = 1336, 2176  # ragged last weight tile (1336 = 10 * 128 + 56), 17 K blocks: uneven split ranges
    a, a_s, w, w_s, cols, want = case(orc, M, N, K, seed=6)
    dt = torch.float32 if mode == "f32" else torch.bfloat16
    res = None
    if mode == "residual":
        res = torch.from_numpy(np.random.default_rng(8).standard_normal((M, N)).astype(np.float32)).to(dt).cuda()
    outs = []
    try:
        for reduce_mode in (0, 1, 3):  # push + mbarrier arrivals (ring push above 32 rows), pull, push + cluster barrier
            _lib.lib().rvllm_fp8_gemm_tc_tune(0, splits)
            _lib.lib().rvllm_fp8_gemm_tc_reduce(reduce_mode)
            outs.append(run(TC, a, a_s, w, w_s, dt, residual=res))
    finally:
        _lib.lib().rvllm_fp8_gemm_tc_tune(0, 0)
        _lib.lib().rvllm_fp8_gemm_tc_reduce(0)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    ref = want + (res.float().cpu().numpy() if res is not None else 0.0)
    close(outs[0].float().cpu().numpy(), ref)


def test_both_families_agree(orc):
    M, N, K = 32, 8192, 5376
    a, a_s, w, w_s, cols, want = case(orc, M, N, K, seed=4, n_cols=64)
    o1 = run(STREAM, a, a_s, w, w_s, torch.float32).cpu().numpy()
    o2 = run(TC, a, a_s, w, w_s, torch.float32).cpu().numpy()
    # two summation orders of the same f32 products: 1e-4 of |value| + row rms; elements a thousand times smaller
    # than their row's rms carry the same absolute difference, so their pure relative bound is 1e-3
    close(o1, o2.astype(np.float64), rtol=1e-4, pure_rtol=1e-3)


@pytest.mark.parametrize("impl", [STREAM, TC], ids=["stream", "tc"])
def test_reference_named_entry_points(orc, impl):
    """cutlass_fp8_gemm_channelscale and the scalar-B-scale v0 pair, called as the reference
    loader would (v3/crates/rvllm-cutlass/src/lib_so.rs:500-512,734-746)."""
    from rvllm_b200 import _lib
    L = _lib.lib()
    M, N, K = 8, 1024, 512
    a, a_s, w, w_s, cols, want = case(orc, M, N, K, seed=6)
    d = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    A, W, AS, WS = d(a), d(w), d(a_s), d(w_s)
    out = torch.empty((M, N), dtype=torch.float16, device="cuda")
    ws_bytes = max(int(L.cutlass_fp8_gemm_channelscale_workspace(M, N, K)), 256)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    s = _lib.current_stream()
    assert L.cutlass_fp8_gemm_channelscale(out.data_ptr(), A.data_ptr(), W.data_ptr(), AS.data_ptr(), WS.data_ptr(),
                                           M, N, K, ws.data_ptr(), ws_bytes, s) == 0
    torch.cuda.synchronize()
    close(out.float().cpu().numpy(), want)
    # scalar weight scale + residual
    b_scale = torch.tensor([0.01], dtype=torch.float32, device="cuda")
    res = torch.ones((M, N), dtype=torch.float16, device="cuda")
    n2 = int(L.cutlass_fp8_gemm_residual_v0_workspace_size(M, N, K))
    ws2 = torch.empty(max(n2, 256), dtype=torch.uint8, device="cuda")
    out2 = torch.empty_like(out)
    assert L.cutlass_fp8_gemm_residual_v0(out2.data_ptr(), A.data_ptr(), W.data_ptr(), AS.data_ptr(),
                                          b_scale.data_ptr(), res.data_ptr(), M, N, K, ws2.data_ptr(), n2, s) == 0
    torch.cuda.synchronize()
    want2 = orc.fp8_gemm(a, w, a_s, np.full(N, 0.01, np.float32), out_kind=2) + 1.0
    close(out2.float().cpu().numpy(), want2)
    # an undersized workspace is refused before any launch
    assert L.cutlass_fp8_gemm_residual_v0(out2.data_ptr(), A.data_ptr(), W.data_ptr(), AS.data_ptr(),
                                          b_scale.data_ptr(), res.data_ptr(), M, N, K, ws2.data_ptr(), 16, s) != 0


SINGLE = 3  # rvllm_fp8_gemm_gateup_act_quant: the one-launch form or RVLLM_E_UNSUPPORTED


@pytest.mark.parametrize("impl", [STREAM, TC, SINGLE, 0], ids=["stream", "tc", "single-launch", "auto"])
@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("M,I,K", [(32, 2048, 512), (7, 1024, 1024), (32, 21504, 5376)])
def test_gateup_act_quant_equals_unfused_chain(orc, impl, act, M, I, K):
    """The gate|up + act + quant entry point == GEMM, then the stand-alone act-mul-quant kernel (itself bit-equal to
    the reference's kernels, test_gpu_rowops), bit for bit: the two-launch forms against their own GEMM family, the
    one-launch form (products never leave the chip, row maxima across a grid barrier) against the tcgen05 chain; and
    close to the oracle."""
    from rvllm_b200 import gemm
    from rvllm_b200.launchers import FusedActMulFp8QuantLaunch
    if I > 4096 and impl == STREAM:
        pytest.skip("the full-size case runs on the tensor-core forms")
    big = I > 4096
    if big:   # operands straight on the device: the CPU oracle is not asked for 43008 x 5376 x 32
        g = torch.Generator(device="cuda")
        g.manual_seed(11)
        A = torch.randint(0, 255, (M, K), dtype=torch.uint8, device="cuda", generator=g)
        A[A == 0x7F] = 0x7E
        W = torch.randint(0, 127, (2 * I, K), dtype=torch.uint8, device="cuda", generator=g) ^ \
            (torch.randint(0, 2, (2 * I, K), dtype=torch.uint8, device="cuda", generator=g) << 7)
        W[(W & 0x7F) == 0x7F] = 0x7E
        AS = torch.rand(M, dtype=torch.float32, device="cuda", generator=g) * 1e-2 + 1e-3
        WS = torch.rand(2 * I, dtype=torch.float32, device="cuda", generator=g) * 1e-4 + 1e-5
    else:
        a, a_s, w, w_s, cols, want = case(orc, M, 2 * I, K, seed=7)
        d = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
        A, W, AS, WS = d(a), d(w), d(a_s), d(w_s)
    ws = torch.empty(gemm.gateup_workspace_bytes(M, I, K), dtype=torch.uint8, device="cuda")
    ws.fill_(0xA5)                                            # the entry point must not count on a clean workspace
    out = torch.empty((M, I), dtype=torch.uint8, device="cuda")
    sc = torch.empty(M, dtype=torch.float32, device="cuda")
    for _ in range(2):                                        # twice: the barrier words are left clean
        gemm.fp8_gemm_gateup_act_quant(out, sc, A, W, AS, WS, act, 1, ws, impl=impl)
    gu = torch.empty((M, 2 * I), dtype=torch.bfloat16, device="cuda")
    gemm.fp8_gemm_channelscale(gu, A, W, AS, WS, impl=STREAM if impl == STREAM else TC)
    out2 = torch.empty_like(out)
    sc2 = torch.empty_like(sc)
    FusedActMulFp8QuantLaunch(M, I, act).launch(out2, sc2, gu)
    torch.cuda.synchronize()
    assert gemm.tc_status() == 0
    assert torch.equal(sc, sc2) and torch.equal(out, out2)
    if big:
        return
    # against the oracle chain: dequantised values agree within the GEMM tolerance + one FP8 step
    wb, wsc = orc.act_mul_fp8_quant(orc.to_bits16(want, orc.BF16), act, orc.BF16, orc.MODE_CUDA)
    got = orc.e4m3_decode(out.cpu().numpy()) * sc.cpu().numpy()[:, None]
    ref = orc.e4m3_decode(wb) * wsc[:, None]
    assert np.abs(got - ref).max() <= 0.07 * np.abs(ref).max()


def test_gemm_rejects_bad_arguments():
    from rvllm_b200 import _lib
    L = _lib.lib()
    t = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    f = torch.zeros(64, dtype=torch.float32, device="cuda")
    o = torch.zeros(4096, dtype=torch.float16, device="cuda")
    p, s = t.data_ptr(), _lib.current_stream()
    args = lambda M, N, K, a=p: (o.data_ptr(), 0, a, p, f.data_ptr(), f.data_ptr(), None, M, N, K, 1, None, 0, s)
    assert L.rvllm_fp8_gemm_channelscale(*args(0, 8, 64)) == _lib.E_INVALID
    assert L.rvllm_fp8_gemm_channelscale(*args(4, 8, 0)) == _lib.E_INVALID
    assert L.rvllm_fp8_gemm_channelscale(*args(4, 8, 72)) == _lib.E_UNSUPPORTED
    assert L.rvllm_fp8_gemm_channelscale(*args(4, 8, 64, a=p + 1)) == _lib.E_INVALID
    assert L.rvllm_fp8_gemm_channelscale(*args(4, 8, 64, a=None)) == _lib.E_INVALID


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("M,heads,kv_heads,K", [(32, 32, 16, 5376), (7, 8, 4, 1024), (1, 4, 4, 640), (128, 32, 16, 5376),
                                                 (100, 32, 16, 5376), (50, 8, 4, 1024), (64, 32, 16, 5376)])
def test_fused_qkv_rope_epilogue_equals_gemm_then_rope(orc, dtype, M, heads, kv_heads, K):
    """The QKV GEMM with RoPE + Q quantisation + paged KV write in its epilogue must leave the same
    bytes and scale bits as the GEMM into a 16-bit buffer followed by the RoPE / KV-write kernel:
    Q codes and scales, K / V cache rows and per-slot scales, untouched slots included; one token
    has no cache slot and one has a position outside the tables."""
    from rvllm_b200 import gemm, launchers
    HD = 128
    N = (heads + 2 * kv_heads) * HD
    dt = getattr(torch, dtype)
    g = np.random.default_rng(M + heads + K)
    a, a_s = datagen.quant_rows(orc, g.standard_normal((M, K), dtype=np.float32))
    w, w_s = datagen.quant_rows(orc, g.standard_normal((N, K), dtype=np.float32) * 0.05)
    d = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    da, das, dw, dws = d(a), d(a_s), d(w), d(w_s)
    max_pos, slots = 96, 3 * M + 5
    ang = g.uniform(0, 6.28, (max_pos, HD // 2)).astype(np.float32)
    cos, sin = torch.from_numpy(np.cos(ang)).to(dt).cuda(), torch.from_numpy(np.sin(ang)).to(dt).cuda()
    positions = g.integers(0, max_pos, M).astype(np.int32)
    slot_mapping = g.permutation(slots)[:M].astype(np.int32)
    if M > 2:
        positions[1] = max_pos + 3      # nothing may be written for this token
        slot_mapping[2] = -1            # Q written, no cache write
    dpos, dslot = d(positions), d(slot_mapping)

    def fresh():
        gg = np.random.default_rng(5)
        return dict(q8=torch.full((M, heads, HD), 0xAB, dtype=torch.uint8, device="cuda"),
                    qs=torch.full((M, heads), -7.0, dtype=torch.float32, device="cuda"),
                    kc=d(gg.integers(0, 255, (slots, kv_heads, HD), dtype=np.uint8)),
                    vc=d(gg.integers(0, 255, (slots, kv_heads, HD), dtype=np.uint8)),
                    ks=d(gg.uniform(0.1, 1, slots * kv_heads).astype(np.float32)),
                    vs=d(gg.uniform(0.1, 1, slots * kv_heads).astype(np.float32)))
    ref = fresh()
    qkv = torch.empty((M, N), dtype=dt, device="cuda")
    gemm.fp8_gemm_channelscale(qkv, da, dw, das, dws, impl=TC)
    launchers.rope_fp8kv(qkv, heads, kv_heads, HD, HD, cos, sin, dpos, dslot, ref["q8"], ref["qs"], ref["kc"], ref["vc"],
                         ref["ks"], ref["vs"])
    got = fresh()
    taken = launchers.qkv_rope_fp8kv(da, dw, das, dws, heads, kv_heads, HD, cos, sin, dpos, dslot, got["q8"], got["qs"],
                                     got["kc"], got["vc"], got["ks"], got["vs"])
    torch.cuda.synchronize()
    assert gemm.tc_status() == 0
    if not taken:
        pytest.skip("shape not taken by the fused epilogue (no split-K launch)")
    for key in ("q8", "kc", "vc"):
        assert torch.equal(got[key], ref[key]), key
    for key in ("qs", "ks", "vs"):
        assert torch.equal(got[key].view(torch.int32), ref[key].view(torch.int32)), key


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("M,N,K,parts", [(32, 5376, 4096, 16), (7, 640, 1024, 4), (1, 1336, 2176, 1), (32, 5376, 8192, 16)])
def test_residual_gemm_from_16bit_activations_equals_quantiser_then_gemm(orc, dtype, M, N, K, parts):
    """The residual GEMM that quantises its own A tiles from 16-bit activations (given per-row
    partial maxima) must produce the bytes of: per-token quantiser, then the residual GEMM."""
    import ctypes
    from rvllm_b200 import gemm, _lib
    from rvllm_b200.launchers import QuantizeFp8PerTokenLaunch
    dt = getattr(torch, dtype)
    g = np.random.default_rng(N + K + M)
    x = torch.from_numpy((g.standard_normal((M, K)) * 0.7).astype(np.float32)).to(dt).cuda()
    if M > 2:
        x[1].zero_()                                # an all-zero row: scale 1e-12
    w, w_s = datagen.quant_rows(orc, g.standard_normal((N, K), dtype=np.float32) * 0.05)
    d = lambda t: torch.from_numpy(np.ascontiguousarray(t)).cuda()
    dw, dws = d(w), d(w_s)
    res0 = torch.from_numpy(g.standard_normal((M, N)).astype(np.float32)).to(dt).cuda()
    # reference chain
    a8 = torch.empty((M, K), dtype=torch.uint8, device="cuda")
    a_s = torch.empty(M, dtype=torch.float32, device="cuda")
    QuantizeFp8PerTokenLaunch(M, K).launch(a8, a_s, x)
    ref = res0.clone()
    gemm.fp8_gemm_channelscale(ref, a8, dw, a_s, dws, residual=ref, impl=TC)
    # fused form: partial maxima over `parts` column groups of each row
    amax = x.float().abs().reshape(M, parts, K // parts).amax(dim=2).contiguous()
    got = res0.clone()
    code = 0 if dt == torch.float16 else 1
    rc = _lib.lib().rvllm_fp8_gemm_residual_from16(got.data_ptr(), code, x.data_ptr(), amax.data_ptr(), parts,
                                                   dw.data_ptr(), dws.data_ptr(), got.data_ptr(), M, N, K,
                                                   torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and gemm.tc_status() == 0
    assert torch.equal(got, ref)


@pytest.mark.parametrize("M", [1, 32, 130])
@pytest.mark.parametrize("softcap", [0.0, 30.0])
def test_lm_head_argmax_epilogue_equals_logits_then_argmax(orc, M, softcap):
    """The LM head that keeps only per-tile argmax winners against f32 logits -> [soft cap] -> argmax (C ABI): same
    tokens, including exact ties (two identical weight rows: the lower token id wins), a row whose logits are all
    NaN (-1) and a ragged last weight tile."""
    from rvllm_b200 import _lib, gemm
    from rvllm_b200.launchers import ArgmaxLaunch
    L = _lib.lib()
    V, K = 32768 + 40, 512
    g = np.random.default_rng(M)
    w, w_s = datagen.quant_rows(orc, g.standard_normal((V, K), dtype=np.float32) * 0.02)
    a, a_s = datagen.quant_rows(orc, g.standard_normal((M, K), dtype=np.float32))
    want_first = orc.argmax_f32(orc.fp8_gemm(a, w, a_s, w_s, out_kind=2))
    # plant a tie for row 0: a later row of W equal to the winning row (bytes and scale)
    lo = int(want_first[0])
    hi = (lo + 5000) % V
    lo, hi = min(lo, hi), max(lo, hi)
    w[hi], w_s[hi] = w[int(want_first[0])], w_s[int(want_first[0])]
    w[lo], w_s[lo] = w[int(want_first[0])], w_s[int(want_first[0])]
    if M > 2:
        a_s[2] = np.nan                                    # every logit of row 2 is NaN
    d = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    A, AS, W, WS = d(a), d(a_s), d(w), d(w_s)
    logits = torch.empty((M, V), dtype=torch.float32, device="cuda")
    gemm.fp8_gemm_channelscale(logits, A, W, AS, WS, impl=TC)
    if softcap > 0:
        _lib.check(L.rvllm_logit_softcap_launch(logits.data_ptr(), M, V, softcap, 2, _lib.current_stream()), "softcap f32")
    want = torch.empty(M, dtype=torch.int32, device="cuda")
    ArgmaxLaunch(M, V).launch(logits, want)
    n = int(L.rvllm_fp8_gemm_lm_head_argmax_workspace(M, V))
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    got = torch.full((M,), -5, dtype=torch.int32, device="cuda")
    _lib.check(L.rvllm_fp8_gemm_lm_head_argmax(got.data_ptr(), A.data_ptr(), W.data_ptr(), AS.data_ptr(), WS.data_ptr(), M, V, K,
                                               softcap, ws.data_ptr(), n, _lib.current_stream()), "lm_head_argmax")
    torch.cuda.synchronize()
    assert gemm.tc_status() == 0
    assert got.tolist() == want.tolist()
    assert got[0].item() == lo
    if M > 2:
        assert got[2].item() == -1
    assert L.rvllm_fp8_gemm_lm_head_argmax(got.data_ptr(), A.data_ptr(), W.data_ptr(), AS.data_ptr(), WS.data_ptr(), M, V, K,
                                           softcap, ws.data_ptr(), 16, _lib.current_stream()) == _lib.E_WORKSPACE


def test_two_devices_in_one_process(orc):
    """cudaFuncSetAttribute belongs to a device, not to the process: the tcgen05 GEMM (split-K push form, > 48 KB of
    dynamic shared memory) and the tcgen05 attention launched on device 0 and then on device 1 of the same process,
    local buffers only, must give the same bytes.  Needs two GPUs; skipped otherwise."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in one process")
    from rvllm_b200 import gemm
    from rvllm_b200.attention import PagedDecodeFp8Launcher, PagedDecodeParams
    M, N, K = 32, 5376, 4096
    a, a_s, w, w_s, cols, want = case(orc, M, N, K, seed=12, n_cols=64)
    c = datagen.attention_case(orc, 4, 32, 16, 128, 16, [600, 17, 128, 300], seed=12)
    outs = []
    try:
        for dev in (0, 1):
            torch.cuda.set_device(dev)
            d = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda(dev)
            out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
            gemm.fp8_gemm_channelscale(out, d(a), d(w), d(a_s), d(w_s), impl=TC)
            p = PagedDecodeParams(4, 32, 16, 128, 16, c["max_blocks"], c["num_blocks"], 128 ** -0.5, -1)
            ws = torch.empty(max(p.workspace_bytes(), 16), dtype=torch.uint8, device="cuda")
            o = torch.empty((4, 32, 128), dtype=torch.float16, device="cuda")
            PagedDecodeFp8Launcher(p).launch(d(c["q"]), d(c["k"]), d(c["v"]), o, d(c["tables"]), d(c["ctx"]), workspace=ws,
                                             k_scale_cache=d(c["ks"]), v_scale_cache=d(c["vs"]), q_scale_cache=d(c["qs"]))
            torch.cuda.synchronize()
            assert gemm.tc_status() == 0
            outs.append((out.float().cpu().numpy(), o.float().cpu().numpy()))
    finally:
        torch.cuda.set_device(0)
    close(outs[0][0][:, cols], want)
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
