"""Pins against the reference's own CUDA kernels, compiled under oracle/_ref and run on the same GPU on
the same seeded inputs:

  * FP8 GEMM at M = 1: fp8_channelscale_gemv_{ktiled,splitk}_kernel + f32_to_f16_sat_kernel with the host
    geometry of fp8_channelscale_gemv_m1 (v3/crates/rvllm-runtime/src/gemma4_layer_exec.rs:2376-2457).
    reference ~ oracle pins the oracle's GEMM definition; ours ~ reference is the parity claim.
  * RoPE + Q quantisation + paged FP8 KV write, both forms: fused_rope_partial_fp8kv_kernel (Gemma
    half-split, dynamic scales) and fused_rope_cache_fp8kv_kernel (Llama interleaved pairs, static scales)
    — bytes and scale bits.
  * Gemma-4 decorations and the soft cap: fused_qkv_rmsnorm, fused_norm_add_residual_f16(+in),
    residual_scale_f16, logit_softcap — every output bit.

Each of this repository's kernels is launched both as the PTX artifact at the reference launcher's
geometry and through the C-ABI launcher.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from tests import datagen  # noqa: E402
from tests import ptx_harness as H  # noqa: E402

needs_ref = pytest.mark.skipif(not H.have_reference(), reason="oracle/_ref not built (needs the reference checkout)")


def d(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def dev16(bits, dtype=0):
    t = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).cuda()
    return t.view(torch.float16 if dtype == 0 else torch.bfloat16)


def bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def max_rel(got, want, floor_of_rms):
    """Largest |got - want| / |want| over the elements with |want| > floor_of_rms * rms(want)."""
    want = want.astype(np.float64)
    rms = np.sqrt((want ** 2).mean())
    sel = np.abs(want) > floor_of_rms * rms
    return float((np.abs(got.astype(np.float64) - want)[sel] / np.abs(want)[sel]).max()), int(sel.sum())


# --------------------------------------------------------------------------- GEMM at M = 1
GEMV_SHAPES = [("qkv", 8192, 5376), ("o", 5376, 4096), ("gateup", 43008, 5376), ("down", 5376, 21504),
               ("lm_head_slice", 16384, 5376)]


def reference_gemv_m1(a, a_scale, w, w_scale):
    """fp8_channelscale_gemv_m1: split-K kernel (8 slices, f32 atomics into a zeroed buffer) when
    n <= 8192 and k >= 8192, else the K-tiled kernel; then f32 -> f16 with saturation.  The host passes
    TILE_K = 8192 unchanged, which the kernel refuses when K < 8192 (it returns without writing); the tile
    used here is min(8192, K), what RVLLM_TILE_K = K selects."""
    N, K = w.shape
    out32 = torch.zeros(N, dtype=torch.float32, device="cuda")
    wpb = 8
    grid_x = (N + wpb - 1) // wpb
    if N <= 8192 and K >= 8192:
        H.reference("fp8_channelscale_gemv_splitk").launch(
            "fp8_channelscale_gemv_splitk_kernel", (grid_x, 8), (wpb * 32,), 0,
            [H.P(out32), H.P(w), H.P(w_scale), H.P(a), H.P(a_scale), H.I(N), H.I(K), H.I(8)])
    else:
        tile = min(8192, K)
        H.reference("fp8_channelscale_gemv_ktiled").launch(
            "fp8_channelscale_gemv_ktiled_kernel", (grid_x,), (wpb * 32,), tile * 2,
            [H.P(out32), H.P(w), H.P(w_scale), H.P(a), H.P(a_scale), H.I(N), H.I(K), H.I(tile)])
    out16 = torch.empty(N, dtype=torch.float16, device="cuda")
    H.reference("f32_to_f16_sat").launch("f32_to_f16_sat_kernel", ((N + 255) // 256,), (256,), 0,
                                         [H.P(out16), H.P(out32), H.I(N)])
    torch.cuda.synchronize()
    return out32.cpu().numpy(), out16.float().cpu().numpy()


@needs_ref
@pytest.mark.parametrize("name,N,K", GEMV_SHAPES, ids=[s[0] for s in GEMV_SHAPES])
def test_gemm_m1_against_reference_gemv_kernels(orc, name, N, K):
    from rvllm_b200 import gemm
    g = np.random.default_rng(N + K)
    w, w_s = datagen.quant_rows(orc, g.standard_normal((N, K), dtype=np.float32) * 0.02)
    a, a_s = datagen.quant_rows(orc, g.standard_normal((1, K), dtype=np.float32))
    A, AS, W, WS = d(a), d(a_s), d(w), d(w_s)
    ref32, ref16 = reference_gemv_m1(A, AS, W, WS)
    # (1) the oracle's GEMM definition against the reference kernel: both accumulate exact products in f32,
    # in different orders
    want = orc.fp8_gemm(a, w, a_s, w_s, out_kind=2)[0]
    rel_orc, n_orc = max_rel(ref32, want, 1e-3)
    print(f"{name}: reference GEMV vs oracle, max rel over {n_orc} elements with |want| > 1e-3 rms: {rel_orc:.2e}")
    assert np.abs(ref32 - want).max() <= 2e-5 * np.abs(want).max()
    assert rel_orc <= 2e-2
    # (2) this repository's kernels against the reference kernel: f16 out, both families, no rms floor
    for impl in (gemm.IMPL_TCGEN05, gemm.IMPL_STREAM):
        out = torch.empty((1, N), dtype=torch.float16, device="cuda")
        gemm.fp8_gemm_channelscale(out, A, W, AS, WS, impl=impl)
        torch.cuda.synchronize()
        assert gemm.tc_status() == 0
        got = out.float().cpu().numpy()[0]
        rel_lo, n_lo = max_rel(got, ref16, 1e-3)
        rel_hi, n_hi = max_rel(got, ref16, 5e-2)
        print(f"{name} impl {impl}: ours vs reference f16, max rel {rel_lo:.2e} over |want| > 1e-3 rms ({n_lo}), "
              f"{rel_hi:.2e} over |want| > 5e-2 rms ({n_hi})")
        assert rel_hi <= 2e-2                                   # the contract's tolerance, pure relative error
        assert np.abs(got - ref16).max() <= 2e-3 * np.abs(ref16).max()


# --------------------------------------------------------------------------- RoPE, Gemma half-split form
def rope_inputs(orc, T, heads, kv_heads, HD, rotary, seed, slots=None, max_pos=96):
    g = np.random.default_rng(seed)
    slots = slots or 3 * T + 5
    N = (heads + 2 * kv_heads) * HD
    qkv = orc.to_bits16((g.standard_normal((T, N)) * 1.3).astype(np.float32), 0)
    ang = g.uniform(0, 6.28, (max_pos, max(rotary, 2) // 2)).astype(np.float32)
    cos, sin = orc.to_bits16(np.cos(ang), 0), orc.to_bits16(np.sin(ang), 0)
    positions = g.integers(0, max_pos, T).astype(np.int32)
    slot_mapping = g.permutation(slots)[:T].astype(np.int32)
    if T > 3:
        positions[1] = max_pos + 3      # nothing may be written for this token
        slot_mapping[2] = -1            # Q written, no cache write
        slot_mapping[3] = slots + 7     # beyond the cache: no cache write
    return dict(qkv=qkv, cos=cos, sin=sin, positions=positions, slot_mapping=slot_mapping, slots=slots, max_pos=max_pos, N=N)


def fresh_outputs(T, heads, kv_heads, HD, slots, scales=True):
    gg = np.random.default_rng(5)
    o = dict(q8=torch.full((T, heads, HD), 0xAB, dtype=torch.uint8, device="cuda"),
             kc=d(gg.integers(0, 255, (slots, kv_heads, HD), dtype=np.uint8)),
             vc=d(gg.integers(0, 255, (slots, kv_heads, HD), dtype=np.uint8)))
    if scales:
        o.update(qs=torch.full((T, heads), -7.0, dtype=torch.float32, device="cuda"),
                 ks=d(gg.uniform(0.1, 1, slots * kv_heads).astype(np.float32)),
                 vs=d(gg.uniform(0.1, 1, slots * kv_heads).astype(np.float32)))
    return o


def assert_same(a, b, keys_bytes=("q8", "kc", "vc"), keys_f32=("qs", "ks", "vs")):
    for k in keys_bytes:
        assert torch.equal(a[k], b[k]), k
    for k in keys_f32:
        if k in a:
            assert torch.equal(a[k].view(torch.int32), b[k].view(torch.int32)), k


@needs_ref
@pytest.mark.parametrize("T,heads,kv_heads,HD,rotary", [(32, 32, 16, 128, 128), (6, 32, 16, 256, 64), (5, 8, 4, 128, 64),
                                                       (4, 4, 4, 512, 128)])
def test_rope_partial_fp8kv_bit_exact_vs_reference_kernel(orc, T, heads, kv_heads, HD, rotary):
    """The reference kernel takes compact Q / K / V buffers; ours is given the packed QKV rows (C launcher)
    and the compact buffers (PTX entry point under the reference's name and 21-argument list)."""
    from rvllm_b200 import launchers
    c = rope_inputs(orc, T, heads, kv_heads, HD, rotary, seed=HD + T)
    qkv = dev16(c["qkv"])
    q_dim, kv_dim = heads * HD, kv_heads * HD
    q_c, k_c, v_c = (qkv[:, :q_dim].contiguous(), qkv[:, q_dim:q_dim + kv_dim].contiguous(),
                     qkv[:, q_dim + kv_dim:].contiguous())
    cos, sin, pos, slot = dev16(c["cos"]), dev16(c["sin"]), d(c["positions"]), d(c["slot_mapping"])
    outs = {}
    for tag, mod in (("ref", H.reference("fused_rope_partial_fp8kv")), ("ours_ptx", H.ours("fused_rope_partial_fp8kv"))):
        o = fresh_outputs(T, heads, kv_heads, HD, c["slots"])
        # geometry of FusedRopePartialFp8KvLaunch::launch (gemma4_launcher.rs:393-394)
        mod.launch("fused_rope_partial_fp8kv_kernel", (T, max(heads, kv_heads)), (max(HD // 2, 32),), 0,
                   [H.P(q_c), H.P(k_c), H.P(v_c), H.P(o["q8"]), H.P(o["kc"]), H.P(o["vc"]), H.P(o["ks"]), H.P(o["vs"]),
                    H.P(o["qs"]), H.P(cos), H.P(sin), H.P(pos), H.P(slot), H.NULL(), H.I(T), H.I(heads), H.I(kv_heads),
                    H.I(HD), H.I(rotary), H.I(c["max_pos"]), H.I(c["slots"])])
        outs[tag] = o
    o = fresh_outputs(T, heads, kv_heads, HD, c["slots"])
    launchers.rope_fp8kv(qkv, heads, kv_heads, HD, rotary, cos, sin, pos, slot, o["q8"], o["qs"], o["kc"], o["vc"],
                         o["ks"], o["vs"])
    outs["ours_abi"] = o
    torch.cuda.synchronize()
    assert_same(outs["ours_ptx"], outs["ref"])
    assert_same(outs["ours_abi"], outs["ref"])
    # static Q scale (no per-head scale cache): q_scale_cache = NULL, scalar from q_scale_ptr
    qsc = torch.tensor([0.037], dtype=torch.float32, device="cuda")
    st = {}
    for tag, mod in (("ref", H.reference("fused_rope_partial_fp8kv")), ("ours", H.ours("fused_rope_partial_fp8kv"))):
        o = fresh_outputs(T, heads, kv_heads, HD, c["slots"])
        mod.launch("fused_rope_partial_fp8kv_kernel", (T, max(heads, kv_heads)), (max(HD // 2, 32),), 0,
                   [H.P(q_c), H.P(k_c), H.P(v_c), H.P(o["q8"]), H.P(o["kc"]), H.P(o["vc"]), H.P(o["ks"]), H.P(o["vs"]),
                    H.NULL(), H.P(cos), H.P(sin), H.P(pos), H.P(slot), H.P(qsc), H.I(T), H.I(heads), H.I(kv_heads),
                    H.I(HD), H.I(rotary), H.I(c["max_pos"]), H.I(c["slots"])])
        st[tag] = o
    torch.cuda.synchronize()
    assert_same(st["ours"], st["ref"])


@needs_ref
@pytest.mark.parametrize("M,heads,kv_heads,K", [(32, 32, 16, 5376), (7, 8, 4, 1024), (128, 32, 16, 5376), (50, 8, 4, 1024)])
def test_fused_qkv_rope_epilogue_bit_exact_vs_gemm_then_reference_rope_kernel(orc, M, heads, kv_heads, K):
    """The QKV GEMM with RoPE + Q quantisation + KV write in its epilogue against: the same GEMM into an
    f16 buffer, then the reference's own RoPE / KV-write kernel."""
    from rvllm_b200 import gemm, launchers
    HD = 128
    N = (heads + 2 * kv_heads) * HD
    g = np.random.default_rng(M + K)
    a, a_s = datagen.quant_rows(orc, g.standard_normal((M, K), dtype=np.float32))
    w, w_s = datagen.quant_rows(orc, g.standard_normal((N, K), dtype=np.float32) * 0.05)
    A, AS, W, WS = d(a), d(a_s), d(w), d(w_s)
    c = rope_inputs(orc, M, heads, kv_heads, HD, HD, seed=M)
    cos, sin, pos, slot = dev16(c["cos"]), dev16(c["sin"]), d(c["positions"]), d(c["slot_mapping"])
    qkv = torch.empty((M, N), dtype=torch.float16, device="cuda")
    gemm.fp8_gemm_channelscale(qkv, A, W, AS, WS, impl=gemm.IMPL_TCGEN05)
    q_dim, kv_dim = heads * HD, kv_heads * HD
    q_c, k_c, v_c = (qkv[:, :q_dim].contiguous(), qkv[:, q_dim:q_dim + kv_dim].contiguous(),
                     qkv[:, q_dim + kv_dim:].contiguous())
    ref = fresh_outputs(M, heads, kv_heads, HD, c["slots"])
    H.reference("fused_rope_partial_fp8kv").launch(
        "fused_rope_partial_fp8kv_kernel", (M, max(heads, kv_heads)), (HD // 2,), 0,
        [H.P(q_c), H.P(k_c), H.P(v_c), H.P(ref["q8"]), H.P(ref["kc"]), H.P(ref["vc"]), H.P(ref["ks"]), H.P(ref["vs"]),
         H.P(ref["qs"]), H.P(cos), H.P(sin), H.P(pos), H.P(slot), H.NULL(), H.I(M), H.I(heads), H.I(kv_heads), H.I(HD),
         H.I(HD), H.I(c["max_pos"]), H.I(c["slots"])])
    got = fresh_outputs(M, heads, kv_heads, HD, c["slots"])
    taken = launchers.qkv_rope_fp8kv(A, W, AS, WS, heads, kv_heads, HD, cos, sin, pos, slot, got["q8"], got["qs"],
                                     got["kc"], got["vc"], got["ks"], got["vs"])
    torch.cuda.synchronize()
    assert taken and gemm.tc_status() == 0
    assert_same(got, ref)


# --------------------------------------------------------------------------- RoPE, Llama interleaved form
@needs_ref
@pytest.mark.parametrize("T,heads,kv_heads,HD", [(32, 32, 8, 128), (5, 8, 4, 256), (3, 4, 4, 512)])
def test_rope_cache_fp8kv_bit_exact_vs_reference_kernel(orc, T, heads, kv_heads, HD):
    from rvllm_b200 import _lib
    c = rope_inputs(orc, T, heads, kv_heads, HD, HD, seed=7 * HD + T)
    qkv = dev16(c["qkv"])
    q_dim, kv_dim = heads * HD, kv_heads * HD
    q_c, k_c, v_c = (qkv[:, :q_dim].contiguous(), qkv[:, q_dim:q_dim + kv_dim].contiguous(),
                     qkv[:, q_dim + kv_dim:].contiguous())
    cos, sin, pos, slot = dev16(c["cos"]), dev16(c["sin"]), d(c["positions"]), d(c["slot_mapping"])
    q_scale, kv_scale = 0.011, 0.017
    qsc = torch.tensor([q_scale], dtype=torch.float32, device="cuda")
    kvsc = torch.tensor([kv_scale], dtype=torch.float32, device="cuda")
    outs = {}
    for tag, mod in (("ref", H.reference("fused_rope_cache_fp8kv")), ("ours_ptx", H.ours("fused_rope_cache_fp8kv"))):
        o = fresh_outputs(T, heads, kv_heads, HD, c["slots"], scales=False)
        # geometry of FusedRopeCacheFp8KvLaunch::launch (launcher.rs:705-709)
        mod.launch("fused_rope_cache_fp8kv_kernel", (T, max(heads, kv_heads)), (max(HD // 2, 32),), 0,
                   [H.P(q_c), H.P(k_c), H.P(v_c), H.P(o["q8"]), H.P(o["kc"]), H.P(o["vc"]), H.P(cos), H.P(sin), H.P(pos),
                    H.P(slot), H.P(qsc), H.P(kvsc), H.I(T), H.I(heads), H.I(kv_heads), H.I(HD), H.I(c["max_pos"]),
                    H.I(c["slots"])])
        outs[tag] = o
    o = fresh_outputs(T, heads, kv_heads, HD, c["slots"], scales=False)
    es = 2
    base = qkv.data_ptr()
    _lib.check(_lib.lib().rvllm_rope_cache_fp8kv_launch(
        base, base + es * q_dim, base + es * (q_dim + kv_dim), c["N"], o["q8"].data_ptr(), o["kc"].data_ptr(),
        o["vc"].data_ptr(), cos.data_ptr(), sin.data_ptr(), pos.data_ptr(), slot.data_ptr(), qsc.data_ptr(),
        kvsc.data_ptr(), T, heads, kv_heads, HD, c["max_pos"], c["slots"], 0, _lib.current_stream()), "rope_cache_fp8kv")
    outs["ours_abi"] = o
    torch.cuda.synchronize()
    assert_same(outs["ours_ptx"], outs["ref"], keys_f32=())
    assert_same(outs["ours_abi"], outs["ref"], keys_f32=())
    # and the CPU restatement: no transcendental on this path, so at most a rounding-boundary byte may differ
    gg = np.random.default_rng(5)
    kc = gg.integers(0, 255, (c["slots"], kv_heads, HD), dtype=np.uint8)
    vc = gg.integers(0, 255, (c["slots"], kv_heads, HD), dtype=np.uint8)
    q8 = np.full((T, heads, HD), 0xAB, np.uint8)
    orc.rope_cache_fp8kv(c["qkv"], heads, kv_heads, HD, c["cos"], c["sin"], c["positions"], c["slot_mapping"], kc, vc,
                         q_scale, kv_scale, 0, q_fp8=q8)
    for got, want in ((outs["ref"]["q8"], q8), (outs["ref"]["kc"], kc), (outs["ref"]["vc"], vc)):
        got = got.cpu().numpy()
        assert H.fp8_codes_adjacent(got, want).all()
        assert (got != want).mean() <= 1e-3


def test_rope_cache_fp8kv_launcher_validation_kats():
    """FusedRopeCacheFp8KvLaunch::validate (launcher.rs:586-616): head_dim in {128, 256, 512}, heads a
    multiple of kv_heads, positive token count."""
    from rvllm_b200 import _lib
    L = _lib.lib()
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    f = torch.ones(4, dtype=torch.float32, device="cuda")
    p, s = t.data_ptr(), _lib.current_stream()

    def call(tokens=2, heads=4, kv=2, hd=128):
        return L.rvllm_rope_cache_fp8kv_launch(p, p, p, 1024, p, p, p, p, p, p, p, f.data_ptr(), f.data_ptr(), tokens,
                                               heads, kv, hd, 16, 8, 0, s)
    assert call() == 0
    assert call(hd=64) == _lib.E_INVALID
    assert call(heads=5, kv=2) == _lib.E_INVALID
    assert call(tokens=0) == _lib.E_INVALID
    torch.cuda.synchronize()


# --------------------------------------------------------------------------- Gemma-4 decorations
@needs_ref
@pytest.mark.parametrize("T,heads,kv_heads,HD", [(32, 32, 16, 128), (3, 32, 16, 256), (2, 8, 4, 512), (5, 4, 2, 96)])
def test_fused_qkv_rmsnorm_bit_exact_vs_reference_kernel(orc, T, heads, kv_heads, HD):
    from rvllm_b200 import _lib
    g = np.random.default_rng(HD + T)
    stride = (heads + 2 * kv_heads) * HD + 64          # a row stride wider than the packed QKV row
    qkv_b = orc.to_bits16((g.standard_normal((T, stride)) * 2.0).astype(np.float32), 0)
    qg_b = orc.to_bits16((1 + 0.2 * g.standard_normal(HD)).astype(np.float32), 0)
    kg_b = orc.to_bits16((1 + 0.2 * g.standard_normal(HD)).astype(np.float32), 0)
    qkv, qg, kg = dev16(qkv_b), dev16(qg_b), dev16(kg_b)
    q_dim, kv_dim = heads * HD, kv_heads * HD
    es = 2
    base = qkv.data_ptr()
    outs = {}
    block = min(HD, 1024)
    for tag, mod in (("ref", H.reference("fused_qkv_rmsnorm")), ("ours_ptx", H.ours("fused_qkv_rmsnorm"))):
        o = [torch.zeros((T, n, HD), dtype=torch.float16, device="cuda") for n in (heads, kv_heads, kv_heads)]
        # geometry of FusedQkvRmsnormLaunch::launch (gemma4_launcher.rs:237-238)
        mod.launch("fused_qkv_rmsnorm_kernel", (T, heads + 2 * kv_heads), (block,), 0,
                   [(H.ctypes.c_void_p, base), (H.ctypes.c_void_p, base + es * q_dim),
                    (H.ctypes.c_void_p, base + es * (q_dim + kv_dim)), H.P(o[0]), H.P(o[1]), H.P(o[2]), H.P(qg), H.P(kg),
                    H.I(T), H.I(heads), H.I(kv_heads), H.I(HD), H.F(1e-6), H.I(stride)])
        outs[tag] = o
    o = [torch.zeros((T, n, HD), dtype=torch.float16, device="cuda") for n in (heads, kv_heads, kv_heads)]
    _lib.check(_lib.lib().rvllm_fused_qkv_rmsnorm_launch(base, base + es * q_dim, base + es * (q_dim + kv_dim),
                                                         o[0].data_ptr(), o[1].data_ptr(), o[2].data_ptr(), qg.data_ptr(),
                                                         kg.data_ptr(), T, heads, kv_heads, HD, 1e-6, stride, 0,
                                                         _lib.current_stream()), "fused_qkv_rmsnorm")
    outs["ours_abi"] = o
    torch.cuda.synchronize()
    for tag in ("ours_ptx", "ours_abi"):
        for a, b in zip(outs[tag], outs["ref"]):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16)), tag
    # against the CPU restatement: rsqrtf is not correctly rounded on the device, so a 16-bit result may sit
    # one unit in the last place away
    wq, wk, wv = orc.qkv_rmsnorm(qkv_b, qg_b, kg_b, heads, kv_heads, HD, 1e-6, 0, block_dim=max(32, block // 32 * 32))
    for got, want in zip(outs["ref"], (wq, wk, wv)):
        gb = bits(got).astype(np.int32)
        assert np.abs(gb - want.astype(np.int32)).max() <= 1
        assert (gb != want).mean() <= 0.02


@needs_ref
@pytest.mark.parametrize("T,hidden", [(32, 5376), (3, 1536), (2, 10240)])
@pytest.mark.parametrize("scalar", [None, 0.75])
def test_norm_add_residual_bit_exact_vs_reference_kernels(orc, T, hidden, scalar):
    from rvllm_b200 import _lib
    g = np.random.default_rng(hidden + T)
    x32 = (g.standard_normal((T, hidden)) * 30).astype(np.float32)
    cs = g.uniform(0.01, 0.05, hidden).astype(np.float32)
    x16_b = orc.to_bits16(x32 * cs, 0)
    gamma_b = orc.to_bits16((1 + 0.2 * g.standard_normal(hidden)).astype(np.float32), 0)
    res_b = orc.to_bits16(g.standard_normal((T, hidden)).astype(np.float32), 0)
    ls_b = None if scalar is None else orc.to_bits16(np.array([scalar], np.float32), 0)
    X32, CS, X16, G = d(x32), d(cs), dev16(x16_b), dev16(gamma_b)
    LS = None if ls_b is None else dev16(ls_b)
    lsp = H.NULL() if LS is None else H.P(LS)
    block = min(hidden, 1024)
    out = {}
    for tag, mod in (("ref", H.reference("fused_norm_add_residual_f16")), ("ours", H.ours("fused_norm_add_residual_f16"))):
        r1, r2 = dev16(res_b), dev16(res_b)
        # geometry of FusedNormAddResidualF16Launch::launch (gemma4_launcher.rs:817-820): dynamic smem = hidden * 4
        mod.launch("fused_norm_add_residual_f16_kernel", (T,), (block,), hidden * 4,
                   [H.P(X32), H.P(CS), H.P(G), H.P(r1), lsp, H.I(hidden), H.F(1e-6)])
        mod.launch("fused_norm_add_residual_f16in_kernel", (T,), (block,), hidden * 4,
                   [H.P(X16), H.P(G), H.P(r2), lsp, H.I(hidden), H.F(1e-6)])
        out[tag] = (r1, r2)
    r1, r2 = dev16(res_b), dev16(res_b)
    L, s = _lib.lib(), _lib.current_stream()
    lp = None if LS is None else LS.data_ptr()
    _lib.check(L.rvllm_fused_norm_add_residual_launch(X32.data_ptr(), 1, CS.data_ptr(), G.data_ptr(), r1.data_ptr(), lp, T,
                                                      hidden, 1e-6, 0, s), "norm_add_residual f32")
    _lib.check(L.rvllm_fused_norm_add_residual_launch(X16.data_ptr(), 0, None, G.data_ptr(), r2.data_ptr(), lp, T, hidden,
                                                      1e-6, 0, s), "norm_add_residual 16")
    torch.cuda.synchronize()
    for got in (out["ours"], (r1, r2)):
        for a, b in zip(got, out["ref"]):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    want1 = orc.norm_add_residual(res_b, x32, gamma_b, 1e-6, channelscale=cs, layer_scalar16=ls_b, dtype=0,
                                  block_dim=max(32, block // 32 * 32))
    want2 = orc.norm_add_residual(res_b, x16_b, gamma_b, 1e-6, layer_scalar16=ls_b, dtype=0,
                                  block_dim=max(32, block // 32 * 32))
    for got, want in zip(out["ref"], (want1, want2)):
        gf, wf = orc.from_bits16(bits(got), 0), orc.from_bits16(want, 0)
        assert np.abs(gf - wf).max() <= 2e-3 * np.abs(wf).max()
        assert (bits(got) != want).mean() <= 0.02


@needs_ref
def test_residual_scale_and_logit_softcap_bit_exact_vs_reference_kernels(orc):
    from rvllm_b200 import _lib
    L, s = _lib.lib(), _lib.current_stream()
    g = np.random.default_rng(3)
    T, hidden, vocab = 7, 5376, 262144
    res_b = orc.to_bits16(g.standard_normal((T, hidden)).astype(np.float32), 0)
    sc_b = orc.to_bits16(np.array([0.3125], np.float32), 0)
    lg_b = orc.to_bits16((g.standard_normal((2, vocab)) * 25).astype(np.float32), 0)
    SC = dev16(sc_b)
    got = {}
    for tag, rs, sm in (("ref", H.reference("residual_scale_f16"), H.reference("logit_softcap")),
                        ("ours", H.ours("residual_scale_f16"), H.ours("logit_softcap"))):
        r, lg = dev16(res_b), dev16(lg_b)
        rs.launch("residual_scale_f16_kernel", (T,), (min(hidden, 1024),), 0, [H.P(r), H.P(SC), H.I(hidden)])
        sm.launch("logit_softcap_kernel", (2,), (min(vocab, 1024),), 0, [H.P(lg), H.I(vocab), H.F(30.0)])
        got[tag] = (r, lg)
    r, lg = dev16(res_b), dev16(lg_b)
    _lib.check(L.rvllm_residual_scale_launch(r.data_ptr(), SC.data_ptr(), T, hidden, 0, s), "residual_scale")
    _lib.check(L.rvllm_logit_softcap_launch(lg.data_ptr(), 2, vocab, 30.0, 0, s), "logit_softcap")
    torch.cuda.synchronize()
    for cand in (got["ours"], (r, lg)):
        for a, b in zip(cand, got["ref"]):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert np.array_equal(bits(got["ref"][0]), orc.residual_scale(res_b, sc_b, 0))     # exact: one multiply, one rounding
    want = orc.logit_softcap(lg_b, 30.0, 0)
    gb = bits(got["ref"][1]).astype(np.int32)
    assert np.abs(gb - want.astype(np.int32)).max() <= 1                                 # device tanhf vs libm tanhf
    assert L.rvllm_logit_softcap_launch(lg.data_ptr(), 2, vocab, 0.0, 0, s) == _lib.E_INVALID   # cap must be > 0
    assert L.rvllm_logit_softcap_launch(lg.data_ptr(), 0, vocab, 30.0, 0, s) == _lib.E_INVALID  # zero dim


@needs_ref
@pytest.mark.parametrize("M,N,K", [(1, 5376, 4096), (4, 1000, 5376), (2, 8192, 21504)])
def test_blockscale_gemv_bit_exact_vs_reference_kernel(orc, M, N, K):
    """FP8 weights with 128 x 128 block scales x f16 activations: the reference's warp-per-row kernel
    (kernels/fp8_gemv.cu:811-891) against this repository's entry point of the same name and its C launcher."""
    from rvllm_b200 import _lib
    g = np.random.default_rng(N + K)
    w = g.integers(0, 256, (N, K), dtype=np.uint8)
    w[(w & 0x7F) == 0x7F] ^= 1                                     # no NaN codes
    ncb = (K + 127) // 128
    sc = g.uniform(0.002, 0.02, ((N + 127) // 128, ncb)).astype(np.float32)
    x_b = orc.to_bits16(g.standard_normal((M, K)).astype(np.float32), 0)
    W, SC, X = d(w), d(sc), dev16(x_b)
    outs = {}
    for tag, mod in (("ref", H.reference("fp8_gemv")), ("ours", H.ours("fp8_gemv"))):
        o = torch.zeros((M, N), dtype=torch.float16, device="cuda")
        # geometry of Fp8GemvF16InLaunch::launch (gemma4_launcher.rs:882-883)
        mod.launch("fp8_gemv_blockwise_wpr_native_f16in_kernel", ((N + 7) // 8, M), (256,), 0,
                   [H.P(o), H.P(W), H.P(SC), H.P(X), H.I(M), H.I(N), H.I(K), H.I(ncb)])
        outs[tag] = o
    o = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    _lib.check(_lib.lib().rvllm_fp8_gemv_blockscale_launch(o.data_ptr(), W.data_ptr(), SC.data_ptr(), X.data_ptr(), M, N, K, 0,
                                                           _lib.current_stream()), "fp8_gemv_blockscale")
    torch.cuda.synchronize()
    assert torch.equal(outs["ours"].view(torch.int16), outs["ref"].view(torch.int16))
    assert torch.equal(o.view(torch.int16), outs["ref"].view(torch.int16))
    want = orc.fp8_gemv_blockscale(w, sc, x_b, 0)
    gb = bits(outs["ref"]).astype(np.int32)
    assert np.abs(gb - want.astype(np.int32)).max() <= 1 and (gb != want).mean() <= 0.01
