"""GPU parity of the fused row kernels (RMSNorm-quant, per-token quant, act-mul-quant,
argmax, FP8 encode) through the C ABI, against the CPU oracle and — bit for bit — against
the reference's own CUDA kernels compiled under oracle/_ref.

Bit-exactness protocol: the encoder itself and argmax must match exactly.  For the row
kernels the CPU oracle differs from any GPU in two library functions (rsqrtf, expf/tanhf
are not correctly rounded on the device), so against the oracle a scale may differ in the
last place and a byte may land on the neighbouring code for values that sit on a rounding
boundary; against the reference kernel run on the same GPU every scale and byte must be
identical.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from tests import ptx_harness as H  # noqa: E402


def dev16(bits, dtype):
    t = torch.from_numpy(bits.view(np.int16).copy()).cuda()
    return t.view(torch.float16 if dtype == 0 else torch.bfloat16)


def rand16(orc, shape, dtype, seed, scale=1.0):
    g = np.random.default_rng(seed)
    return orc.to_bits16((g.standard_normal(shape) * scale).astype(np.float32), dtype)


def assert_quant_close(orc, got_bytes, got_scale, want_bytes, want_scale, max_frac=2e-3):
    np.testing.assert_allclose(got_scale, want_scale, rtol=4e-7, atol=0)
    neq = got_bytes != want_bytes
    assert H.fp8_codes_adjacent(got_bytes, want_bytes).all(), "a byte is more than one code away from the oracle"
    assert neq.mean() <= max_frac, f"{neq.mean():.2e} of bytes differ from the oracle"


# --------------------------------------------------------------------------- encoder
def test_fp8_encode_exhaustive_bit_exact(orc):
    from rvllm_b200 import _lib
    # every f32 whose low 16 mantissa bits are zero, plus every rounding tie and its neighbours
    hi = (np.arange(1 << 16, dtype=np.uint32) << 16).view(np.float32)
    codes = orc.e4m3_decode(np.arange(0x7F, dtype=np.uint8))
    mids = (codes[:-1] + codes[1:]) / 2
    ties = np.concatenate([mids, np.nextafter(mids, np.float32(1e9)), np.nextafter(mids, np.float32(-1e9))])
    g = np.random.default_rng(0)
    rnd = (g.standard_normal(1 << 18) * np.exp(g.uniform(-12, 7, 1 << 18))).astype(np.float32)
    x = np.concatenate([hi, ties, -ties, rnd]).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    out = torch.empty(x.size, dtype=torch.uint8, device="cuda")
    _lib.check(_lib.lib().rvllm_e4m3_encode_f32(out.data_ptr(), xd.data_ptr(), x.size, _lib.current_stream()), "encode")
    got = out.cpu().numpy()
    want = orc.e4m3_encode(x, orc.MODE_CUDA)
    assert np.array_equal(got, want)
    rust = orc.e4m3_encode(x, orc.MODE_RUST)
    assert np.all(got[rust != got] == 0x80)  # the Rust host encoder only canonicalises -0


def test_fp8_decode_all_codes(orc):
    from rvllm_b200 import _lib
    c = torch.arange(256, dtype=torch.uint8, device="cuda")
    out = torch.empty(256, dtype=torch.float32, device="cuda")
    _lib.check(_lib.lib().rvllm_e4m3_decode_f32(out.data_ptr(), c.data_ptr(), 256, _lib.current_stream()), "decode")
    got, want = out.cpu().numpy(), orc.e4m3_decode(np.arange(256, dtype=np.uint8))
    ok = ~np.isnan(want)
    assert np.array_equal(got[ok], want[ok])  # by value: the hardware convert keeps the sign of -0
    assert np.isnan(got[~ok]).all()


# --------------------------------------------------------------------------- stage 1
@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("tokens,hidden", [(4, 512), (1, 5376), (32, 5376), (3, 3584), (2, 16392), (5, 72)])
def test_rmsnorm_quant_vs_oracle(orc, dtype, tokens, hidden):
    from rvllm_b200.launchers import FusedRmsnormFp8QuantLaunch
    x = rand16(orc, (tokens, hidden), dtype, 10 + hidden)
    gamma = orc.to_bits16((1.0 + 0.1 * np.random.default_rng(3).standard_normal(hidden)).astype(np.float32), dtype)
    out = torch.empty((tokens, hidden), dtype=torch.uint8, device="cuda")
    scale = torch.empty(tokens, dtype=torch.float32, device="cuda")
    FusedRmsnormFp8QuantLaunch(tokens, hidden, 1e-6).launch(out, scale, dev16(x, dtype), dev16(gamma, dtype))
    wb, ws = orc.rmsnorm_fp8_quant(x, gamma, 1e-6, dtype, orc.MODE_CUDA, block_dim=max(32, min(hidden, 1024) // 32 * 32))
    assert_quant_close(orc, out.cpu().numpy(), scale.cpu().numpy(), wb, ws)


@pytest.mark.parametrize("dtype", [0, 1])
def test_add_rmsnorm_quant_vs_oracle(orc, dtype):
    from rvllm_b200.launchers import FusedAddRmsnormFp8QuantLaunch
    tokens, hidden = 6, 5376
    x = rand16(orc, (tokens, hidden), dtype, 1)
    r = rand16(orc, (tokens, hidden), dtype, 2, 3.0)
    gamma = rand16(orc, (hidden,), dtype, 3)
    out = torch.empty((tokens, hidden), dtype=torch.uint8, device="cuda")
    scale = torch.empty(tokens, dtype=torch.float32, device="cuda")
    res_out = torch.empty((tokens, hidden), dtype=torch.int16, device="cuda")
    FusedAddRmsnormFp8QuantLaunch(tokens, hidden, 1e-5).launch(out, scale, res_out, dev16(x, dtype), dev16(r, dtype),
                                                               dev16(gamma, dtype))
    wb, ws, wr = orc.rmsnorm_fp8_quant(x, gamma, 1e-5, dtype, orc.MODE_CUDA, block_dim=1024, residual16=r)
    assert np.array_equal(res_out.cpu().numpy().view(np.uint16), wr)  # rounded sum is exact
    assert_quant_close(orc, out.cpu().numpy(), scale.cpu().numpy(), wb, ws)


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("tokens,dim", [(4, 512), (32, 4096), (2, 8192), (1, 65536), (3, 264)])
def test_quantize_per_token_bit_exact(orc, dtype, tokens, dim):
    # no transcendental involved: bytes and scales must equal the oracle exactly
    from rvllm_b200.launchers import QuantizeFp8PerTokenLaunch
    x = rand16(orc, (tokens, dim), dtype, dim, 2.5)
    x[0, :8] = 0  # exact zeros and a negative zero
    x[0, 1] = 0x8000
    out = torch.empty((tokens, dim), dtype=torch.uint8, device="cuda")
    scale = torch.empty(tokens, dtype=torch.float32, device="cuda")
    QuantizeFp8PerTokenLaunch(tokens, dim).launch(out, scale, dev16(x, dtype))
    wb, ws = orc.quantize_fp8_per_token(x, dtype, orc.MODE_CUDA)
    assert np.array_equal(scale.cpu().numpy().view(np.uint32), ws.view(np.uint32))
    assert np.array_equal(out.cpu().numpy(), wb)


def test_quantize_all_zero_row(orc):
    from rvllm_b200.launchers import QuantizeFp8PerTokenLaunch
    x = torch.zeros((2, 64), dtype=torch.float16, device="cuda")
    out = torch.full((2, 64), 7, dtype=torch.uint8, device="cuda")
    scale = torch.empty(2, dtype=torch.float32, device="cuda")
    QuantizeFp8PerTokenLaunch(2, 64).launch(out, scale, x)
    assert (out == 0).all() and np.allclose(scale.cpu().numpy(), 1e-12)


# --------------------------------------------------------------------------- stage 2c
@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("tokens,inter", [(4, 2048), (32, 21504), (1, 40960), (2, 72)])
def test_act_mul_quant_vs_oracle(orc, dtype, act, tokens, inter):
    from rvllm_b200.launchers import FusedActMulFp8QuantLaunch
    gu = rand16(orc, (tokens, 2 * inter), dtype, inter + act, 2.0)
    out = torch.empty((tokens, inter), dtype=torch.uint8, device="cuda")
    scale = torch.empty(tokens, dtype=torch.float32, device="cuda")
    FusedActMulFp8QuantLaunch(tokens, inter, act).launch(out, scale, dev16(gu, dtype))
    wb, ws = orc.act_mul_fp8_quant(gu, act, dtype, orc.MODE_CUDA)
    assert_quant_close(orc, out.cpu().numpy(), scale.cpu().numpy(), wb, ws, max_frac=5e-3)


def test_act_mul_quant_nonfinite_row_gives_nan_scale(orc):
    from rvllm_b200.launchers import FusedActMulFp8QuantLaunch
    gu = torch.ones((2, 128), dtype=torch.float16, device="cuda")
    gu[1, 3] = float("inf")
    out = torch.empty((2, 64), dtype=torch.uint8, device="cuda")
    scale = torch.empty(2, dtype=torch.float32, device="cuda")
    FusedActMulFp8QuantLaunch(2, 64, 0).launch(out, scale, gu)
    s = scale.cpu().numpy()
    assert np.isfinite(s[0]) and np.isnan(s[1])


# --------------------------------------------------------------------------- stage 4
@pytest.mark.parametrize("grid", [False, True])
@pytest.mark.parametrize("tokens,vocab", [(4, 2048), (32, 262144), (1, 262144), (3, 1000), (2, 5), (5, 32770), (3, 40001)])
def test_argmax_exact(orc, grid, tokens, vocab):
    from rvllm_b200.launchers import ArgmaxLaunch
    g = np.random.default_rng(vocab + tokens)
    x = g.standard_normal((tokens, vocab)).astype(np.float32)
    # injected ties (first must win), NaNs, and -inf
    x[0, vocab // 2] = x[0].max() + 1
    x[0, vocab - 1] = x[0, vocab // 2]
    if tokens > 1:
        x[1, ::3] = np.nan
        x[1, 1] = x[1, 4] = 50.0
    if tokens > 2:
        x[2, :] = -np.inf
    xd = torch.from_numpy(x).cuda()
    out = torch.full((tokens,), -7, dtype=torch.int32, device="cuda")
    ArgmaxLaunch(tokens, vocab).launch(xd, out, grid=grid)
    want = orc.argmax_f32(x, orc.MODE_CUDA)
    assert out.cpu().numpy().tolist() == want.tolist()
    finite_rows = np.isfinite(x).all(axis=1)
    if finite_rows.any():
        rust = orc.argmax_f32(x[finite_rows], orc.MODE_RUST)
        assert out.cpu().numpy()[finite_rows].tolist() == rust.tolist()


def test_argmax_all_nan_row(orc):
    from rvllm_b200.launchers import ArgmaxLaunch
    x = torch.full((2, 4096), float("nan"), device="cuda")
    x[1, 77] = -3.0
    out = torch.zeros(2, dtype=torch.int32, device="cuda")
    ArgmaxLaunch(2, 4096).launch(x, out)
    assert out.cpu().numpy().tolist() == [-1, 77]


def test_argmax_long_rows_edge_candidates(orc):
    """Rows long enough for the launcher to spread each over a cluster: no candidate at all, a single
    candidate in the last element, and a tie between the first and the last slice."""
    from rvllm_b200.launchers import ArgmaxLaunch
    vocab = 65538
    x = np.full((4, vocab), np.nan, np.float32)
    x[1, vocab - 1] = -np.inf
    x[2, :] = -1.0
    x[2, 3] = x[2, vocab - 2] = 9.0
    x[3, :] = 0.0
    out = torch.full((4,), -7, dtype=torch.int32, device="cuda")
    ArgmaxLaunch(4, vocab).launch(torch.from_numpy(x).cuda(), out)
    assert out.cpu().numpy().tolist() == [-1, vocab - 1, 3, 0] == orc.argmax_f32(x, orc.MODE_CUDA).tolist()


# --------------------------------------------------------------------------- reference kernels, same GPU
needs_ref = pytest.mark.skipif(not H.have_reference(), reason="oracle/_ref not built (needs the reference checkout)")


@needs_ref
@pytest.mark.parametrize("tokens,hidden", [(4, 512), (32, 5376), (2, 3584)])
def test_rmsnorm_quant_bit_exact_vs_reference_kernel(orc, tokens, hidden):
    x = dev16(rand16(orc, (tokens, hidden), 0, hidden), 0)
    gamma = dev16(rand16(orc, (hidden,), 0, 5), 0)
    res = {}
    for tag, mod in (("ref", H.reference("fused_rmsnorm_fp8_quant")), ("ours", H.ours("fused_rmsnorm_fp8_quant"))):
        out = torch.empty((tokens, hidden), dtype=torch.uint8, device="cuda")
        scale = torch.empty(tokens, dtype=torch.float32, device="cuda")
        # geometry of FusedRmsnormFp8QuantLaunch::launch (launcher.rs:218-221)
        mod.launch("fused_rmsnorm_fp8_quant_kernel", (tokens,), (min(hidden, 1024),), 128,
                   [H.P(out), H.P(scale), H.P(x), H.P(gamma), H.F(1e-6), H.I(hidden)])
        torch.cuda.synchronize()
        res[tag] = (out.cpu().numpy(), scale.cpu().numpy())
    assert np.array_equal(res["ours"][1].view(np.uint32), res["ref"][1].view(np.uint32))
    assert np.array_equal(res["ours"][0], res["ref"][0])


@needs_ref
def test_quantize_and_add_variant_bit_exact_vs_reference_kernel(orc):
    tokens, dim = 8, 4096
    x = dev16(rand16(orc, (tokens, dim), 0, 1), 0)
    r = dev16(rand16(orc, (tokens, dim), 0, 2), 0)
    gamma = dev16(rand16(orc, (dim,), 0, 3), 0)
    got = {}
    for tag, mod in (("ref", H.reference("fused_rmsnorm_fp8_quant")), ("ours", H.ours("fused_rmsnorm_fp8_quant"))):
        out = torch.empty((tokens, dim), dtype=torch.uint8, device="cuda")
        scale = torch.empty(tokens, dtype=torch.float32, device="cuda")
        mod.launch("quantize_fp8_per_token_kernel", (tokens,), (max(256, min(dim, 1024)),), 128,
                   [H.P(out), H.P(scale), H.P(x), H.I(dim)])
        out2 = torch.empty_like(out)
        scale2 = torch.empty_like(scale)
        ro = torch.empty_like(x)
        mod.launch("fused_add_rmsnorm_fp8_quant_kernel", (tokens,), (min(dim, 1024),), 128,
                   [H.P(out2), H.P(scale2), H.P(ro), H.P(x), H.P(r), H.P(gamma), H.F(1e-6), H.I(dim)])
        torch.cuda.synchronize()
        got[tag] = [t.cpu().numpy().view(np.uint8) for t in (out, scale.view(torch.uint8), out2, scale2.view(torch.uint8), ro.view(torch.uint8))]
    for a, b in zip(got["ours"], got["ref"]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("dtype,suffix", [(0, "_kernel"), (1, "_bf16_kernel")])
@pytest.mark.parametrize("act,stem,sym", [(0, "fused_silu_fp8_quant", "fused_silu_mul_fp8_quant"),
                                          (1, "fused_gelu_mul_fp8_quant", "fused_gelu_mul_fp8_quant")])
@pytest.mark.parametrize("tokens,inter", [(32, 21504), (3, 73728), (64, 21504), (96, 21504), (80, 40960),
                                          (130, 4096), (300, 8200)])
def test_act_mul_quant_cluster_launch_equals_one_cta_per_row(orc, dtype, suffix, act, stem, sym, tokens, inter):
    """The C launcher spreads each row of a small batch over a cluster of CTAs; the PTX entry point
    keeps the reference geometry of one CTA per row.  Bytes and scale bits must be identical,
    including a row with a non-finite product (NaN scale)."""
    from rvllm_b200.launchers import FusedActMulFp8QuantLaunch
    gu_np = rand16(orc, (tokens, 2 * inter), dtype, 31 + inter, 2.0)
    gu = dev16(gu_np, dtype)
    gu[tokens - 1, inter + 5] = float("inf")
    out_a = torch.empty((tokens, inter), dtype=torch.uint8, device="cuda")
    scale_a = torch.empty(tokens, dtype=torch.float32, device="cuda")
    FusedActMulFp8QuantLaunch(tokens, inter, act).launch(out_a, scale_a, gu)
    out_b = torch.empty_like(out_a)
    scale_b = torch.empty_like(scale_a)
    H.ours(stem).launch(sym + suffix, (tokens,), (min(inter - inter % 32, 1024),), 128,
                        [H.P(out_b), H.P(scale_b), H.P(gu), H.I(inter)])
    torch.cuda.synchronize()
    sa, sb = scale_a.cpu().numpy(), scale_b.cpu().numpy()
    assert np.isnan(sa[-1]) and np.isnan(sb[-1])
    assert np.array_equal(sa[:-1].view(np.uint32), sb[:-1].view(np.uint32))
    assert np.array_equal(out_a.cpu().numpy()[:-1], out_b.cpu().numpy()[:-1])


@needs_ref
@pytest.mark.parametrize("stem,sym", [("fused_silu_fp8_quant", "fused_silu_mul_fp8_quant_kernel"),
                                      ("fused_gelu_mul_fp8_quant", "fused_gelu_mul_fp8_quant_kernel")])
def test_act_mul_quant_bit_exact_vs_reference_kernel(orc, stem, sym):
    tokens, inter = 16, 21504
    gu = dev16(rand16(orc, (tokens, 2 * inter), 0, 9, 2.0), 0)
    got = {}
    for tag, mod in (("ref", H.reference(stem)), ("ours", H.ours(stem))):
        out = torch.empty((tokens, inter), dtype=torch.uint8, device="cuda")
        scale = torch.empty(tokens, dtype=torch.float32, device="cuda")
        mod.launch(sym, (tokens,), (min(inter, 1024),), 128, [H.P(out), H.P(scale), H.P(gu), H.I(inter)])
        torch.cuda.synchronize()
        got[tag] = (out.cpu().numpy(), scale.cpu().numpy())
    assert np.array_equal(got["ours"][1].view(np.uint32), got["ref"][1].view(np.uint32))
    assert np.array_equal(got["ours"][0], got["ref"][0])


@needs_ref
@pytest.mark.parametrize("sym,grid_variant", [("argmax_kernel", False), ("argmax_grid_f32_kernel", True)])
def test_argmax_matches_reference_kernel(orc, sym, grid_variant):
    tokens, vocab = 8, 262144
    g = np.random.default_rng(4)
    x = g.standard_normal((tokens, vocab)).astype(np.float32)
    x[0, 5] = x[0, 99999] = 100.0
    x[1, ::2] = np.nan
    xd = torch.from_numpy(x).cuda()
    got = {}
    for tag, mod in (("ref", H.reference("argmax")), ("ours", H.ours("argmax"))):
        out = torch.zeros(tokens, dtype=torch.int32, device="cuda")  # the launcher's cuMemsetD32Async(out, 0)
        if grid_variant:
            mod.launch(sym, ((vocab + 1023) // 1024, tokens), (256,), 0, [H.P(xd), H.P(out), H.I(vocab)])
        else:
            mod.launch(sym, (tokens,), (min(vocab, 1024),), 0, [H.P(xd), H.P(out), H.I(vocab)])
        torch.cuda.synchronize()
        got[tag] = out.cpu().numpy()
    assert got["ours"].tolist() == got["ref"].tolist() == orc.argmax_f32(x, orc.MODE_CUDA).tolist()


def test_manifest_loader_launch_raw_matches_c_abi(orc):
    """The verified PTX bundle, loaded and launched through the library's own manifest loader
    (the KernelLoader::load_ptx -> launch_raw path), gives the bytes the C-ABI launcher gives."""
    import ctypes as C
    import os
    from rvllm_b200 import build
    from rvllm_b200.launchers import FusedRmsnormFp8QuantLaunch
    from rvllm_b200.manifest import VerifiedManifest
    kdir = os.path.join(os.path.dirname(build.LIB), "kernels", "sm_100")
    digest = open(os.path.join(kdir, "manifest.sha256")).read().split()[0]
    vm = VerifiedManifest(os.path.join(kdir, "manifest.json"), digest, build.REVISION, "sm_100")
    mod = vm.load_ptx("fused_rmsnorm_fp8_quant")
    tokens, hidden = 7, 5376
    x = dev16(rand16(orc, (tokens, hidden), 1, 77), 1)
    gamma = dev16(rand16(orc, (hidden,), 1, 78), 1)
    out = [torch.empty((tokens, hidden), dtype=torch.uint8, device="cuda") for _ in range(2)]
    sc = [torch.empty(tokens, dtype=torch.float32, device="cuda") for _ in range(2)]
    vp = C.c_void_p
    mod.launch_raw("fused_rmsnorm_fp8_quant_bf16_kernel", (tokens,), (1024,), 128,
                   [(vp, out[0].data_ptr()), (vp, sc[0].data_ptr()), (vp, x.data_ptr()), (vp, gamma.data_ptr()),
                    (C.c_float, 1e-6), (C.c_int, hidden)])
    FusedRmsnormFp8QuantLaunch(tokens, hidden, 1e-6).launch(out[1], sc[1], x, gamma)
    torch.cuda.synchronize()
    assert torch.equal(out[0], out[1]) and torch.equal(sc[0], sc[1])
    from rvllm_b200 import RvllmError
    with pytest.raises(RvllmError):
        mod.function("no_such_kernel")
    with pytest.raises(RvllmError):
        mod.launch_raw("fused_rmsnorm_fp8_quant_bf16_kernel", (tokens,), (2048,), 0, [])
    mod.close()


# --------------------------------------------------------------------------- rope + paged KV write
@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary", [(32, 16, 128, 128), (32, 16, 256, 64), (8, 4, 64, 64),
                                                           (4, 4, 512, 128)])
def test_rope_fp8kv_matches_oracle(orc, dtype, heads, kv_heads, head_dim, rotary):
    """RoPE + Q quantisation + paged FP8 KV write against the CPU oracle: Q bytes and scales, and
    the K/V cache bytes and per-slot scales, including a token whose slot is out of range (no
    cache write), a position out of range (nothing written for that token) and a non-finite K
    element (NaN scale for that slot and head only)."""
    from rvllm_b200 import launchers
    T, slots, max_pos = 6, 40, 64
    g = np.random.default_rng(head_dim + heads + dtype)
    width = (heads + 2 * kv_heads) * head_dim
    qkv_f = (g.standard_normal((T, width)) * 1.5).astype(np.float32)
    qkv_f[2, heads * head_dim + head_dim + 3] = np.inf            # K head 1 of token 2
    qkv = orc.to_bits16(qkv_f, dtype)
    ang = g.uniform(0, 6.28, (max_pos, rotary // 2)).astype(np.float32)
    cos, sin = orc.to_bits16(np.cos(ang), dtype), orc.to_bits16(np.sin(ang), dtype)
    positions = np.array([0, 5, 63, 7, 64, 9], np.int32)          # token 4: position out of range
    slot_mapping = np.array([3, 39, 17, -1, 8, 21], np.int32)      # token 3: no cache slot
    kc0 = g.integers(0, 255, (slots, kv_heads, head_dim), dtype=np.uint8)
    vc0 = g.integers(0, 255, (slots, kv_heads, head_dim), dtype=np.uint8)
    ks0 = g.uniform(0.1, 1, slots * kv_heads).astype(np.float32)
    vs0 = g.uniform(0.1, 1, slots * kv_heads).astype(np.float32)
    kc, vc, ks, vs = kc0.copy(), vc0.copy(), ks0.copy(), vs0.copy()
    want_q, want_qs = orc.rope_fp8kv(qkv, heads, kv_heads, head_dim, rotary, cos, sin, positions, slot_mapping,
                                     kc, vc, ks, vs, dtype)
    d = lambda a: torch.from_numpy(a.copy()).cuda()
    q8 = torch.full((T, heads, head_dim), 0xAB, dtype=torch.uint8, device="cuda")
    qs = torch.full((T, heads), -7.0, dtype=torch.float32, device="cuda")
    dkc, dvc, dks, dvs = d(kc0), d(vc0), d(ks0), d(vs0)
    launchers.rope_fp8kv(dev16(qkv, dtype), heads, kv_heads, head_dim, rotary, dev16(cos, dtype), dev16(sin, dtype),
                         d(positions), d(slot_mapping), q8, qs, dkc, dvc, dks, dvs)
    torch.cuda.synchronize()
    live = positions < max_pos                                     # rows the kernel may write
    got_q, got_qs = q8.cpu().numpy(), qs.cpu().numpy()
    assert (got_q[~live] == 0xAB).all() and (got_qs[~live] == -7.0).all()
    np.testing.assert_array_equal(got_qs[live].view(np.uint32), want_qs[live].view(np.uint32))
    np.testing.assert_array_equal(got_q[live], want_q[live])
    got_k, got_v = dkc.cpu().numpy(), dvc.cpu().numpy()
    # the row quantised with a NaN scale holds NaN codes (0x7f or 0xff: the sign of a NaN is not defined)
    assert ((got_k[17, 1] & 0x7F) == 0x7F).all() and ((kc[17, 1] & 0x7F) == 0x7F).all()
    got_k[17, 1] = kc[17, 1]
    np.testing.assert_array_equal(got_k, kc)
    np.testing.assert_array_equal(got_v, vc)
    for got, want in ((dks, ks), (dvs, vs)):
        got = got.cpu().numpy()
        assert np.array_equal(np.isnan(got), np.isnan(want))       # NaN payloads differ between C and CUDA
        fin = ~np.isnan(want)
        np.testing.assert_array_equal(got[fin].view(np.uint32), want[fin].view(np.uint32))
    assert np.isnan(ks[17 * kv_heads + 1]) and not np.isnan(vs[17 * kv_heads + 1])
