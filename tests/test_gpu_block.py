"""The layer-block kernel (O projection -> RMSNorm+quant -> gate|up -> act*up+quant -> down -> RMSNorm+quant in one
launch, CTAs resident across the stages behind grid-wide barriers) against the chain of stand-alone kernels it
replaces: every stage alone (stage mask) and all of them together must leave the same bytes — residual stream,
FP8 activations and their scales — for both 16-bit types and both forms of the O projection's input."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

O, N1, GU, D, N2, ALL = 1, 2, 4, 8, 16, 31
TC = 2


def make_case(M, H, F, KO, dt, seed, parts=4):
    from rvllm_b200.stack import _quant_weight
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    c = dict(M=M, H=H, F=F, KO=KO, dt=dt, parts=parts)
    c["attn16"] = (torch.randn((M, KO), generator=gen, device="cuda") * 0.7).to(dt)
    if M > 2:
        c["attn16"][1].zero_()                      # an all-zero row: scale 1e-12
    c["amax"] = c["attn16"].float().abs().reshape(M, parts, KO // parts).amax(dim=2).contiguous()
    c["o_w"], c["o_s"] = _quant_weight(H, KO, gen, 0.03)
    c["gu_w"], c["gu_s"] = _quant_weight(2 * F, H, gen, 0.03)
    c["d_w"], c["d_s"] = _quant_weight(H, F, gen, 0.03)
    c["res0"] = torch.randn((M, H), generator=gen, device="cuda").to(dt)
    c["g1"] = (1 + 0.1 * torch.randn(H, generator=gen, device="cuda")).to(dt)
    c["g2"] = (1 + 0.1 * torch.randn(H, generator=gen, device="cuda")).to(dt)
    return c


def chain(c, act, fp8_attn=False):
    """The stand-alone kernels, launched as the decode stack launches them (split-K 8 for the residual GEMMs, none
    for gate|up — the plans the benchmark shapes get anyway, forced here so small test shapes take them too)."""
    from rvllm_b200 import _lib, gemm
    from rvllm_b200.launchers import FusedActMulFp8QuantLaunch, FusedRmsnormFp8QuantLaunch, QuantizeFp8PerTokenLaunch
    L = _lib.lib()
    M, H, F, KO, dt = c["M"], c["H"], c["F"], c["KO"], c["dt"]
    code = 0 if dt == torch.float16 else 1
    out = {}
    u8 = lambda *s: torch.empty(s, dtype=torch.uint8, device="cuda")
    f32 = lambda *s: torch.empty(s, dtype=torch.float32, device="cuda")
    try:
        L.rvllm_fp8_gemm_tc_tune(0, 8)
        res = c["res0"].clone()
        a8, a_s = u8(M, KO), f32(M)
        QuantizeFp8PerTokenLaunch(M, KO).launch(a8, a_s, c["attn16"])
        if fp8_attn:
            gemm.fp8_gemm_channelscale(res, a8, c["o_w"], a_s, c["o_s"], residual=res, impl=TC)
        else:
            _lib.check(L.rvllm_fp8_gemm_residual_from16(res.data_ptr(), code, c["attn16"].data_ptr(), c["amax"].data_ptr(),
                                                        c["parts"], c["o_w"].data_ptr(), c["o_s"].data_ptr(), res.data_ptr(),
                                                        M, H, KO, _lib.current_stream()), "residual_from16")
        out["a8"], out["a_s"] = a8, a_s
        out["res1"] = res.clone()
        x8, xs = u8(M, H), f32(M)
        FusedRmsnormFp8QuantLaunch(M, H, 1e-6).launch(x8, xs, res, c["g1"])
        out["x8_1"], out["xs_1"] = x8, xs
        L.rvllm_fp8_gemm_tc_tune(0, 1)
        gu = torch.empty((M, 2 * F), dtype=dt, device="cuda")
        gemm.fp8_gemm_channelscale(gu, x8, c["gu_w"], xs, c["gu_s"], impl=TC)
        h8, hs = u8(M, F), f32(M)
        FusedActMulFp8QuantLaunch(M, F, act).launch(h8, hs, gu)
        out["h8"], out["hs"] = h8, hs
        L.rvllm_fp8_gemm_tc_tune(0, 8)
        gemm.fp8_gemm_channelscale(res, h8, c["d_w"], hs, c["d_s"], residual=res, impl=TC)
        out["res2"] = res.clone()
        x8b, xsb = u8(M, H), f32(M)
        FusedRmsnormFp8QuantLaunch(M, H, 1e-6).launch(x8b, xsb, res, c["g2"])
        out["x8_2"], out["xs_2"] = x8b, xsb
        torch.cuda.synchronize()
    finally:
        L.rvllm_fp8_gemm_tc_tune(0, 0)
    assert gemm.tc_status() == 0
    return out


class Block:
    def __init__(self, c, act):
        from rvllm_b200 import _lib
        self.c, self.act, self.L = c, act, _lib.lib()
        self.ws_bytes = int(self.L.rvllm_fp8_layer_block_workspace(c["H"], c["F"]))
        self.ws = torch.zeros(self.ws_bytes, dtype=torch.uint8, device="cuda")   # the barrier words start at zero

    def run(self, stages, residual, x8, xs, h8, hs, attn_fp8=None, attn_scale=None):
        from rvllm_b200 import _lib
        c = self.c
        code = 0 if c["dt"] == torch.float16 else 1
        a16 = None if attn_fp8 is not None else c["attn16"].data_ptr()
        rc = self.L.rvllm_fp8_layer_block(
            c["M"], c["H"], c["F"], c["KO"], self.act, code, 1e-6, a16, c["amax"].data_ptr(), c["parts"],
            None if attn_fp8 is None else attn_fp8.data_ptr(), None if attn_scale is None else attn_scale.data_ptr(),
            c["o_w"].data_ptr(), c["o_s"].data_ptr(), residual.data_ptr(), c["g1"].data_ptr(), c["g2"].data_ptr(),
            x8.data_ptr(), xs.data_ptr(), c["gu_w"].data_ptr(), c["gu_s"].data_ptr(), h8.data_ptr(), hs.data_ptr(),
            c["d_w"].data_ptr(), c["d_s"].data_ptr(), self.ws.data_ptr(), self.ws_bytes, stages, _lib.current_stream())
        _lib.check(rc, "fp8_layer_block")
        torch.cuda.synchronize()
        from rvllm_b200 import gemm
        assert gemm.tc_status() == 0, "a bounded wait in the layer-block kernel ran out"
        assert int(self.ws[:256].view(torch.int32).abs().sum()) == 0, "the barrier words were not left at zero"


def eqf(a, b):
    return torch.equal(a.view(torch.int32), b.view(torch.int32))


SHAPES = [(32, 5376, 21504, 4096), (32, 5376, 21504, 8192), (7, 1024, 2048, 4096), (1, 512, 2048, 1024), (19, 1536, 6144, 640)]


@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
@pytest.mark.parametrize("M,H,F,KO", SHAPES)
def test_layer_block_stages_equal_standalone_kernels(M, H, F, KO, dt):
    dt = getattr(torch, dt)
    act = 0 if H != 1536 else 1
    c = make_case(M, H, F, KO, dt, seed=M + H)
    want = chain(c, act)
    blk = Block(c, act)
    u8 = lambda *s: torch.full(s, 0xAB, dtype=torch.uint8, device="cuda")
    f32 = lambda *s: torch.full(s, -7.0, dtype=torch.float32, device="cuda")
    # O projection alone
    res = c["res0"].clone()
    blk.run(O, res, u8(M, H), f32(M), u8(M, F), f32(M))
    assert torch.equal(res, want["res1"]), "O stage"
    # RMSNorm + quant alone
    x8, xs = u8(M, H), f32(M)
    blk.run(N1, want["res1"].clone(), x8, xs, u8(M, F), f32(M))
    assert torch.equal(x8, want["x8_1"]) and eqf(xs, want["xs_1"]), "norm stage"
    # gate|up + act + quant alone
    h8, hs = u8(M, F), f32(M)
    blk.run(GU, want["res1"].clone(), want["x8_1"].clone(), want["xs_1"].clone(), h8, hs)
    assert eqf(hs, want["hs"]) and torch.equal(h8, want["h8"]), "gate|up stage"
    # down projection alone
    res = want["res1"].clone()
    blk.run(D, res, want["x8_1"].clone(), want["xs_1"].clone(), want["h8"].clone(), want["hs"].clone())
    assert torch.equal(res, want["res2"]), "down stage"
    # closing norm alone
    x8, xs = u8(M, H), f32(M)
    blk.run(N2, want["res2"].clone(), x8, xs, u8(M, F), f32(M))
    assert torch.equal(x8, want["x8_2"]) and eqf(xs, want["xs_2"]), "closing norm stage"
    # everything, twice in a row on the same workspace (the barrier words return to zero)
    for _ in range(2):
        res, x8, xs, h8, hs = c["res0"].clone(), u8(M, H), f32(M), u8(M, F), f32(M)
        blk.run(ALL, res, x8, xs, h8, hs)
        assert torch.equal(res, want["res2"]), "all stages: residual"
        assert torch.equal(h8, want["h8"]) and eqf(hs, want["hs"]), "all stages: act(gate)*up"
        assert torch.equal(x8, want["x8_2"]) and eqf(xs, want["xs_2"]), "all stages: closing norm"


@pytest.mark.parametrize("M,H,F,KO", [(32, 5376, 21504, 4096), (1, 5376, 21504, 8192), (5, 1024, 4096, 512)])
def test_layer_block_with_fp8_attention_rows(M, H, F, KO):
    """O projection fed FP8 rows + per-row scales (what the split-KV combine pass leaves) instead of 16-bit values."""
    c = make_case(M, H, F, KO, torch.bfloat16, seed=3 * M + KO)
    want = chain(c, 0, fp8_attn=True)
    blk = Block(c, 0)
    res = c["res0"].clone()
    x8 = torch.empty((M, H), dtype=torch.uint8, device="cuda")
    xs = torch.empty(M, dtype=torch.float32, device="cuda")
    h8 = torch.empty((M, F), dtype=torch.uint8, device="cuda")
    hs = torch.empty(M, dtype=torch.float32, device="cuda")
    blk.run(ALL, res, x8, xs, h8, hs, attn_fp8=want["a8"], attn_scale=want["a_s"])
    assert torch.equal(res, want["res2"]) and torch.equal(x8, want["x8_2"]) and eqf(xs, want["xs_2"])
    assert torch.equal(h8, want["h8"]) and eqf(hs, want["hs"])


def test_layer_block_rejects_shapes_it_does_not_take():
    from rvllm_b200 import _lib
    L = _lib.lib()
    t = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    p, s = t.data_ptr(), _lib.current_stream()

    def call(M=4, H=512, F=1024, KO=512, ws=None, wsb=1 << 20, stages=ALL):
        return L.rvllm_fp8_layer_block(M, H, F, KO, 0, 1, 1e-6, p, p, 1, None, None, p, p, p, p, p, p, p, p, p, p, p, p, p,
                                       p if ws is None else ws, wsb, stages, s)
    assert call(M=33) == _lib.E_UNSUPPORTED
    assert call(H=520) == _lib.E_UNSUPPORTED
    assert call(H=6400) == _lib.E_UNSUPPORTED
    assert call(F=4096 + 64) == _lib.E_UNSUPPORTED          # more than one gate|up unit per CTA
    assert call(F=1000) == _lib.E_UNSUPPORTED
    assert call(wsb=16) == _lib.E_WORKSPACE
    assert call(ws=p + 8) == _lib.E_WORKSPACE
    assert call(stages=0) == _lib.E_INVALID
    assert call(M=0) == _lib.E_INVALID
