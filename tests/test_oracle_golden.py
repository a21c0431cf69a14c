"""Pins the CPU oracle to the known-answer vectors the reference's own tests hold.

Each block names the reference test it replays (paths relative to the reference
checkout).  If one of these fails the oracle is wrong and no parity claim stands.
"""
import math
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def enc1(orc, x, mode):
    return int(orc.lib().orc_e4m3_encode(np.float32(x), mode))


# ---- v3/crates/rvllm-core/src/fp8.rs:71-103 -------------------------------------------
def test_fp8_rs_zero_and_underflow_canonical(orc):
    tiny = np.frombuffer(np.uint32(1).tobytes(), np.float32)[0]
    for x in (-0.0, 0.0, tiny, -tiny):
        assert enc1(orc, x, orc.MODE_RUST) == 0x00


def test_fp8_rs_saturation_boundary(orc):
    for x, code in ((256.0, 0x78), (288.0, 0x79), (448.0, 0x7E), (-448.0, 0xFE), (449.0, 0x7E),
                    (-10000.0, 0xFE)):
        assert enc1(orc, x, orc.MODE_RUST) == code
        assert enc1(orc, x, orc.MODE_CUDA) == code


def test_fp8_rs_ties_to_even(orc):
    for x, code in ((1.0625, 0x38), (1.1875, 0x3A), (1.1, 0x39)):
        assert enc1(orc, x, orc.MODE_RUST) == code
        assert enc1(orc, x, orc.MODE_CUDA) == code


def test_fp8_rs_denormals(orc):
    s = 2.0 ** -9
    for x, code in ((s, 0x01), (s / 2, 0x00), (-s / 4, 0x00), (s * 0.75, 0x01)):
        assert enc1(orc, x, orc.MODE_RUST) == code
    # the device encoder keeps the sign of a negative value that rounds to zero
    assert enc1(orc, -s / 4, orc.MODE_CUDA) == 0x80


# ---- v3/crates/rvllm-fused/src/reference.rs:365-387 -----------------------------------
def test_reference_rs_nan_and_zero(orc):
    assert enc1(orc, -0.0, orc.MODE_RUST) == 0x00
    assert enc1(orc, float("nan"), orc.MODE_RUST) == 0x7F
    neg_nan = np.frombuffer(np.uint32(0xFFC00000).tobytes(), np.float32)[0]
    assert enc1(orc, neg_nan, orc.MODE_RUST) == 0x7F
    assert enc1(orc, neg_nan, orc.MODE_CUDA) == 0x7F


def test_reference_rs_roundtrip_every_positive_code(orc):
    for code in range(0x7F):
        e, m = (code >> 3) & 0xF, code & 7
        val = m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7)
        assert orc.lib().orc_e4m3_decode(code) == np.float32(val)
        assert enc1(orc, val, orc.MODE_RUST) == code
        assert enc1(orc, val, orc.MODE_CUDA) == code
        if code:
            assert enc1(orc, -val, orc.MODE_CUDA) == code | 0x80


# ---- scripts/test_fp8_encode.py:10-31 (torch.float8_e4m3fn vectors) -------------------
SCRIPT_VECTORS = [
    (0.0, 0x00), (-0.0, 0x80), (1.0, 0x38), (-1.0, 0xB8), (0.001953125, 0x01), (0.00390625, 0x02),
    (10.0, 0x52), (448.0, 0x7E), (449.0, 0x7E), (math.inf, 0x7F), (-math.inf, 0xFF),
    (math.nan, 0x7F), (-10.071, 0xD2), (-80.569, 0xEA), (9.352, 0x51), (-74.814, 0xE9),
    (-63.304, 0xE8), (-25.897, 0xDD), (-4.316, 0xC9), (-20.142, 0xDA),
]


def test_script_vectors(orc):
    for x, code in SCRIPT_VECTORS:
        if math.isinf(x):
            # torch turns inf into NaN; the device's saturate-to-finite convert and
            # the Rust encoder both clamp to +-448 instead.
            assert enc1(orc, x, orc.MODE_CUDA) == (0x7E | (0x80 if x < 0 else 0))
            assert enc1(orc, x, orc.MODE_RUST) == (0x7E | (0x80 if x < 0 else 0))
            continue
        assert enc1(orc, x, orc.MODE_CUDA) == code
        if not (x == 0 and math.copysign(1, x) < 0):
            assert enc1(orc, x, orc.MODE_RUST) == code


def test_torch_generated_vectors(orc):
    z = np.load(os.path.join(GOLD, "fp8_e4m3_torch.npz"))
    x = z["bits"].view(np.float32)
    got = orc.e4m3_encode(x, orc.MODE_CUDA)
    assert np.array_equal(got, z["code"])
    rust = orc.e4m3_encode(x, orc.MODE_RUST)
    differ = rust != z["code"]
    assert np.all(z["code"][differ] == 0x80)  # only the sign of a negative zero result


def test_decode_all_codes_match_float8(orc):
    # v3/kernels/fp8_decode_v2_parity_bench.cu:66-105 — every non-NaN code decodes to
    # the value the bit layout defines.
    torch = pytest.importorskip("torch")
    codes = np.arange(256, dtype=np.uint8)
    want = torch.from_numpy(codes).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    got = orc.e4m3_decode(codes)
    ok = ~np.isnan(want)
    assert np.array_equal(got[ok], want[ok])
    assert np.isnan(got[0x7F]) and np.isnan(got[0xFF])


# ---- reference.rs:341-350 (RMSNorm hand calculation) ----------------------------------
def test_rmsnorm_hand_calc(orc):
    x = np.array([[1.0, 2.0, 3.0]], np.float32)
    out = orc.rmsnorm_f32(x, np.ones(3, np.float32), 0.0)
    rms = np.sqrt(np.float32(14.0) / np.float32(3.0))
    assert np.all(np.abs(out[0] - x[0] / rms) < 1e-6)


def test_rmsnorm_rejects_bad_eps(orc):
    with pytest.raises(ValueError):
        orc.rmsnorm_f32(np.ones((1, 1), np.float32), np.ones(1, np.float32), float("nan"))


# ---- reference.rs:389-405 and rvllm-invariants/tests/identity.rs:91-128 ---------------
def test_argmax_vectors(orc):
    l = np.array([[0.1, 0.9, 0.3], [0.5, -1.0, 0.8]], np.float32)
    for mode in (orc.MODE_RUST, orc.MODE_CUDA):
        assert orc.argmax_f32(l, mode).tolist() == [1, 2]
        assert orc.argmax_f32(np.full((1, 4), 1.5, np.float32), mode).tolist() == [0]
        assert orc.argmax_f32(np.array([[2.0, 9.0, 4.0, 9.0, 1.0]], np.float32), mode).tolist() == [1]
        two = np.array([[0.1, 0.2, 9.9, 0.3], [7.0, 0.0, 1.0, 2.0]], np.float32)
        assert orc.argmax_f32(two, mode).tolist() == [2, 0]


def test_argmax_nan_rules(orc):
    # kernels/argmax.cu:16-25,101-109: NaN never wins, -inf can, all-NaN row -> -1;
    # the Rust reference refuses non-finite input instead (reference.rs:213).
    row = np.array([[np.nan, -np.inf, np.nan]], np.float32)
    assert orc.argmax_f32(row, orc.MODE_CUDA).tolist() == [1]
    assert orc.argmax_f32(np.full((1, 3), np.nan, np.float32), orc.MODE_CUDA).tolist() == [-1]
    with pytest.raises(ValueError):
        orc.argmax_f32(row, orc.MODE_RUST)


def test_embedding_gather_vector(orc):
    table = orc.to_bits16(np.array([[10.0, 11.0], [20.0, 21.0], [30.0, 31.0]], np.float32), orc.F16)
    out = orc.from_bits16(orc.embedding_gather(table, [2, 0]), orc.F16)
    assert out.reshape(-1).tolist() == [30.0, 31.0, 10.0, 11.0]
    with pytest.raises(ValueError):
        orc.embedding_gather(table, [3])


# ---- reference.rs:407-420 (fused SiLU quant runs, identity RoPE) ----------------------
def test_silu_quant_and_identity_rope(orc):
    gate_up = np.array([[0.0, 1.0, -1.0, 2.0, 1.0, 1.0, 1.0, 1.0]], np.float32)
    out, scale = orc.act_mul_fp8_quant_f32(gate_up, orc.ACT_SILU, orc.MODE_RUST)
    assert out.any() and scale[0] > 0
    # largest element silu(2)*1 maps to +-448 exactly
    assert out[0, 3] == 0x7E and out[0, 0] == 0x00 and out[0, 2] & 0x80


# ---- gemma4_reference.rs:352-382 (partial RoPE golden vector: 32 heads x 512, rotary 128, position 7) ----
def test_gemma4_global_partial_rope_golden_vector(orc):
    heads, hd, rot = 32, 512, 128
    x = np.zeros((1, (heads + 2) * hd), np.float32)           # one KV head behind the 32 query heads
    x[0, 0], x[0, hd // 2], x[0, 1], x[0, hd // 2 + 1], x[0, rot // 2] = 1.0, 2.0, 3.0, 4.0, 7.0
    cos = np.ones((8, rot // 2), np.float32)
    sin = np.zeros((8, rot // 2), np.float32)
    cos[7, 0], sin[7, 0], cos[7, 1], sin[7, 1] = 0.5, 0.8660254, -0.25, 0.96824586
    kc = np.zeros((4, 1, hd), np.uint8)
    vc = np.zeros_like(kc)
    ksc, vsc = np.zeros(4, np.float32), np.zeros(4, np.float32)
    q8, qs = orc.rope_fp8kv(orc.to_bits16(x, 0), heads, 1, hd, rot, orc.to_bits16(cos, 0), orc.to_bits16(sin, 0),
                            np.array([7], np.int32), np.array([2], np.int32), kc, vc, ksc, vsc)
    # The kernel form works on 16-bit tables and stores E4M3 with the head's scale (absmax 7 -> 7 / 448): the
    # golden values must come back to within the table's 16-bit rounding plus half an E4M3 step at their size.
    assert qs[0, 0] == np.float32(7.0) / np.float32(448.0)
    deq = orc.e4m3_decode(q8[0, 0]) * qs[0, 0]
    expected = {0: -1.2320508, hd // 2: 1.8660254, 1: -4.6229835, hd // 2 + 1: 1.9047375}
    for idx, want in expected.items():
        step = 2.0 ** (np.floor(np.log2(abs(want) / qs[0, 0])) - 3) * qs[0, 0]   # E4M3 spacing at this magnitude
        assert abs(deq[idx] - want) <= 0.5 * step + 3e-3, (idx, deq[idx], want)
    assert deq[rot // 2] == 7.0                                  # outside the rotary span: untouched
    mag = q8 & 0x7F                                              # (0 * -0.25 is -0: code 0x80 as the kernels store it)
    assert not mag[0, 1:].any() and not np.delete(mag[0, 0], list(expected) + [rot // 2]).any()


# ---- 16-bit conversions used everywhere: exhaustive against numpy/torch ---------------
def test_half_conversions_exhaustive(orc):
    torch = pytest.importorskip("torch")
    bits = np.arange(65536, dtype=np.uint16)
    lib = orc.lib()
    f = np.array([lib.orc_h2f(int(b), 0) for b in bits[::7]], np.float32)
    want = bits[::7].view(np.float16).astype(np.float32)
    ok = ~np.isnan(want)  # NaN payloads are not part of the contract
    assert np.array_equal(f.view(np.uint32)[ok], want.view(np.uint32)[ok])
    assert np.all(np.isnan(f[~ok]))
    g = np.random.default_rng(1)
    x = np.concatenate([g.standard_normal(4000).astype(np.float32) * s for s in (1e-7, 1e-4, 1.0, 3e4)])
    x = np.concatenate([x, np.array([65504.0, 65519.9, 65520.0, 70000.0, 2.0 ** -25, 2.0 ** -24 * 1.5], np.float32)])
    got = np.array([lib.orc_f2h(np.float32(v), 0) for v in x], np.uint16)
    assert np.array_equal(got, x.astype(np.float16).view(np.uint16))
    gotb = np.array([lib.orc_f2h(np.float32(v), 1) for v in x], np.uint16)
    wantb = torch.from_numpy(x).to(torch.bfloat16).view(torch.uint16).numpy()
    assert np.array_equal(gotb, wantb)
    assert np.array_equal(orc.to_bits16(x, orc.BF16), wantb)
