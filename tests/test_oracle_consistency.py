"""CPU cross-checks inside the oracle: the three attention restatements (f64 two-pass,
f32 scalar-kernel order, f32 split-KV + combine) agree, block-table resolution handles the
ring, and the GEMM modes agree with a numpy evaluation."""
import numpy as np
import pytest

from tests import datagen


@pytest.mark.parametrize("window", [-1, 40])
def test_attention_restatements_agree(orc, window):
    bs = 16
    ctxs = [1, 17, 130, 300]
    mb = None if window < 0 else (window + 1 + bs - 1) // bs + 1
    c = datagen.attention_case(orc, 4, 8, 4, 64, bs, ctxs, seed=0, window=window, max_blocks=mb)
    kw = dict(window_size_left=window, k_scale_cache=c["ks"], v_scale_cache=c["vs"], q_scale_cache=c["qs"])
    a = orc.from_bits16(orc.paged_decode_fp8(c["q"], c["k"], c["v"], c["tables"], c["ctx"], 0.125, 8, 4, 64, bs,
                                             precise=True, **kw), 0)
    b = orc.from_bits16(orc.paged_decode_fp8(c["q"], c["k"], c["v"], c["tables"], c["ctx"], 0.125, 8, 4, 64, bs,
                                             precise=False, **kw), 0)
    s, ws = orc.paged_decode_fp8_split(c["q"], c["k"], c["v"], c["tables"], c["ctx"], 0.125, 8, 4, 64, bs, 3,
                                       c["ks"], c["vs"], c["qs"], window_size_left=window)
    s = orc.from_bits16(s, 0)
    assert np.abs(a - b).max() < 2e-3 and np.abs(a - s).max() < 2e-3
    assert ws.shape == (4, 8, 3, 66)


def test_attention_matches_dense_numpy(orc):
    c = datagen.attention_case(orc, 2, 4, 2, 64, 16, [50, 33], seed=1)
    got = orc.from_bits16(orc.paged_decode_fp8(c["q"], c["k"], c["v"], c["tables"], c["ctx"], 0.125, 4, 2, 64, 16,
                                               precise=True, k_scale_cache=c["ks"], v_scale_cache=c["vs"],
                                               q_scale_cache=c["qs"]), 0)
    kf = orc.e4m3_decode(c["k"]).reshape(-1, 2, 64) * c["ks"].reshape(-1, 2, 1)
    vf = orc.e4m3_decode(c["v"]).reshape(-1, 2, 64) * c["vs"].reshape(-1, 2, 1)
    qf = orc.e4m3_decode(c["q"]) * c["qs"].reshape(2, 4, 1)
    for b in range(2):
        slots = [c["tables"][b, t // 16] * 16 + t % 16 for t in range(c["ctx"][b])]
        for h in range(4):
            s = kf[slots, h // 2] @ qf[b, h] * 0.125
            p = np.exp(s - s.max())
            want = (p / p.sum()) @ vf[slots, h // 2]
            assert np.abs(got[b, h] - want).max() < 2e-3


def test_ring_slot_resolution(orc):
    tables = np.array([[5, 9, 2]], np.int32)
    ctx = np.array([100], np.int32)
    # window 19 -> tokens 80..99; pages 5, 6 -> ring entries 5 % 3 = 2, 6 % 3 = 0
    slots = orc.attended_slots(tables, ctx, 16, 12, 19, 20)[0]
    want = [tables[0, (t // 16) % 3] * 16 + t % 16 for t in range(80, 100)]
    assert slots.tolist() == want
    bad = orc.attended_slots(np.array([[5, 99, 2]], np.int32), np.array([20], np.int32), 16, 12, -1, 20)[0]
    assert bad[15] == 5 * 16 + 15 and bad[16] == -1


def test_gemm_modes(orc):
    a, a_s, w, w_s = datagen.gemm_case(orc, 5, 24, 128, 0)
    f32 = orc.fp8_gemm(a, w, a_s, w_s, out_kind=2)
    f64 = orc.fp8_gemm(a, w, a_s, w_s, out_kind=2, acc64=True)
    dense = (orc.e4m3_decode(a).astype(np.float64) @ orc.e4m3_decode(w).astype(np.float64).T) * a_s[:, None] * w_s[None, :]
    assert np.abs(f64 - dense).max() <= 1e-6 * np.abs(dense).max()
    assert np.abs(f32 - dense).max() <= 1e-5 * np.abs(dense).max()
    res = orc.to_bits16(np.ones((5, 24), np.float32), orc.F16)
    h = orc.from_bits16(orc.fp8_gemm(a, w, a_s, w_s, residual=res, out_kind=0), orc.F16)
    assert np.abs(h - (dense + 1)).max() <= 2e-3 * np.abs(dense + 1).max()
    # f16 output saturates instead of overflowing to inf
    big = orc.from_bits16(orc.fp8_gemm(a, w, a_s * 1e9, w_s, out_kind=0), orc.F16)
    assert np.isfinite(big).all() and np.abs(big).max() == 65504.0


def test_rope_kv_write_matches_numpy(orc):
    T, heads, kvh, hd = 3, 4, 2, 64
    g = np.random.default_rng(0)
    qkv = g.standard_normal((T, (heads + 2 * kvh) * hd)).astype(np.float32)
    pos = np.array([0, 5, 9], np.int32)
    inv = 1.0 / (10000 ** (np.arange(hd // 2) / (hd // 2)))
    ang = np.arange(16)[:, None] * inv[None, :]
    cos16, sin16 = orc.to_bits16(np.cos(ang).astype(np.float32), 0), orc.to_bits16(np.sin(ang).astype(np.float32), 0)
    slots = 32
    kc = np.zeros((slots, kvh, hd), np.uint8)
    vc = np.zeros_like(kc)
    ksc = np.zeros(slots * kvh, np.float32)
    vsc = np.zeros_like(ksc)
    slot_map = np.array([7, -1, 30], np.int32)
    q8, qs = orc.rope_fp8kv(orc.to_bits16(qkv, 0), heads, kvh, hd, hd, cos16, sin16, pos, slot_map, kc, vc, ksc, vsc)
    x = orc.from_bits16(orc.to_bits16(qkv, 0), 0)
    c, s = orc.from_bits16(cos16, 0), orc.from_bits16(sin16, 0)
    q = x[:, : heads * hd].reshape(T, heads, hd)
    lo, hi = q[..., :32], q[..., 32:]
    rot = np.concatenate([lo * c[pos][:, None] - hi * s[pos][:, None], lo * s[pos][:, None] + hi * c[pos][:, None]], -1)
    deq = orc.e4m3_decode(q8) * qs[..., None]
    assert np.abs(deq - rot).max() <= 0.07 * np.abs(rot).max()
    assert np.allclose(qs, np.abs(rot).max(-1) / 448, rtol=1e-6)
    assert ksc.reshape(slots, kvh)[7].all() and not ksc.reshape(slots, kvh)[8].any()  # slot -1 skipped
    v = x[:, (heads + kvh) * hd:].reshape(T, kvh, hd)
    assert np.abs(orc.e4m3_decode(vc[30]) * vsc.reshape(slots, kvh)[30][:, None] - v[2]).max() <= 0.07 * np.abs(v[2]).max()


def test_thread_count_override_survives_launcher_env():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the timed CPU arm asks for
    every CPU the process may use instead."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = "import oracle as o; a = o.num_threads(); b = o.use_all_host_threads(); print(a, b)"
    env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONPATH=root)
    out = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    before, after = map(int, out.stdout.split())
    assert before == 1
    assert after == len(os.sched_getaffinity(0))
