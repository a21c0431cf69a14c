"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations: weights N(0, 0.02) quantised per output channel (absmax / 448),
activations N(0, 1) quantised per token, K/V N(0, 1) quantised per (slot, kv_head), Q per
(sequence, head), block tables a seeded permutation of the physical blocks."""
from __future__ import annotations

import numpy as np


def quant_rows(orc, x):
    """f32 [R, C] -> (E4M3 bytes [R, C], scale [R]) with scale = max(absmax/448, 1e-12)."""
    return orc.quantize_fp8_per_token_f32(np.ascontiguousarray(x, np.float32), orc.MODE_CUDA)


def gemm_case(orc, M, N, K, seed):
    g = np.random.default_rng(seed)
    w, w_scale = quant_rows(orc, g.standard_normal((N, K), dtype=np.float32) * 0.02)
    a, a_scale = quant_rows(orc, g.standard_normal((M, K), dtype=np.float32))
    return a, a_scale, w, w_scale


def attention_case(orc, batch, heads, kv_heads, head_dim, block_size, ctx_lens, seed, window=-1,
                   recipe="normal", extra_blocks=3, max_blocks=None):
    """Returns a dict of numpy arrays.  recipe "normal": N(0,1) values quantised with
    per-row scales; "bytes": uniformly random non-NaN codes with scales U[0.002, 0.01]
    (the data recipe of the reference's parity bench,
    v3/kernels/fp8_decode_v2_parity_bench.cu:318-346)."""
    g = np.random.default_rng(seed)
    ctx_lens = np.asarray(ctx_lens, np.int32)
    need_tokens = int(max(int(ctx_lens.max()), 1))
    if window >= 0:
        need_tokens = min(need_tokens, window + 1 + block_size)  # ring only keeps the window
    blocks_per_seq = (need_tokens + block_size - 1) // block_size
    if max_blocks is None:
        max_blocks = blocks_per_seq
    num_blocks = batch * max_blocks + extra_blocks
    slots = num_blocks * block_size
    if recipe == "bytes":
        def rb(n):
            b = g.integers(0, 256, n, dtype=np.uint8)
            b[(b & 0x7F) == 0x7F] ^= 1
            return b
        k = rb(slots * kv_heads * head_dim).reshape(slots * kv_heads, head_dim)
        v = rb(slots * kv_heads * head_dim).reshape(slots * kv_heads, head_dim)
        q = rb(batch * heads * head_dim).reshape(batch * heads, head_dim)
        ks = g.uniform(0.002, 0.01, slots * kv_heads).astype(np.float32)
        vs = g.uniform(0.002, 0.01, slots * kv_heads).astype(np.float32)
        qs = g.uniform(0.002, 0.01, batch * heads).astype(np.float32)
    else:
        k, ks = quant_rows(orc, g.standard_normal((slots * kv_heads, head_dim), dtype=np.float32))
        v, vs = quant_rows(orc, g.standard_normal((slots * kv_heads, head_dim), dtype=np.float32))
        q, qs = quant_rows(orc, g.standard_normal((batch * heads, head_dim), dtype=np.float32))
    perm = g.permutation(num_blocks).astype(np.int32)
    tables = perm[: batch * max_blocks].reshape(batch, max_blocks).copy()
    return dict(q=q.reshape(batch, heads, head_dim), k=k.reshape(num_blocks, block_size, kv_heads, head_dim),
                v=v.reshape(num_blocks, block_size, kv_heads, head_dim), ks=ks, vs=vs, qs=qs,
                tables=np.ascontiguousarray(tables), ctx=ctx_lens, num_blocks=num_blocks, max_blocks=max_blocks,
                window=window, block_size=block_size, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                batch=batch)
