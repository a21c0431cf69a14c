"""The allocation-free decode-attention entry point (rvllm_paged_decode_fp8_static_scratch).

It exists for callers that have no way to allocate device memory — a runtime whose memory was
divided into fixed regions when it started, or a plug-in whose host does not allow it to call the
CUDA allocator — so its split-KV partials live in a scratch array built into the library instead
of a caller workspace.  The test calls it through the C ABI twice in a row (the second call finds
the first call's partials still in the scratch) and requires the outputs to equal those of the
ordinary entry point with a caller-allocated workspace; it also checks that a launch too large for
the built-in scratch is refused instead of launched.  Collected last on purpose: a run that stops
at the first failure has then already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from tests import datagen  # noqa: E402


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def call_static(L, t, out, c, scale, window):
    from rvllm_b200 import _lib
    return L.rvllm_paged_decode_fp8_static_scratch(
        t["q"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr(), out.data_ptr(), 0, t["tables"].data_ptr(),
        t["ctx"].data_ptr(), t["ks"].data_ptr(), t["vs"].data_ptr(), t["qs"].data_ptr(), None, None, None, scale,
        c["batch"], c["heads"], c["kv_heads"], c["head_dim"], c["block_size"], c["max_blocks"], c["num_blocks"], window,
        _lib.current_stream())


def test_static_scratch_matches_workspace_entry_point_twice(orc):
    from rvllm_b200 import _lib
    from rvllm_b200.attention import PagedDecodeFp8Launcher, PagedDecodeParams
    L = _lib.lib()
    assert L.rvllm_paged_decode_static_scratch_bytes() == 8 << 20
    # two different launches that both split the KV range (batch 2 and 3 -> many chunks per sequence)
    cases = [datagen.attention_case(orc, 2, 32, 16, 128, 16, [3000, 700], seed=31),
             datagen.attention_case(orc, 3, 32, 16, 256, 16, [5000, 64, 1500], seed=32)]
    for c in cases:
        scale = float(c["head_dim"] ** -0.5)
        p = PagedDecodeParams(c["batch"], c["heads"], c["kv_heads"], c["head_dim"], c["block_size"], c["max_blocks"],
                              c["num_blocks"], scale, -1)
        assert p.max_chunks() > 1 and 0 < p.workspace_bytes() <= 8 << 20
        t = {k: dev(c[k]) for k in ("q", "k", "v", "tables", "ctx", "ks", "vs", "qs")}
        want = torch.empty((c["batch"], c["heads"], c["head_dim"]), dtype=torch.float16, device="cuda")
        ws = torch.empty(p.workspace_bytes(), dtype=torch.uint8, device="cuda")
        PagedDecodeFp8Launcher(p).launch(t["q"], t["k"], t["v"], want, t["tables"], t["ctx"], workspace=ws,
                                         k_scale_cache=t["ks"], v_scale_cache=t["vs"], q_scale_cache=t["qs"])
        for _ in range(2):  # second call runs over the first call's leftovers
            got = torch.full_like(want, 7.0)
            _lib.check(call_static(L, t, got, c, scale, -1), "static-scratch decode")
            torch.cuda.synchronize()
            assert torch.equal(got, want)
        ref = orc.from_bits16(orc.paged_decode_fp8(c["q"], c["k"], c["v"], c["tables"], c["ctx"], scale, c["heads"],
                                                   c["kv_heads"], c["head_dim"], c["block_size"], k_scale_cache=c["ks"],
                                                   v_scale_cache=c["vs"], q_scale_cache=c["qs"], precise=True,
                                                   num_blocks_total=c["num_blocks"]), 0)
        assert np.abs(want.float().cpu().numpy() - ref).max() <= 2e-3 + 1e-2 * np.abs(ref).max()


def test_static_scratch_refuses_oversized_launch(orc):
    from rvllm_b200 import _lib
    L = _lib.lib()
    # batch 3, 64 heads over 2 KV heads, head_dim 512: 32 chunks * 3 * 64 * 514 * 4 B = 12.6 MB > 8 MiB
    need = L.rvllm_paged_decode_workspace_size(3, 64, 2, 512)
    assert need > 8 << 20
    z = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    f = torch.ones(1 << 16, dtype=torch.float32, device="cuda")
    i = torch.zeros(1 << 12, dtype=torch.int32, device="cuda")
    out = torch.zeros(3 * 64 * 512, dtype=torch.float16, device="cuda")
    rc = L.rvllm_paged_decode_fp8_static_scratch(z.data_ptr(), z.data_ptr(), z.data_ptr(), out.data_ptr(), 0,
                                                 i.data_ptr(), i.data_ptr(), f.data_ptr(), f.data_ptr(), f.data_ptr(),
                                                 None, None, None, 0.05, 3, 64, 2, 512, 16, 64, 4, -1,
                                                 _lib.current_stream())
    assert rc == _lib.E_WORKSPACE
    assert "built-in scratch" in _lib.last_error()
    torch.cuda.synchronize()
    assert (out == 0).all()
