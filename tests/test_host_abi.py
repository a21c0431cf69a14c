"""CPU-only checks of the C-ABI library: it loads without a GPU, exports every symbol the
headers declare, and its validation logic reproduces the reference launchers' own unit
tests (v3/crates/rvllm-fused/src/launcher.rs:746-802, v3/crates/rvllm-attention/src/decode.rs:
714-767, v3/kernels/fp8_decode_v2.cu:945-957).  No kernel is launched here."""
import ctypes as C
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from rvllm_b200 import _lib, build
    build.build_library()
    return _lib.lib()


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        text = "\n".join(l for l in text.splitlines() if not l.lstrip().startswith("#"))
        names |= set(re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}]*\)\s*;", text))
    return names


def test_every_declared_symbol_is_exported(L):
    names = declared_symbols()
    assert len(names) > 30
    missing = [n for n in sorted(names) if not hasattr(L, n)]
    assert not missing, missing


def test_every_exported_function_is_declared():
    """The reverse direction: nothing callable is exported behind the headers' back.  The only
    undeclared C symbols are the host stubs of the `extern "C" __global__` kernels, whose names
    are the reference's PTX entry points (they end in `_kernel`)."""
    import subprocess
    from rvllm_b200 import _lib, build
    build.build_library()
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = {f[2] for f in (l.split() for l in out.splitlines()) if len(f) == 3 and f[1] == "T" and not f[2].startswith("_")}
    extra = sorted(n for n in exported - declared_symbols() if not n.endswith("_kernel"))
    assert not extra, extra


def test_python_binding_table_matches_header():
    from rvllm_b200 import _lib
    assert set(_lib.SIGNATURES) <= declared_symbols()


def test_identity(L):
    assert L.rvllm_b200_abi_version() == 1
    assert L.rvllm_b200_build_arch() == b"sm_100a"
    assert L.rvllm_fa_sm89_abi_version() == 2            # v3/crates/rvllm-attention/src/lib.rs ABI handshake
    assert L.fa_sm89_fp8_output_dtype() == 1 and L.fa_sm89_fp8_output_element_size() == 2


def test_per_device_setup_bookkeeping(L):
    """cudaFuncSetAttribute belongs to a device: the once-flags are kept per device ordinal, a failed
    set-up is retried, and an unknown ordinal sets up every time (self-test in the library, no CUDA call)."""
    assert L.rvllm_b200_selftest_device_once() == 0


def test_row_launcher_validation_kats():
    from rvllm_b200 import InvalidArgument
    from rvllm_b200.launchers import (ArgmaxLaunch, FusedRmsnormFp8QuantLaunch, FusedSiluMulFp8QuantLaunch,
                                      QuantizeFp8PerTokenLaunch)
    with pytest.raises(InvalidArgument):
        FusedRmsnormFp8QuantLaunch(1, 13, 1e-6).validate()      # hidden not a multiple of 8
    FusedRmsnormFp8QuantLaunch(1, 3584, 1e-6).validate()
    with pytest.raises(InvalidArgument):
        FusedRmsnormFp8QuantLaunch(0, 3584, 1e-6).validate()
    with pytest.raises(InvalidArgument):
        FusedRmsnormFp8QuantLaunch(1, 3584, float("nan")).validate()
    with pytest.raises(InvalidArgument):
        QuantizeFp8PerTokenLaunch(1, 65544).validate()           # dim > 65536
    QuantizeFp8PerTokenLaunch(4, 65536).validate()
    with pytest.raises(InvalidArgument):
        FusedSiluMulFp8QuantLaunch(1, 12).validate()
    FusedSiluMulFp8QuantLaunch(1, 18944).validate()
    with pytest.raises(InvalidArgument):
        ArgmaxLaunch(1, 0).validate()                            # zero vocab
    with pytest.raises(InvalidArgument):
        ArgmaxLaunch(0, 10).validate()
    ArgmaxLaunch(1, 262144).validate()


def test_launch_with_null_pointers_is_refused_before_cuda(L):
    from rvllm_b200 import _lib
    assert L.rvllm_fused_rmsnorm_fp8_quant_launch(1, 64, 1e-6, None, None, None, None, 0, None) == _lib.E_INVALID
    assert b"null" in L.rvllm_b200_last_error()
    assert L.rvllm_argmax_launch(1, 8, None, None, 0, None) == _lib.E_INVALID
    assert L.rvllm_fp8_gemm_channelscale(None, 0, None, None, None, None, None, 1, 1, 64, 0, None, 0, None) == _lib.E_INVALID
    assert L.fa_sm89_paged_decode(*([None] * 7), 0, 1.0, *([1] * 8), None) == -1
    assert L.fa_sm89_paged_prefill_fp8(*([None] * 8), 0, *([None] * 6), 1.0, *([1] * 10), None) == -1


def test_paged_decode_params_kats():
    from rvllm_b200 import InvalidArgument
    from rvllm_b200.attention import PagedDecodeParams
    ok = dict(num_seqs=4, num_heads=32, num_kv_heads=16, head_dim=128, block_size=16, max_blocks_per_seq=64,
              num_blocks_total=1024, scale=0.088)
    for hd in (64, 128, 256, 512):
        PagedDecodeParams(**{**ok, "head_dim": hd}).validate()
    for bad in (dict(head_dim=96), dict(num_heads=7, num_kv_heads=4), dict(num_seqs=0), dict(block_size=0),
                dict(scale=0.0), dict(scale=float("inf")), dict(window_size_left=-2),
                dict(window_size_left=16 * 64), dict(num_heads=66, num_kv_heads=2)):
        with pytest.raises(InvalidArgument):
            PagedDecodeParams(**{**ok, **bad}).validate()
    PagedDecodeParams(**{**ok, "window_size_left": 16 * 64 - 1}).validate()


def test_attention_workspace_query_is_self_consistent(L):
    U64_MAX = 2 ** 64 - 1
    # the reference-named query keeps the reference's head_dim set
    assert L.fa_sm89_decode_workspace_size(1, 32, 16, 64) == U64_MAX
    assert L.fa_sm89_decode_workspace_size(1, 32, 16, 96) == U64_MAX
    assert L.fa_sm89_decode_workspace_size(1, 7, 4, 128) == U64_MAX
    for batch, heads, kvh, hd in ((1, 32, 16, 256), (32, 32, 16, 128), (64, 32, 16, 256), (1024, 32, 16, 128)):
        chunks = L.rvllm_paged_decode_max_chunks(batch, kvh)
        want = 0 if chunks <= 1 else batch * heads * chunks * (hd + 2) * 4   # [B][H][C][HD+2] f32
        assert L.fa_sm89_decode_workspace_size(batch, heads, kvh, hd) == want
        assert 1 <= chunks <= 32


def test_gemm_workspace_queries(L):
    assert L.cutlass_fp8_gemm_channelscale_workspace(32, 8192, 5376) == L.rvllm_fp8_gemm_workspace(32, 8192, 5376)
    assert L.cutlass_fp8_gemm_v0_workspace_size(32, 8192, 5376) >= 8192 * 4
    assert L.rvllm_fp8_gemm_gateup_workspace(32, 21504, 5376) >= 32 * 2 * 21504 * 2
    assert L.rvllm_fp8_gemm_workspace(0, 1, 1) == 0


def test_missing_library_is_a_hard_error(monkeypatch, tmp_path):
    from rvllm_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.RvllmError):
        _lib.lib()


def test_build_register_budget_check():
    """The build refuses a kernel that counts on three CTAs per SM when ptxas gave it more than 96 registers."""
    from rvllm_b200 import build

    ok = ("ptxas info    : Compiling entry function '_ZN4rvtc18fp8_gemm_tc_kernelILi32ELi1E13__nv_bfloat16EEv' for 'sm_100a'\n"
          "ptxas info    : Function properties for x\n    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads\n"
          "ptxas info    : Used 96 registers, used 2 barriers, 128 bytes smem\n"
          "ptxas info    : Compiling entry function '_ZN4rvtc18fp8_gemm_tc_kernelILi256ELi1E13__nv_bfloat16EEv' for 'sm_100a'\n"
          "ptxas info    : Used 120 registers, used 2 barriers\n")
    build.check_register_budget(ok)  # the 256-row tile runs one CTA per SM: no budget
    with pytest.raises(RuntimeError, match="register budget"):
        build.check_register_budget(ok.replace("Used 96 registers", "Used 97 registers"))


def test_library_is_not_the_time_stamp_build():
    """The GEMM's %globaltimer stamps are a build option (they cost the decode step 1.2 % even when off): the library
    that ships must refuse a trace buffer, unless the build was asked for them."""
    import ctypes
    from rvllm_b200 import _lib

    if os.environ.get("RVLLM_TC_TRACE", "0") not in ("", "0"):
        pytest.skip("a time-stamp build was asked for")
    L = _lib.lib()
    try:
        assert L.rvllm_fp8_gemm_tc_trace(ctypes.c_void_p(4096), 1) == _lib.E_UNSUPPORTED
    finally:
        assert L.rvllm_fp8_gemm_tc_trace(None, 0) == _lib.OK
