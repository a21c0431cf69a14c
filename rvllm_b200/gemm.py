"""FP8 E4M3 GEMM entry points (host mirror of the reference's `CutlassLib` call sites,
v3/crates/rvllm-cutlass/src/lib_so.rs:500-512,621-634,734-746): argument checks happen in
the C ABI; these wrappers only marshal torch tensors.  IMPL_* selects the kernel family."""
from __future__ import annotations

from . import _lib
from ._lib import OUT_BF16, OUT_F16, OUT_F32, check, lib, ptr

IMPL_AUTO, IMPL_STREAM, IMPL_TCGEN05 = 0, 1, 2


def _out_kind(t) -> int:
    import torch

    return {torch.float16: OUT_F16, torch.bfloat16: OUT_BF16, torch.float32: OUT_F32}[t.dtype]


def fp8_gemm_channelscale(out, a_fp8, w_fp8, a_scale, w_scale, residual=None, impl=IMPL_AUTO, workspace=None,
                          stream=None) -> None:
    """out[M, N] = cast(a_scale[m] * (w_scale[n] * A[M, K] . W[N, K]^T) (+ residual))."""
    M, K = a_fp8.shape
    N = w_fp8.shape[0]
    ws_ptr, ws_len = (ptr(workspace), workspace.numel() * workspace.element_size()) if workspace is not None else (None, 0)
    check(lib().rvllm_fp8_gemm_channelscale(ptr(out), _out_kind(out), ptr(a_fp8), ptr(w_fp8), ptr(a_scale),
                                            ptr(w_scale), ptr(residual), M, N, K, impl, ws_ptr, ws_len,
                                            _lib.current_stream() if stream is None else stream), "fp8_gemm_channelscale")


def gateup_workspace_bytes(M: int, I: int, K: int) -> int:
    return int(lib().rvllm_fp8_gemm_gateup_workspace(M, I, K))


def fp8_gemm_gateup_act_quant(out_fp8, out_scale, a_fp8, w_fp8, a_scale, w_scale, act, dtype, workspace,
                              impl=IMPL_AUTO, stream=None) -> None:
    M, K = a_fp8.shape
    I = w_fp8.shape[0] // 2
    check(lib().rvllm_fp8_gemm_gateup_act_quant(ptr(out_fp8), ptr(out_scale), ptr(a_fp8), ptr(w_fp8), ptr(a_scale),
                                                ptr(w_scale), M, I, K, act, dtype, impl, ptr(workspace),
                                                workspace.numel() * workspace.element_size(),
                                                _lib.current_stream() if stream is None else stream),
          "fp8_gemm_gateup_act_quant")


def tc_status(reset: bool = True) -> int:
    import ctypes as C

    v = C.c_int(0)
    check(lib().rvllm_fp8_gemm_tc_status(C.byref(v), int(reset)), "fp8_gemm_tc_status")
    return v.value
