"""Loader of the C-ABI shared library (``librvllm_b200.so``).

A missing library is a hard error, as a missing kernel artifact is in the reference
(v3/crates/rvllm-kernels/src/loader.rs:104-114): there is no CPU or eager fallback.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librvllm_b200.so")

OK, E_INVALID, E_LAUNCH, E_UNSUPPORTED, E_WORKSPACE, E_ARTIFACT, E_NO_DEVICE = 0, -1, -2, -3, -4, -5, -6
F16, BF16 = 0, 1
OUT_F16, OUT_BF16, OUT_F32 = 0, 1, 2
ACT_SILU, ACT_GELU_TANH = 0, 1


class RvllmError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, what: str, detail: str):
        super().__init__(f"{what} failed (rc={code}): {detail}")
        self.code = code
        self.detail = detail


class InvalidArgument(RvllmError):
    pass


_lib = None

_u32, _i32, _f32, _vp, _sz, _u64 = C.c_uint32, C.c_int, C.c_float, C.c_void_p, C.c_size_t, C.c_uint64

# name -> (restype, argtypes); every symbol include/rvllm_b200*.h declares
SIGNATURES = {
    "rvllm_b200_abi_version": (_i32, []),
    "rvllm_b200_last_error": (C.c_char_p, []),
    "rvllm_b200_build_arch": (C.c_char_p, []),
    "rvllm_b200_set_pdl": (None, [_i32]),
    "rvllm_b200_get_pdl": (_i32, []),
    "rvllm_b200_selftest_device_once": (_i32, []),
    "rvllm_stack_debug_skip": (None, [_i32]),
    "rvllm_paged_decode_cluster_combine": (None, [_i32]),
    "rvllm_paged_decode_cluster_tune": (None, [_i32, _i32]),
    "rvllm_paged_decode_early_meta": (None, [_i32]),
    "rvllm_paged_decode_hint_early_meta": (None, []),
    "rvllm_fused_rmsnorm_fp8_quant_validate": (_i32, [_u32, _u32, _f32]),
    "rvllm_fused_rmsnorm_fp8_quant_launch": (_i32, [_u32, _u32, _f32, _vp, _vp, _vp, _vp, _i32, _vp]),
    "rvllm_fused_add_rmsnorm_fp8_quant_launch": (_i32, [_u32, _u32, _f32, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp]),
    "rvllm_quantize_fp8_per_token_validate": (_i32, [_u32, _u32]),
    "rvllm_quantize_fp8_per_token_launch": (_i32, [_u32, _u32, _vp, _vp, _vp, _i32, _vp]),
    "rvllm_fused_act_mul_fp8_quant_validate": (_i32, [_u32, _u32]),
    "rvllm_fused_act_mul_fp8_quant_launch": (_i32, [_u32, _u32, _i32, _vp, _vp, _vp, _i32, _vp]),
    "rvllm_argmax_validate": (_i32, [_u32, _u32]),
    "rvllm_argmax_launch": (_i32, [_u32, _u32, _vp, _vp, _i32, _vp]),
    "cutlass_fp8_gemm_channelscale": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _sz, _vp]),
    "cutlass_fp8_gemm_channelscale_workspace": (_sz, [_i32, _i32, _i32]),
    "cutlass_fp8_gemm_v0": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _sz, _vp]),
    "cutlass_fp8_gemm_v0_workspace_size": (_sz, [_i32, _i32, _i32]),
    "cutlass_fp8_gemm_residual_v0": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _sz, _vp]),
    "cutlass_fp8_gemm_residual_v0_workspace_size": (_sz, [_i32, _i32, _i32]),
    "rvllm_fp8_gemm_channelscale": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "rvllm_fp8_gemm_workspace": (_sz, [_i32, _i32, _i32]),
    "rvllm_fp8_gemm_gateup_act_quant": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "rvllm_fp8_gemm_gateup_workspace": (_sz, [_i32, _i32, _i32]),
    "rvllm_fp8_gemm_tc_status": (_i32, [C.POINTER(_i32), _i32]),
    "rvllm_fp8_gemm_tc_tune": (None, [_i32, _i32]),
    "rvllm_fp8_gemm_tc_reduce": (None, [_i32]),
    "rvllm_fp8_gemm_tc_split_target": (None, [_i32]),
    "rvllm_fp8_gemm_tc_split_for": (None, [_i32, _i32, _i32, _i32]),
    "rvllm_fp8_gemm_tc_trace": (_i32, [_vp, _i32]),
    "rvllm_fp8_gemm_residual_from16": (_i32, [_vp, _i32, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "rvllm_fp8_gemm_qkv_rope_fp8kv": (_i32, [_vp] * 4 + [_i32] * 6 + [_vp] * 10 + [_i32] * 2 + [_vp]),
    "rvllm_fp8_gemm_lm_head_argmax_workspace": (_sz, [_i32, _i32]),
    "rvllm_fp8_gemm_lm_head_argmax": (_i32, [_vp] * 5 + [_i32] * 3 + [_f32, _vp, _sz, _vp]),
    "rvllm_fp8_layer_block_trace": (None, [_vp]),
    "rvllm_fp8_layer_block_capacity": (_i32, [C.POINTER(_i32), C.POINTER(_i32), _i32]),
    "rvllm_fp8_layer_block_workspace": (_sz, [_i32, _i32]),
    "rvllm_fp8_layer_block": (_i32, [_i32] * 6 + [_f32, _vp, _vp, _i32] + [_vp] * 16 + [_sz, _i32, _vp]),
    "rvllm_fa_sm89_abi_version": (_i32, []),
    "fa_sm89_fp8_output_dtype": (_i32, []),
    "fa_sm89_fp8_output_element_size": (_i32, []),
    "fa_sm89_decode_workspace_size": (_u64, [_i32, _i32, _i32, _i32]),
    "fa_sm89_paged_decode_fp8": (_i32, [_vp] * 7 + [_sz] + [_vp] * 6 + [_f32] + [_i32] * 8 + [_vp]),
    "fa_sm89_paged_decode": (_i32, [_vp] * 7 + [_sz, _f32] + [_i32] * 8 + [_vp]),
    "fa_sm89_paged_prefill_fp8": (_i32, [_vp] * 8 + [_sz] + [_vp] * 6 + [_f32] + [_i32] * 10 + [_vp]),
    "rvllm_paged_decode_fp8_validate": (_i32, [_i32] * 8 + [_f32]),
    "rvllm_paged_decode_workspace_size": (_u64, [_i32, _i32, _i32, _i32]),
    "rvllm_paged_decode_max_chunks": (_i32, [_i32, _i32]),
    "rvllm_paged_decode_tune": (None, [_i32, _i32, _i32]),
    "rvllm_paged_decode_tc_status": (_i32, [_vp, _i32]),
    "rvllm_paged_decode_ring": (None, [_i32]),
    "rvllm_paged_decode_kernel_for": (_i32, [_i32] * 5),
    "rvllm_paged_decode_quant_workspace_size": (_u64, [_i32, _i32, _i32, _i32]),
    "rvllm_paged_decode_fp8_quant": (_i32, [_vp] * 5 + [_i32] + [_vp] * 3 + [_sz] + [_vp] * 6 + [_f32] + [_i32] * 8 + [_vp]),
    "rvllm_paged_decode_fp8": (_i32, [_vp] * 4 + [_i32] + [_vp] * 3 + [_sz] + [_vp] * 6 + [_f32] + [_i32] * 8 + [_vp]),
    "rvllm_paged_decode_fp8_amax": (_i32, [_vp] * 4 + [_i32] + [_vp] * 4 + [_sz] + [_vp] * 6 + [_f32] + [_i32] * 8 + [_vp]),
    "rvllm_paged_decode_static_scratch_bytes": (_sz, []),
    "rvllm_paged_decode_fp8_static_scratch": (_i32, [_vp] * 4 + [_i32] + [_vp] * 2 + [_vp] * 6 + [_f32] + [_i32] * 8 + [_vp]),
    "rvllm_rope_fp8kv_launch": (_i32, [_vp, _vp, _vp, _i32] + [_vp] * 10 + [_i32] * 8 + [_vp]),
    "rvllm_rope_cache_fp8kv_launch": (_i32, [_vp, _vp, _vp, _i32] + [_vp] * 9 + [_i32] * 7 + [_vp]),
    "rvllm_fused_qkv_rmsnorm_launch": (_i32, [_vp] * 8 + [_i32] * 4 + [_f32, _i32, _i32, _vp]),
    "rvllm_fused_norm_add_residual_launch": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _f32, _i32, _vp]),
    "rvllm_residual_scale_launch": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp]),
    "rvllm_logit_softcap_launch": (_i32, [_vp, _i32, _i32, _f32, _i32, _vp]),
    "rvllm_fp8_gemv_blockscale_launch": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "rvllm_embedding_gather_launch": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "rvllm_e4m3_encode_f32": (_i32, [_vp, _vp, _sz, _vp]),
    "rvllm_e4m3_decode_f32": (_i32, [_vp, _vp, _sz, _vp]),
}


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built (``python -m rvllm_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RvllmError(E_ARTIFACT, "load", f"{LIB_PATH} is missing; build it with `python -m rvllm_b200.build`")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here = header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def last_error() -> str:
    return lib().rvllm_b200_last_error().decode()


def check(rc: int, what: str) -> None:
    if rc != 0:
        cls = InvalidArgument if rc == E_INVALID else RvllmError
        raise cls(rc, what, last_error())


def ptr(t):
    """Device pointer of a torch tensor (or None -> NULL); ints pass through."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def current_stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream
