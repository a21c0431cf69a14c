"""Host-side mirror of the reference's launch descriptors for the fused row kernels.

Same names, fields, validation rules and error behaviour as the Rust structs in
v3/crates/rvllm-fused/src/launcher.rs (FusedRmsnormFp8QuantLaunch :175,
FusedAddRmsnormFp8QuantLaunch :96, QuantizeFp8PerTokenLaunch :229,
FusedSiluMulFp8QuantLaunch :280, ArgmaxLaunch :329): ``validate()`` raises
``InvalidArgument`` where the Rust one returns ``Err``, ``launch()`` validates and then
enqueues the kernel on the given stream through the C ABI.  Arguments are torch CUDA
tensors (or raw device addresses); nothing here computes on the host.
"""
from __future__ import annotations

from dataclasses import dataclass

from . import _lib
from ._lib import ACT_GELU_TANH, ACT_SILU, BF16, F16, check, lib, ptr


def _dtype_code(t) -> int:
    import torch

    if isinstance(t, int):
        return t
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.bfloat16:
        return BF16
    raise _lib.InvalidArgument(_lib.E_INVALID, "dtype", f"activations must be float16 or bfloat16, got {t.dtype}")


def _stream(stream):
    return _lib.current_stream() if stream is None else stream


@dataclass
class FusedRmsnormFp8QuantLaunch:
    num_tokens: int
    hidden: int
    eps: float

    def validate(self) -> None:
        check(lib().rvllm_fused_rmsnorm_fp8_quant_validate(self.num_tokens, self.hidden, self.eps),
              "FusedRmsnormFp8QuantLaunch.validate")

    def launch(self, out_fp8, scale, in_hidden, gamma, stream=None, dtype=None) -> None:
        self.validate()
        d = _dtype_code(in_hidden if dtype is None else dtype)
        check(lib().rvllm_fused_rmsnorm_fp8_quant_launch(self.num_tokens, self.hidden, self.eps, ptr(out_fp8),
                                                         ptr(scale), ptr(in_hidden), ptr(gamma), d, _stream(stream)),
              "fused_rmsnorm_fp8_quant")


@dataclass
class FusedAddRmsnormFp8QuantLaunch:
    num_tokens: int
    hidden: int
    eps: float

    def validate(self) -> None:
        check(lib().rvllm_fused_rmsnorm_fp8_quant_validate(self.num_tokens, self.hidden, self.eps),
              "FusedAddRmsnormFp8QuantLaunch.validate")

    def launch(self, out_fp8, scale, residual_out, in_hidden, residual_in, gamma, stream=None, dtype=None) -> None:
        self.validate()
        d = _dtype_code(in_hidden if dtype is None else dtype)
        check(lib().rvllm_fused_add_rmsnorm_fp8_quant_launch(self.num_tokens, self.hidden, self.eps, ptr(out_fp8),
                                                             ptr(scale), ptr(residual_out), ptr(in_hidden),
                                                             ptr(residual_in), ptr(gamma), d, _stream(stream)),
              "fused_add_rmsnorm_fp8_quant")


@dataclass
class QuantizeFp8PerTokenLaunch:
    num_tokens: int
    dim: int

    def validate(self) -> None:
        check(lib().rvllm_quantize_fp8_per_token_validate(self.num_tokens, self.dim),
              "QuantizeFp8PerTokenLaunch.validate")

    def launch(self, out_fp8, scale, in_16, stream=None, dtype=None) -> None:
        self.validate()
        d = _dtype_code(in_16 if dtype is None else dtype)
        check(lib().rvllm_quantize_fp8_per_token_launch(self.num_tokens, self.dim, ptr(out_fp8), ptr(scale),
                                                        ptr(in_16), d, _stream(stream)), "quantize_fp8_per_token")


@dataclass
class FusedActMulFp8QuantLaunch:
    """``act`` = ACT_SILU reproduces FusedSiluMulFp8QuantLaunch; ACT_GELU_TANH the Gemma twin."""

    num_tokens: int
    intermediate: int
    act: int = ACT_SILU

    def validate(self) -> None:
        check(lib().rvllm_fused_act_mul_fp8_quant_validate(self.num_tokens, self.intermediate),
              "FusedActMulFp8QuantLaunch.validate")
        if self.act not in (ACT_SILU, ACT_GELU_TANH):
            raise _lib.InvalidArgument(_lib.E_INVALID, "FusedActMulFp8QuantLaunch.validate", "unknown activation")

    def launch(self, out_fp8, scale, gate_up, stream=None, dtype=None) -> None:
        self.validate()
        d = _dtype_code(gate_up if dtype is None else dtype)
        check(lib().rvllm_fused_act_mul_fp8_quant_launch(self.num_tokens, self.intermediate, self.act, ptr(out_fp8),
                                                         ptr(scale), ptr(gate_up), d, _stream(stream)),
              "fused_act_mul_fp8_quant")


def FusedSiluMulFp8QuantLaunch(num_tokens: int, intermediate: int) -> FusedActMulFp8QuantLaunch:
    return FusedActMulFp8QuantLaunch(num_tokens, intermediate, ACT_SILU)


def FusedGeluMulFp8QuantLaunch(num_tokens: int, intermediate: int) -> FusedActMulFp8QuantLaunch:
    return FusedActMulFp8QuantLaunch(num_tokens, intermediate, ACT_GELU_TANH)


@dataclass
class ArgmaxLaunch:
    num_tokens: int
    vocab: int

    def validate(self) -> None:
        check(lib().rvllm_argmax_validate(self.num_tokens, self.vocab), "ArgmaxLaunch.validate")

    def launch(self, logits, out, stream=None, grid: bool = False) -> None:
        self.validate()
        check(lib().rvllm_argmax_launch(self.num_tokens, self.vocab, ptr(logits), ptr(out), int(grid),
                                        _stream(stream)), "argmax")


def rope_fp8kv(qkv, heads, kv_heads, head_dim, rotary_dim, cos, sin, positions, slot_mapping, q_fp8, q_scale,
               k_cache, v_cache, k_scale_cache, v_scale_cache, stream=None) -> None:
    """RoPE + Q quantisation + paged FP8 KV write over a packed [T, (heads + 2*kv_heads)*head_dim] row."""
    T, stride = qkv.shape
    es = qkv.element_size()
    q_dim, kv_dim = heads * head_dim, kv_heads * head_dim
    base = qkv.data_ptr()
    slots = k_scale_cache.numel() // kv_heads
    check(lib().rvllm_rope_fp8kv_launch(base, base + es * q_dim, base + es * (q_dim + kv_dim), stride, ptr(q_fp8),
                                        ptr(k_cache), ptr(v_cache), ptr(k_scale_cache), ptr(v_scale_cache),
                                        ptr(q_scale), ptr(cos), ptr(sin), ptr(positions), ptr(slot_mapping), T, heads,
                                        kv_heads, head_dim, rotary_dim, cos.shape[0], slots, _dtype_code(qkv),
                                        _stream(stream)), "rope_fp8kv")


def qkv_rope_fp8kv(a_fp8, w_fp8, a_scale, w_scale, heads, kv_heads, head_dim, cos, sin, positions, slot_mapping, q_fp8,
                   q_scale, k_cache, v_cache, k_scale_cache, v_scale_cache, stream=None) -> bool:
    """QKV projection with RoPE + Q quantisation + paged FP8 KV write in the GEMM epilogue.  Returns
    False when the library does not take the shape (the caller then runs the GEMM and rope_fp8kv)."""
    from ._lib import RvllmError
    M, K = a_fp8.shape
    slots = k_scale_cache.numel() // kv_heads
    rc = lib().rvllm_fp8_gemm_qkv_rope_fp8kv(ptr(a_fp8), ptr(w_fp8), ptr(a_scale), ptr(w_scale), M, K, heads, kv_heads,
                                             head_dim, _dtype_code(cos), ptr(q_fp8), ptr(q_scale), ptr(k_cache),
                                             ptr(v_cache), ptr(k_scale_cache), ptr(v_scale_cache), ptr(cos), ptr(sin),
                                             ptr(positions), ptr(slot_mapping), cos.shape[0], slots, _stream(stream))
    if rc == -3:
        return False
    check(rc, "fp8_gemm_qkv_rope_fp8kv")
    return True


def embedding_gather(out, table, token_ids, stream=None) -> None:
    vocab, hidden = table.shape
    check(lib().rvllm_embedding_gather_launch(ptr(out), ptr(table), ptr(token_ids), token_ids.numel(), hidden, vocab,
                                              _stream(stream)), "embedding_gather")
