"""FP8-KV paged GQA decode attention: host mirror of PagedDecodeParams and
PagedDecodeFp8Launcher (v3/crates/rvllm-attention/src/decode.rs:14-102,458-711)."""
from __future__ import annotations

from dataclasses import dataclass

from . import _lib
from ._lib import BF16, F16, check, lib, ptr


@dataclass
class PagedDecodeParams:
    num_seqs: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    block_size: int
    max_blocks_per_seq: int
    num_blocks_total: int
    scale: float
    window_size_left: int = -1

    def validate(self) -> None:
        check(lib().rvllm_paged_decode_fp8_validate(self.num_seqs, self.num_heads, self.num_kv_heads, self.head_dim,
                                                    self.block_size, self.max_blocks_per_seq, self.num_blocks_total,
                                                    self.window_size_left, self.scale), "PagedDecodeParams.validate")

    def workspace_bytes(self) -> int:
        n = int(lib().rvllm_paged_decode_workspace_size(self.num_seqs, self.num_heads, self.num_kv_heads, self.head_dim))
        if n == 2 ** 64 - 1:
            raise _lib.InvalidArgument(_lib.E_INVALID, "workspace_bytes", "shape rejected by the workspace query")
        return n

    def max_chunks(self) -> int:
        return int(lib().rvllm_paged_decode_max_chunks(self.num_seqs, self.num_kv_heads))


class PagedDecodeFp8Launcher:
    """launch(): q [B, H, HD] u8, caches [blocks, block_size, KVH, HD] u8, out [B, H, HD] 16-bit."""

    def __init__(self, params: PagedDecodeParams):
        self.params = params

    def launch(self, q_fp8, k_cache, v_cache, out, block_tables, context_lens, workspace=None, k_scale_cache=None,
               v_scale_cache=None, q_scale_cache=None, q_descale=None, k_descale=None, v_descale=None,
               stream=None) -> None:
        import torch

        p = self.params
        p.validate()
        dt = F16 if out.dtype == torch.float16 else BF16
        ws_len = workspace.numel() * workspace.element_size() if workspace is not None else 0
        check(lib().rvllm_paged_decode_fp8(ptr(q_fp8), ptr(k_cache), ptr(v_cache), ptr(out), dt, ptr(block_tables),
                                           ptr(context_lens), ptr(workspace), ws_len, ptr(k_scale_cache),
                                           ptr(v_scale_cache), ptr(q_scale_cache), ptr(q_descale), ptr(k_descale),
                                           ptr(v_descale), p.scale, p.num_seqs, p.num_heads, p.num_kv_heads,
                                           p.head_dim, p.block_size, p.max_blocks_per_seq, p.num_blocks_total,
                                           p.window_size_left, _lib.current_stream() if stream is None else stream),
              "paged_decode_fp8")


    def quant_workspace_bytes(self) -> int:
        p = self.params
        return int(lib().rvllm_paged_decode_quant_workspace_size(p.num_seqs, p.num_heads, p.num_kv_heads, p.head_dim))

    def launch_quant(self, q_fp8, k_cache, v_cache, out_fp8, out_scale, round_dtype, block_tables, context_lens,
                     workspace, k_scale_cache=None, v_scale_cache=None, q_scale_cache=None, q_descale=None,
                     k_descale=None, v_descale=None, stream=None) -> None:
        """Attention + LSE combine + per-token FP8 quantisation of the [heads*head_dim] row in one call."""
        p = self.params
        p.validate()
        check(lib().rvllm_paged_decode_fp8_quant(ptr(q_fp8), ptr(k_cache), ptr(v_cache), ptr(out_fp8), ptr(out_scale),
                                                 round_dtype, ptr(block_tables), ptr(context_lens), ptr(workspace),
                                                 workspace.numel() * workspace.element_size(), ptr(k_scale_cache),
                                                 ptr(v_scale_cache), ptr(q_scale_cache), ptr(q_descale), ptr(k_descale),
                                                 ptr(v_descale), p.scale, p.num_seqs, p.num_heads, p.num_kv_heads,
                                                 p.head_dim, p.block_size, p.max_blocks_per_seq, p.num_blocks_total,
                                                 p.window_size_left, _lib.current_stream() if stream is None else stream),
              "paged_decode_fp8_quant")
