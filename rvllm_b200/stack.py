"""Python handle of the decode stack (``include/rvllm_b200_stack.h``) and a builder of
synthetic random-init weights with the reference's layouts: FP8 E4M3 weights ``[N, K]`` with a
per-output-channel f32 scale (absmax / 448), 16-bit norm gains and embedding table.

torch is used only to own device memory and to draw / quantise the random weights at set-up;
every step of the decode runs in the C library's CUDA graph.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

from . import _lib
from ._lib import ACT_SILU, BF16, F16, check, lib


class StackConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("hidden", "ffn", "vocab", "num_layers", "heads", "kv_heads",
                                       "sliding_head_dim", "global_head_dim", "sliding_window", "global_every",
                                       "act", "dtype", "batch", "block_size", "max_context", "max_steps",
                                       "prompt_len", "gemm_impl")] + \
               [("rms_eps", C.c_float), ("rope_theta", C.c_float), ("seed", C.c_uint64), ("kv_pool_blocks", C.c_int), ("fused_block", C.c_int),
                ("fused_argmax", C.c_int), ("logit_softcap", C.c_float)]


class LayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("attn_norm_gamma", "qkv_w", "qkv_scale", "o_w", "o_scale",
                                          "mlp_norm_gamma", "gateup_w", "gateup_scale", "down_w", "down_scale")]


class HeadWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("embedding", "final_norm_gamma", "lm_head_w", "lm_head_scale")]


_bound = False


def _bind():
    global _bound
    L = lib()
    if _bound:
        return L
    vp, i32 = C.c_void_p, C.c_int
    L.rvllm_stack_config_validate.argtypes = [C.POINTER(StackConfig)]
    L.rvllm_stack_device_bytes.argtypes = [C.POINTER(StackConfig)]
    L.rvllm_stack_device_bytes.restype = C.c_uint64
    L.rvllm_stack_create.argtypes = [C.POINTER(vp), C.POINTER(StackConfig), C.POINTER(LayerWeights),
                                     C.POINTER(HeadWeights)]
    L.rvllm_stack_destroy.argtypes = [vp]
    L.rvllm_stack_destroy.restype = None
    L.rvllm_stack_reset.argtypes = [vp, vp]
    L.rvllm_stack_run.argtypes = [vp, i32]
    L.rvllm_stack_seed_context.argtypes = [vp, i32]
    L.rvllm_stack_seed_contexts.argtypes = [vp, vp]
    L.rvllm_stack_run_eager.argtypes = [vp, i32]
    L.rvllm_stack_sync.argtypes = [vp]
    L.rvllm_stack_step_host.argtypes = [vp, vp, vp]
    L.rvllm_stack_read_tokens.argtypes = [vp, i32, i32, vp]
    L.rvllm_stack_steps_done.argtypes = [vp]
    L.rvllm_stack_launches_per_step.argtypes = [vp]
    L.rvllm_stack_stream.argtypes = [vp]
    L.rvllm_stack_stream.restype = vp
    L.rvllm_stack_debug_read.argtypes = [vp, i32, vp, C.c_size_t]
    _bound = True
    return L


def gemma31b_shape(batch: int, **over) -> dict:
    """The 31B-class decode shape of the benchmark: 62 layers, 5 sliding : 1 global, hidden 5376,
    ffn 21504, vocab 262144, 32 query / 16 KV heads, sliding head_dim 128 (window 1024), global 256.
    fused_block is off: at this shape the one-launch layer block measured slower than the chain of stand-alone
    kernels under programmatic dependent launch (112 us against about 92 us per layer)."""
    cfg = dict(hidden=5376, ffn=21504, vocab=262144, num_layers=62, heads=32, kv_heads=16, sliding_head_dim=128,
               global_head_dim=256, sliding_window=1024, global_every=6, act=ACT_SILU, dtype=BF16, batch=batch,
               block_size=16, max_context=1024, max_steps=1024, prompt_len=512, gemm_impl=0, rms_eps=1e-6,
               rope_theta=10000.0, seed=3, kv_pool_blocks=0, fused_block=0, fused_argmax=1, logit_softcap=0.0)
    cfg.update(over)
    return cfg


def tiny_shape(batch: int = 4, **over) -> dict:
    """The CPU-checkable single-layer configuration: hidden 512, 8 query / 4 KV heads, head_dim 64,
    ffn 2048, context 128."""
    cfg = dict(hidden=512, ffn=2048, vocab=2048, num_layers=1, heads=8, kv_heads=4, sliding_head_dim=64,
               global_head_dim=64, sliding_window=64, global_every=1, act=ACT_SILU, dtype=F16, batch=batch,
               block_size=16, max_context=512, max_steps=512, prompt_len=128, gemm_impl=0, rms_eps=1e-6,
               rope_theta=10000.0, seed=0, kv_pool_blocks=0, fused_block=1, fused_argmax=0, logit_softcap=0.0)
    cfg.update(over)
    return cfg


@dataclass
class Weights:
    """Device tensors of a random-init model; kept alive for as long as a stack uses them."""
    layers: list = field(default_factory=list)
    head: dict = field(default_factory=dict)

    def nbytes(self) -> int:
        n = sum(t.numel() * t.element_size() for l in self.layers for t in l.values())
        return n + sum(t.numel() * t.element_size() for t in self.head.values())


def _quant_weight(n, k, gen, std, share=None):
    """[n, k] N(0, std) -> (fp8 bytes as uint8 tensor, per-row scale).  Drawn in row chunks so
    the f32 staging stays small."""
    import torch

    w8 = torch.empty((n, k), dtype=torch.uint8, device="cuda")
    sc = torch.empty(n, dtype=torch.float32, device="cuda")
    rows = max(1, (64 << 20) // (4 * k))
    for r0 in range(0, n, rows):
        r1 = min(n, r0 + rows)
        x = torch.randn((r1 - r0, k), generator=gen, device="cuda", dtype=torch.float32) * std
        s = (x.abs().amax(dim=1) / 448.0).clamp_min(1e-12)
        sc[r0:r1] = s
        w8[r0:r1] = (x / s[:, None]).to(torch.float8_e4m3fn).view(torch.uint8)
    return w8, sc


def random_weights(cfg: dict, seed: int = 3, std: float = 0.02) -> Weights:
    import torch

    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    tdt = torch.float16 if cfg["dtype"] == F16 else torch.bfloat16
    H, F = cfg["hidden"], cfg["ffn"]
    w = Weights()
    for l in range(cfg["num_layers"]):
        is_global = cfg["global_every"] != 0 and (l + 1) % cfg["global_every"] == 0
        hd = cfg["global_head_dim"] if is_global else cfg["sliding_head_dim"]
        q_dim, kv_dim = cfg["heads"] * hd, cfg["kv_heads"] * hd
        layer = {}
        layer["attn_norm_gamma"] = torch.ones(H, dtype=tdt, device="cuda")
        layer["qkv_w"], layer["qkv_scale"] = _quant_weight(q_dim + 2 * kv_dim, H, gen, std)
        layer["o_w"], layer["o_scale"] = _quant_weight(H, q_dim, gen, std)
        layer["mlp_norm_gamma"] = torch.ones(H, dtype=tdt, device="cuda")
        layer["gateup_w"], layer["gateup_scale"] = _quant_weight(2 * F, H, gen, std)
        layer["down_w"], layer["down_scale"] = _quant_weight(H, F, gen, std)
        w.layers.append(layer)
    emb = torch.empty((cfg["vocab"], H), dtype=tdt, device="cuda")
    rows = max(1, (64 << 20) // (4 * H))
    for r0 in range(0, cfg["vocab"], rows):
        r1 = min(cfg["vocab"], r0 + rows)
        emb[r0:r1] = torch.randn((r1 - r0, H), generator=gen, device="cuda", dtype=torch.float32).to(tdt)
    w.head["embedding"] = emb
    w.head["final_norm_gamma"] = torch.ones(H, dtype=tdt, device="cuda")
    w.head["lm_head_w"], w.head["lm_head_scale"] = _quant_weight(cfg["vocab"], H, gen, std)
    # the tensors are written by kernels on torch's stream; a decode stack runs on its own stream and does not
    # wait for them, so they must be complete before they are handed over
    torch.cuda.synchronize()
    return w


class DecodeStack:
    def __init__(self, cfg: dict, weights: Weights):
        L = _bind()
        self.cfg = dict(cfg)
        self.weights = weights  # keeps the device memory alive
        if weights.layers:
            import torch

            torch.cuda.synchronize()  # weights may still be in flight on another stream (see rvllm_stack_create)
        self._c = StackConfig(**cfg)
        check(L.rvllm_stack_config_validate(C.byref(self._c)), "stack config")
        layers = (LayerWeights * cfg["num_layers"])()
        for i, lw in enumerate(weights.layers):
            for name, _ in LayerWeights._fields_:
                setattr(layers[i], name, lw[name].data_ptr())
        head = HeadWeights(**{n: weights.head[n].data_ptr() for n, _ in HeadWeights._fields_})
        h = C.c_void_p()
        check(L.rvllm_stack_create(C.byref(h), C.byref(self._c), layers, C.byref(head)), "stack create")
        self._h = h
        self._L = L

    def close(self):
        if getattr(self, "_h", None):
            self._L.rvllm_stack_destroy(self._h)
            self._h = None

    __del__ = close

    @property
    def batch(self) -> int:
        return self.cfg["batch"]

    def device_bytes(self) -> int:
        return int(self._L.rvllm_stack_device_bytes(C.byref(self._c)))

    def reset(self, prompt=None) -> None:
        import numpy as np

        p = None
        if prompt is not None:
            prompt = np.ascontiguousarray(prompt, np.int32)
            assert prompt.shape == (self.cfg["batch"], self.cfg["prompt_len"])
            p = prompt.ctypes.data
        check(self._L.rvllm_stack_reset(self._h, p), "stack reset")

    def seed_context(self, context: int) -> None:
        check(self._L.rvllm_stack_seed_context(self._h, context), "stack seed context")

    def seed_contexts(self, contexts) -> None:
        """One context length per sequence (a ragged batch); numpy int32 [batch]."""
        import numpy as np

        contexts = np.ascontiguousarray(contexts, np.int32)
        assert contexts.shape == (self.cfg["batch"],)
        check(self._L.rvllm_stack_seed_contexts(self._h, contexts.ctypes.data), "stack seed contexts")

    def run(self, n: int, eager: bool = False) -> None:
        fn = self._L.rvllm_stack_run_eager if eager else self._L.rvllm_stack_run
        check(fn(self._h, n), "stack run")

    def sync(self) -> None:
        check(self._L.rvllm_stack_sync(self._h), "stack sync")

    def step_host(self, tokens_in, tokens_out) -> None:
        """tokens_in / tokens_out: numpy int32 [batch] (tokens_in may be None)."""
        check(self._L.rvllm_stack_step_host(self._h, None if tokens_in is None else tokens_in.ctypes.data,
                                            tokens_out.ctypes.data), "stack step")

    def tokens(self, first: int = 0, count=None):
        import numpy as np

        done = self._L.rvllm_stack_steps_done(self._h)
        count = done - first if count is None else count
        out = np.zeros((max(count, 0), self.cfg["batch"]), np.int32)
        if count > 0:
            n = self._L.rvllm_stack_read_tokens(self._h, first, count, out.ctypes.data)
            if n < 0:
                check(n, "read tokens")
            out = out[:n]
        return out

    def launches_per_step(self) -> int:
        return int(self._L.rvllm_stack_launches_per_step(self._h))

    def stream(self) -> int:
        return int(self._L.rvllm_stack_stream(self._h))

    def debug_read(self, what: int):
        import numpy as np

        B = self.cfg["batch"]
        if what == 0:
            out = np.empty((B, self.cfg["hidden"]), np.uint16)
        elif what == 1:
            out = np.empty((B, self.cfg["vocab"]), np.float32)
        else:
            out = np.empty(B, np.int32)
        check(self._L.rvllm_stack_debug_read(self._h, what, out.ctypes.data, out.nbytes), "debug read")
        return out
