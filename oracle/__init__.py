"""ctypes binding of the CPU oracle (``liboracle.so``, built from ``oracle.c``).

Test infrastructure only: imported by the test-suite, by ``__graft_entry__.smoke``
and by ``bench.py``'s CPU-baseline / reference arm.  The product package never
imports this module.

All arrays are numpy; 16-bit activations travel as ``uint16`` bit patterns
(``dtype=0`` IEEE half, ``dtype=1`` bfloat16).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

F16, BF16 = 0, 1
MODE_RUST, MODE_CUDA = 0, 1
ACT_SILU, ACT_GELU = 0, 1


def build(force: bool = False) -> str:
    """Compile ``oracle.c`` with the Makefile beside it (gcc, OpenMP)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_h2f.restype = C.c_float
        _lib.orc_h2f.argtypes = [C.c_uint16, C.c_int]
        _lib.orc_f2h.restype = C.c_uint16
        _lib.orc_f2h.argtypes = [C.c_float, C.c_int]
        _lib.orc_e4m3_encode.restype = C.c_uint8
        _lib.orc_e4m3_encode.argtypes = [C.c_float, C.c_int]
        _lib.orc_e4m3_decode.restype = C.c_float
        _lib.orc_e4m3_decode.argtypes = [C.c_uint8]
        _lib.orc_resolve_slot.restype = C.c_longlong
    return _lib


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _chk(rc: int, what: str) -> None:
    if rc != 0:
        raise ValueError(f"oracle {what} rejected its arguments (rc={rc})")


# --------------------------------------------------------------------------- scalars / fp8
def e4m3_encode(x, mode: int = MODE_CUDA) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint8)
    lib().orc_e4m3_encode_n(_p(x), _p(out), C.c_size_t(x.size), C.c_int(mode))
    return out


def e4m3_decode(codes) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    out = np.empty(codes.shape, dtype=np.float32)
    lib().orc_e4m3_decode_n(_p(codes), _p(out), C.c_size_t(codes.size))
    return out


def to_bits16(x, dtype: int) -> np.ndarray:
    """f32 array -> uint16 bit patterns of the 16-bit type (round-to-nearest-even)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dtype == F16:
        return x.astype(np.float16).view(np.uint16)
    u = x.view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def from_bits16(b, dtype: int) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    if dtype == F16:
        return b.view(np.float16).astype(np.float32)
    return (b.astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------- stage 1
def rmsnorm_fp8_quant(x16, gamma16, eps, dtype=F16, mode=MODE_CUDA, block_dim=None,
                      residual16=None):
    T, H = x16.shape
    if block_dim is None:
        block_dim = min(H, 1024)
    out = np.empty((T, H), np.uint8)
    scales = np.empty(T, np.float32)
    res_out = np.empty((T, H), np.uint16) if residual16 is not None else None
    _chk(lib().orc_rmsnorm_fp8_quant(_p(out), _p(scales), _p(res_out), _p(x16), _p(residual16),
                                     _p(gamma16), C.c_float(eps), T, H, dtype, mode, block_dim),
         "rmsnorm_fp8_quant")
    return (out, scales, res_out) if residual16 is not None else (out, scales)


def rmsnorm_f32(x, gamma, eps):
    x = np.ascontiguousarray(x, np.float32)
    gamma = np.ascontiguousarray(gamma, np.float32)
    rows, hidden = x.shape
    out = np.empty_like(x)
    _chk(lib().orc_rmsnorm_f32(_p(x), _p(gamma), C.c_float(eps), hidden, rows, _p(out)), "rmsnorm_f32")
    return out


def quantize_fp8_per_token(x16, dtype=F16, mode=MODE_CUDA):
    T, D = x16.shape
    out = np.empty((T, D), np.uint8)
    scales = np.empty(T, np.float32)
    _chk(lib().orc_quantize_fp8_per_token(_p(out), _p(scales), _p(x16), T, D, dtype, mode),
         "quantize_fp8_per_token")
    return out, scales


def quantize_fp8_per_token_f32(x, mode=MODE_CUDA):
    x = np.ascontiguousarray(x, np.float32)
    T, D = x.shape
    out = np.empty((T, D), np.uint8)
    scales = np.empty(T, np.float32)
    _chk(lib().orc_quantize_fp8_per_token_f32(_p(out), _p(scales), _p(x), T, D, mode),
         "quantize_fp8_per_token_f32")
    return out, scales


# --------------------------------------------------------------------------- stage 2
def act_mul_fp8_quant(gate_up16, act=ACT_SILU, dtype=F16, mode=MODE_CUDA):
    T, two_i = gate_up16.shape
    inter = two_i // 2
    out = np.empty((T, inter), np.uint8)
    scales = np.empty(T, np.float32)
    _chk(lib().orc_act_mul_fp8_quant(_p(out), _p(scales), _p(gate_up16), T, inter, act, dtype, mode),
         "act_mul_fp8_quant")
    return out, scales


def act_mul_fp8_quant_f32(gate_up, act=ACT_SILU, mode=MODE_CUDA):
    gate_up = np.ascontiguousarray(gate_up, np.float32)
    T, two_i = gate_up.shape
    inter = two_i // 2
    out = np.empty((T, inter), np.uint8)
    scales = np.empty(T, np.float32)
    _chk(lib().orc_act_mul_fp8_quant_f32(_p(out), _p(scales), _p(gate_up), T, inter, act, mode),
         "act_mul_fp8_quant_f32")
    return out, scales


def fp8_gemm(a, w, a_scale, w_scale, residual=None, out_kind=F16, acc64=False):
    """out_kind 0 f16 bits, 1 bf16 bits, 2 f32.  a [M,K] u8, w [N,K] u8."""
    M, K = a.shape
    N, K2 = w.shape
    assert K == K2
    out = np.empty((M, N), np.float32 if out_kind == 2 else np.uint16)
    _chk(lib().orc_fp8_gemm(_p(out), _p(a), _p(w), _p(a_scale), _p(w_scale), _p(residual),
                            M, N, K, out_kind, int(acc64)), "fp8_gemm")
    return out


# --------------------------------------------------------------------------- stage 3
def paged_decode_fp8(q, k_cache, v_cache, block_tables, context_lens, scale, heads, kv_heads,
                     head_dim, block_size, window_size_left=-1, k_scale_cache=None,
                     v_scale_cache=None, q_scale_cache=None, q_descale=None, k_descale=None,
                     v_descale=None, precise=False, dtype=F16, num_blocks_total=None):
    batch, max_blocks = block_tables.shape
    if num_blocks_total is None:
        num_blocks_total = k_cache.size // (block_size * kv_heads * head_dim)
    out = np.empty((batch, heads, head_dim), np.uint16)

    def scal(v):
        return None if v is None else np.asarray([v], np.float32)

    qd, kd, vd = scal(q_descale), scal(k_descale), scal(v_descale)
    _chk(lib().orc_paged_decode_fp8(_p(out), _p(q), _p(k_cache), _p(v_cache), _p(block_tables),
                                    _p(context_lens), _p(k_scale_cache), _p(v_scale_cache),
                                    _p(q_scale_cache), _p(qd), _p(kd), _p(vd), C.c_float(scale),
                                    batch, heads, kv_heads, head_dim, block_size, max_blocks,
                                    num_blocks_total, window_size_left, int(precise), dtype),
         "paged_decode_fp8")
    return out


def paged_decode_fp8_split(q, k_cache, v_cache, block_tables, context_lens, scale, heads, kv_heads,
                           head_dim, block_size, num_chunks, k_scale_cache, v_scale_cache,
                           q_scale_cache, window_size_left=-1, dtype=F16, num_blocks_total=None):
    batch, max_blocks = block_tables.shape
    if num_blocks_total is None:
        num_blocks_total = k_cache.size // (block_size * kv_heads * head_dim)
    out = np.empty((batch, heads, head_dim), np.uint16)
    ws = np.empty((batch, heads, num_chunks, head_dim + 2), np.float32)
    _chk(lib().orc_paged_decode_fp8_split(_p(out), _p(ws), _p(q), _p(k_cache), _p(v_cache),
                                          _p(block_tables), _p(context_lens), _p(k_scale_cache),
                                          _p(v_scale_cache), _p(q_scale_cache), C.c_float(scale),
                                          batch, heads, kv_heads, head_dim, block_size, max_blocks,
                                          num_blocks_total, window_size_left, num_chunks, dtype),
         "paged_decode_fp8_split")
    return out, ws


def attended_slots(block_tables, context_lens, block_size, num_blocks_total, window_size_left,
                   max_attend):
    batch, max_blocks = block_tables.shape
    slots = np.empty((batch, max_attend), np.int64)
    _chk(lib().orc_attended_slots(_p(slots), max_attend, _p(block_tables), _p(context_lens), batch,
                                  block_size, max_blocks, num_blocks_total, window_size_left),
         "attended_slots")
    return slots


# --------------------------------------------------------------------------- stage 4
def argmax_f32(logits, mode=MODE_CUDA):
    logits = np.ascontiguousarray(logits, np.float32)
    rows, cols = logits.shape
    out = np.empty(rows, np.int32)
    _chk(lib().orc_argmax_f32(_p(logits), _p(out), rows, cols, mode), "argmax_f32")
    return out


# --------------------------------------------------------------------------- neighbours
def rope_fp8kv(qkv16, heads, kv_heads, head_dim, rotary_dim, cos16, sin16, positions, slot_mapping,
               k_cache, v_cache, k_scale_cache, v_scale_cache, dtype=F16):
    """qkv16 [T, (heads + 2*kv_heads)*head_dim] packed Q|K|V; caches updated in place."""
    T, stride = qkv16.shape
    q_dim, kv_dim = heads * head_dim, kv_heads * head_dim
    flat = qkv16.reshape(-1)
    q_fp8 = np.empty((T, heads, head_dim), np.uint8)
    q_scale = np.empty((T, heads), np.float32)
    max_pos = cos16.shape[0]
    slots = k_scale_cache.size // kv_heads
    base = flat.ctypes.data
    _chk(lib().orc_rope_fp8kv(C.c_void_p(base), C.c_void_p(base + 2 * q_dim),
                              C.c_void_p(base + 2 * (q_dim + kv_dim)), stride, _p(q_fp8),
                              _p(k_cache), _p(v_cache), _p(k_scale_cache), _p(v_scale_cache),
                              _p(q_scale), _p(cos16), _p(sin16), _p(positions), _p(slot_mapping),
                              T, heads, kv_heads, head_dim, rotary_dim, max_pos, slots, dtype),
         "rope_fp8kv")
    return q_fp8, q_scale


def embedding_gather(table16, token_ids):
    vocab, hidden = table16.shape
    token_ids = np.ascontiguousarray(token_ids, np.int32)
    out = np.empty((token_ids.size, hidden), np.uint16)
    _chk(lib().orc_embedding_gather(_p(out), _p(table16), _p(token_ids), token_ids.size, hidden, vocab),
         "embedding_gather")
    return out



# --------------------------------------------------------------------------- Gemma-4 decorations
def qkv_rmsnorm(qkv16, q_gamma16, k_gamma16, heads, kv_heads, head_dim, eps, dtype=F16, block_dim=None):
    """Packed rows [T, stride >= (heads + 2*kv_heads)*head_dim] -> compact (q, k, v) 16-bit bit patterns."""
    T, stride = qkv16.shape
    if block_dim is None:
        block_dim = max(32, min(head_dim, 1024) // 32 * 32)
    q = np.empty((T, heads, head_dim), np.uint16)
    k = np.empty((T, kv_heads, head_dim), np.uint16)
    v = np.empty((T, kv_heads, head_dim), np.uint16)
    _chk(lib().orc_qkv_rmsnorm(_p(q), _p(k), _p(v), _p(qkv16), _p(q_gamma16), _p(k_gamma16), T, heads, kv_heads,
                               head_dim, C.c_float(eps), stride, dtype, block_dim), "qkv_rmsnorm")
    return q, k, v


def norm_add_residual(residual16, gemm_out, gamma16, eps, channelscale=None, layer_scalar16=None, dtype=F16,
                      block_dim=None):
    """residual = (residual + rmsnorm(x) * gamma) * layer_scalar; gemm_out f32 (with channelscale) or 16-bit bits.
    Returns the new residual (the input is not modified)."""
    T, H = residual16.shape
    if block_dim is None:
        block_dim = max(32, min(H, 1024) // 32 * 32)
    out = residual16.copy()
    f32 = gemm_out if gemm_out.dtype == np.float32 else None
    b16 = gemm_out if gemm_out.dtype == np.uint16 else None
    _chk(lib().orc_norm_add_residual(_p(out), _p(f32), _p(b16), _p(channelscale), _p(gamma16), _p(layer_scalar16),
                                     T, H, C.c_float(eps), dtype, block_dim), "norm_add_residual")
    return out


def residual_scale(residual16, scalar16, dtype=F16):
    out = residual16.copy()
    _chk(lib().orc_residual_scale(_p(out), _p(scalar16), C.c_size_t(out.size), dtype), "residual_scale")
    return out


def logit_softcap(logits16, cap, dtype=F16):
    out = logits16.copy()
    _chk(lib().orc_logit_softcap(_p(out), C.c_size_t(out.size), C.c_float(cap), dtype), "logit_softcap")
    return out


def rope_cache_fp8kv(qkv16, heads, kv_heads, head_dim, cos16, sin16, positions, slot_mapping, k_cache, v_cache,
                     q_scale, kv_scale, dtype=F16, q_fp8=None):
    """Llama-form RoPE on packed rows [T, (heads + 2*kv_heads)*head_dim]; caches updated in place; returns q_fp8."""
    T, stride = qkv16.shape
    q_dim, kv_dim = heads * head_dim, kv_heads * head_dim
    flat = qkv16.reshape(-1)
    if q_fp8 is None:
        q_fp8 = np.zeros((T, heads, head_dim), np.uint8)
    base = flat.ctypes.data
    slots = k_cache.size // (kv_heads * head_dim) if kv_heads else 0
    _chk(lib().orc_rope_cache_fp8kv(C.c_void_p(base), C.c_void_p(base + 2 * q_dim), C.c_void_p(base + 2 * (q_dim + kv_dim)),
                                    C.c_longlong(stride), C.c_longlong(stride), _p(q_fp8), _p(k_cache), _p(v_cache),
                                    _p(cos16), _p(sin16), _p(positions), _p(slot_mapping), C.c_float(q_scale),
                                    C.c_float(kv_scale), T, heads, kv_heads, head_dim, cos16.shape[0], slots, dtype),
         "rope_cache_fp8kv")
    return q_fp8


def fp8_gemv_blockscale(w, block_scale, x16, dtype=F16):
    """W [N, K] u8, block_scale f32 [ceil(N/128), ceil(K/128)], x16 [M, K] bits -> out [M, N] bits."""
    N, K = w.shape
    M = x16.shape[0]
    out = np.empty((M, N), np.uint16)
    _chk(lib().orc_fp8_gemv_blockscale(_p(out), _p(w), _p(block_scale), _p(x16), M, N, K, dtype), "fp8_gemv_blockscale")
    return out

def num_threads() -> int:
    return int(lib().orc_num_threads())


def use_all_host_threads() -> int:
    """Run the parallel loops on every CPU this process may use, whatever OMP_NUM_THREADS says
    (torch.distributed.run exports OMP_NUM_THREADS=1 to its workers).  Returns the thread count."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_threads(int(n))
    return num_threads()
