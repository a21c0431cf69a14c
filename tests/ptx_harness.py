"""Loads a PTX text module with the CUDA driver API and launches an entry point with
caller-chosen geometry — what the reference's KernelLoader::load_ptx + KernelFn::launch_raw
do (v3/crates/rvllm-kernels/src/module.rs:56-188,267-329).  Used to run (a) the PTX
artifacts this repo builds, at the geometry the reference's Rust launchers fix, and
(b) the reference's own kernels compiled under oracle/_ref, on the same inputs.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OUR_PTX_DIR = os.path.join(ROOT, "rvllm_b200", "kernels", "sm_100")
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


def _check(res, what):
    from cuda.bindings import driver as drv

    err = res[0]
    if err != drv.CUresult.CUDA_SUCCESS:
        raise RuntimeError(f"{what}: {err}")
    return res[1:] if len(res) > 2 else (res[1] if len(res) == 2 else None)


class PtxModule:
    def __init__(self, path: str):
        import torch
        from cuda.bindings import driver as drv

        torch.cuda.init()
        torch.zeros(1, device="cuda")  # make torch's primary context current
        with open(path, "rb") as f:
            text = f.read()
        if b"\x00" in text:
            raise ValueError("PTX artifact has an interior NUL")  # module.rs:280-289
        self._drv = drv
        self._image = text + b"\x00"
        self.module = _check(drv.cuModuleLoadData(self._image), f"cuModuleLoadData({os.path.basename(path)})")
        self._fns = {}

    def function(self, name: str):
        if name not in self._fns:
            self._fns[name] = _check(self._drv.cuModuleGetFunction(self.module, name.encode()),
                                     f"cuModuleGetFunction({name})")
        return self._fns[name]

    def set_max_dynamic_smem(self, name: str, nbytes: int) -> None:
        """What the reference's launch_raw does before a launch that needs more than 48 KiB."""
        _check(self._drv.cuFuncSetAttribute(self.function(name),
                                            self._drv.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                            int(nbytes)), f"cuFuncSetAttribute({name})")

    def launch(self, name, grid, block, smem, args, stream=None):
        """args: list of (ctype, value); tensors are passed as (c_void_p, tensor.data_ptr())."""
        import torch

        fn = self.function(name)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        holders = [ct(v) for ct, v in args]
        ptrs = (ctypes.c_void_p * len(holders))(*[ctypes.addressof(h) for h in holders])
        grid = tuple(grid) + (1,) * (3 - len(grid))
        block = tuple(block) + (1,) * (3 - len(block))
        _check(self._drv.cuLaunchKernel(fn, *grid, *block, smem, stream, ctypes.addressof(ptrs), 0),
               f"cuLaunchKernel({name})")


def P(t):
    return (ctypes.c_void_p, t.data_ptr())


def NULL():
    return (ctypes.c_void_p, 0)


def I(v):
    return (ctypes.c_int, int(v))


def F(v):
    return (ctypes.c_float, float(v))


def ours(stem: str) -> PtxModule:
    return PtxModule(os.path.join(OUR_PTX_DIR, stem + ".ptx"))


def reference(stem: str) -> PtxModule:
    return PtxModule(os.path.join(REF_DIR, stem + ".ptx"))


def have_reference() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "fused_rmsnorm_fp8_quant.ptx"))


def fp8_codes_adjacent(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Elementwise: True where two E4M3 codes are equal or neighbours on the number line
    (+0 and -0 count as the same point)."""
    def ordinal(c):
        c = c.astype(np.int32)
        mag = c & 0x7F
        return np.where(c & 0x80, -mag, mag)
    return np.abs(ordinal(got) - ordinal(want)) <= 1
