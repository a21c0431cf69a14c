"""rvllm_b200 — hand-written sm_100a kernels for rvLLM's FP8 decode hot path behind a C ABI.

The package holds the CUDA sources (``csrc/``), the build step (``build.py``) and thin
host-side mirrors of the reference's launch descriptors.  Importing it never compiles or
loads anything; the shared library is loaded on first use and its absence is an error.
"""
from ._lib import (ACT_GELU_TANH, ACT_SILU, BF16, F16, OUT_BF16, OUT_F16, OUT_F32, InvalidArgument, RvllmError,
                   lib)

__all__ = ["ACT_GELU_TANH", "ACT_SILU", "BF16", "F16", "OUT_BF16", "OUT_F16", "OUT_F32", "InvalidArgument",
           "RvllmError", "lib"]
