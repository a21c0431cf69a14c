"""Builds the sm_100a artifacts of the package, in-tree:

  rvllm_b200/librvllm_b200.so        the C-ABI shared library (all kernels + host launchers)
  rvllm_b200/kernels/sm_100/*.ptx    PTX modules carrying the reference's entry-point names
  rvllm_b200/kernels/sm_100/manifest.json (+ manifest.sha256)

nvcc cross-compiles without a GPU.  Run as ``python -m rvllm_b200.build``.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import json
import os
import re
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "librvllm_b200.so")
KDIR = os.path.join(HERE, "kernels", "sm_100")
OBJ = os.path.join(HERE, "build")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
          "-ccbin", "/usr/bin/g++"]

# translation units of the shared library
LIB_UNITS = ["abi_core.cu", "abi_gemm.cu", "abi_attn.cu", "manifest.cpp", "decode_stack.cu"]
# PTX module stem (what the reference manifest calls the artifact) -> source file
PTX_MODULES = {
    "fused_rmsnorm_fp8_quant": "rowq_rmsnorm.cu",
    "fused_silu_fp8_quant": "rowq_silu.cu",
    "fused_gelu_mul_fp8_quant": "rowq_gelu.cu",
    "argmax": "greedy_argmax.cu",
    "embedding_gather_f16": "rope_kv_write.cu",
    "fused_rope_partial_fp8kv": "rope_kv_write.cu",
    "flash_attention": "fa2_decode_fp8kv.cu",
    # Gemma-4 decorations, soft cap and the Llama-form RoPE: one source, the reference's five module names
    "fused_qkv_rmsnorm": "rowq_gemma.cu",
    "fused_norm_add_residual_f16": "rowq_gemma.cu",
    "residual_scale_f16": "rowq_gemma.cu",
    "logit_softcap": "rowq_gemma.cu",
    "fused_rope_cache_fp8kv": "rowq_gemma.cu",
    # 128 x 128 block-scaled FP8 weights x 16-bit activations (the f16-input warp-per-row entry point only)
    "fp8_gemv": "rowq_blockscale.cu",
}
REVISION = "b200f8e4d0c1"


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), r.stdout))
    return r.stdout


# Kernels whose launch plan counts on three 192-thread CTAs per SM (18 warps): each of the SM's four
# schedulers owns 16384 registers, so a warp may take at most 16384 / 5 / 32 = 102 -> 96 registers per thread
# (allocated in eights).  One register more and only 16 warps fit: two CTAs per SM, the 336-CTA launches of
# the decode step run in two waves (measured: down projection 25 -> 37 us).
REG_BUDGET = 96
REG_BUDGET_KERNELS = (r"fp8_gemm_tc_kernelILi16E", r"fp8_gemm_tc_kernelILi32E", r"fp8_gemm_tc_kernelILi64E",
                      r"fp8_gemm_tc_kernelILi128E", r"fp8_layer_block_kernel")


def check_register_budget(ptxas_log):
    """Raises if a kernel named in REG_BUDGET_KERNELS was compiled with more than REG_BUDGET registers."""
    over = []
    for m in re.finditer(r"Compiling entry function '([^']+)'(?:.*\n)*?.*Used (\d+) registers", ptxas_log):
        name, regs = m.group(1), int(m.group(2))
        if any(re.search(k, name) for k in REG_BUDGET_KERNELS) and regs > REG_BUDGET:
            over.append("%s: %d registers" % (name, regs))
    if over:
        raise RuntimeError("register budget of %d exceeded (third CTA per SM lost):\n  %s" % (REG_BUDGET, "\n  ".join(over)))


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _all_sources():
    out = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    out.append(os.path.join(os.path.dirname(HERE), "include", "rvllm_b200.h"))
    return [f for f in out if os.path.isfile(f)]


def build_library(force=False, verbose=False):
    srcs = _all_sources()
    units = [u for u in LIB_UNITS if os.path.exists(os.path.join(CSRC, u))]
    if not force and not _newer(LIB, srcs):
        return LIB
    os.makedirs(OBJ, exist_ok=True)

    def compile_one(unit):
        obj = os.path.join(OBJ, os.path.splitext(unit)[0] + ".o")
        cmd = [NVCC, *ARCH, *COMMON, "-Xptxas=-v", "-c", os.path.join(CSRC, unit), "-o", obj]
        if os.environ.get("RVLLM_TC_TRACE", "0") not in ("", "0"):
            cmd.insert(1, "-DRVLLM_TC_TRACE=1")  # timing-aid build: the GEMM's %globaltimer stamps (bench.py --gemm-trace)
        log = _run(cmd)
        check_register_budget(log)
        return obj, log

    with cf.ThreadPoolExecutor(max_workers=len(units)) as ex:
        results = list(ex.map(compile_one, units))
    if verbose:
        for _, log in results:
            sys.stdout.write(log)
    objs = [o for o, _ in results]
    _run([NVCC, *ARCH, "-shared", "-cudart", "static", "-ccbin", "/usr/bin/g++", "-o", LIB, *objs, "-ldl"])
    return LIB


def _sha256(path):
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def build_ptx(force=False):
    """PTX text modules + manifest.json in the reference's schema
    (v3/crates/rvllm-kernels/src/manifest.rs:63-95; kernels/gen_manifest.sh:44-71)."""
    os.makedirs(KDIR, exist_ok=True)
    srcs = _all_sources()
    entries = {}
    for stem, src in PTX_MODULES.items():
        out = os.path.join(KDIR, stem + ".ptx")
        if force or _newer(out, srcs):
            _run([NVCC, "-ptx", "-arch=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-ccbin", "/usr/bin/g++",
                  os.path.join(CSRC, src), "-o", out])
        entries[stem] = {"path": stem + ".ptx", "sha256": _sha256(out), "bytes": os.path.getsize(out),
                         "kind": "ptx", "abi": "cuda-ptx-v1"}
    # the shared library is catalogued under the names the reference loader looks up
    so_copy = os.path.join(KDIR, "librvllm_b200.so")
    if os.path.exists(LIB):
        if force or _newer(so_copy, [LIB]):
            shutil.copyfile(LIB, so_copy)
        for name, abi in (("libcutlass_kernels", "rvllm-cuda-so-v1"), ("libfa_sm89_kernels", "rvllm-cuda-so-v2")):
            entries[name] = {"path": "librvllm_b200.so", "sha256": _sha256(so_copy),
                             "bytes": os.path.getsize(so_copy), "kind": "shared_object", "abi": abi}
    manifest = {"revision": REVISION, "arch": "sm_100", "entries": dict(sorted(entries.items()))}
    mpath = os.path.join(KDIR, "manifest.json")
    text = json.dumps(manifest, indent=2, sort_keys=True) + "\n"
    if not os.path.exists(mpath) or open(mpath).read() != text:
        with open(mpath, "w") as f:
            f.write(text)
    with open(os.path.join(KDIR, "manifest.sha256"), "w") as f:
        f.write(hashlib.sha256(text.encode()).hexdigest() + "  manifest.json\n")
    return KDIR


def build_all(force=False, verbose=False):
    build_library(force=force, verbose=verbose)
    build_ptx(force=force)
    return LIB


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
