"""Host mirror of the reference's KernelManifest / KernelLoader
(v3/crates/rvllm-kernels/src/manifest.rs:157-371, loader.rs:51-114): verify a manifest against
the three trust pins, hand out verified artifact bytes, load PTX modules and launch entry points
with caller-chosen geometry.  Everything is checked in the C library; this file only marshals."""
from __future__ import annotations

import ctypes as C

from . import _lib
from ._lib import check, lib

_bound = False


def _bind():
    global _bound
    L = lib()
    if not _bound:
        vp, cp, u32 = C.c_void_p, C.c_char_p, C.c_uint32
        L.rvllm_sha256_hex.argtypes = [vp, C.c_size_t, cp]
        L.rvllm_manifest_load_and_verify.argtypes = [C.POINTER(vp), cp, cp, cp, cp]
        L.rvllm_manifest_free.argtypes = [vp]
        L.rvllm_manifest_free.restype = None
        L.rvllm_manifest_arch.argtypes = [vp]
        L.rvllm_manifest_arch.restype = cp
        L.rvllm_manifest_revision.argtypes = [vp]
        L.rvllm_manifest_revision.restype = cp
        L.rvllm_manifest_entry_count.argtypes = [vp]
        L.rvllm_manifest_artifact.argtypes = [vp, cp, C.POINTER(vp), C.POINTER(C.c_uint64), C.POINTER(C.c_int),
                                              C.POINTER(cp)]
        L.rvllm_module_load_ptx.argtypes = [C.POINTER(vp), vp, cp]
        L.rvllm_module_unload.argtypes = [vp]
        L.rvllm_module_unload.restype = None
        L.rvllm_module_get_function.argtypes = [vp, cp, C.POINTER(vp)]
        L.rvllm_launch_raw.argtypes = [vp] + [u32] * 7 + [vp, vp]
        L.rvllm_manifest_dlopen.argtypes = [vp, cp, C.POINTER(vp)]
        _bound = True
    return L


def sha256_hex(data: bytes) -> str:
    out = C.create_string_buffer(65)
    check(_bind().rvllm_sha256_hex(data, len(data), out), "sha256")
    return out.value.decode()


def _b(s):
    return None if s is None else s.encode()


class VerifiedManifest:
    """KernelManifest::load_and_verify_trusted: pins given as arguments, or taken from
    RVLLM_KERNEL_MANIFEST_SHA256 / RVLLM_RELEASE_REVISION / RVLLM_KERNEL_ARCH when None."""

    def __init__(self, manifest_path: str, sha256=None, revision=None, arch=None):
        self._L = _bind()
        h = C.c_void_p()
        check(self._L.rvllm_manifest_load_and_verify(C.byref(h), manifest_path.encode(), _b(sha256), _b(revision),
                                                     _b(arch)), "manifest load_and_verify")
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            self._L.rvllm_manifest_free(self._h)
            self._h = None

    __del__ = close

    @property
    def arch(self):
        return self._L.rvllm_manifest_arch(self._h).decode()

    @property
    def revision(self):
        return self._L.rvllm_manifest_revision(self._h).decode()

    def __len__(self):
        return self._L.rvllm_manifest_entry_count(self._h)

    def artifact(self, name: str):
        """(bytes, kind, abi) of a verified artifact; kind is "ptx" or "shared_object"."""
        p, n, k, abi = C.c_void_p(), C.c_uint64(), C.c_int(), C.c_char_p()
        check(self._L.rvllm_manifest_artifact(self._h, name.encode(), C.byref(p), C.byref(n), C.byref(k), C.byref(abi)),
              "manifest artifact")
        return C.string_at(p.value, n.value), ("ptx", "shared_object")[k.value], abi.value.decode()

    def load_ptx(self, name: str) -> "Module":
        return Module(self, name)

    def dlopen(self, name: str) -> C.CDLL:
        h = C.c_void_p()
        check(self._L.rvllm_manifest_dlopen(self._h, name.encode(), C.byref(h)), "manifest dlopen")
        return C.CDLL(None, handle=h.value)


class Module:
    """KernelLoader::load_ptx + LoadedModule::get_function + KernelFn::launch_raw."""

    def __init__(self, manifest: VerifiedManifest, name: str):
        self._L = manifest._L
        h = C.c_void_p()
        check(self._L.rvllm_module_load_ptx(C.byref(h), manifest._h, name.encode()), "load_ptx")
        self._h = h
        self._fns = {}

    def close(self):
        if getattr(self, "_h", None):
            self._L.rvllm_module_unload(self._h)
            self._h = None

    def function(self, symbol: str) -> int:
        if symbol not in self._fns:
            f = C.c_void_p()
            check(self._L.rvllm_module_get_function(self._h, symbol.encode(), C.byref(f)), "get_function")
            self._fns[symbol] = f.value
        return self._fns[symbol]

    def launch_raw(self, symbol, grid, block, smem, args, stream=None):
        """args: list of (ctype, value) pairs, e.g. (c_void_p, tensor.data_ptr())."""
        grid = tuple(grid) + (1,) * (3 - len(grid))
        block = tuple(block) + (1,) * (3 - len(block))
        holders = [ct(v) for ct, v in args]
        ptrs = (C.c_void_p * len(holders))(*[C.addressof(h) for h in holders])
        s = _lib.current_stream() if stream is None else stream
        check(self._L.rvllm_launch_raw(self.function(symbol), *grid, *block, smem, s, ptrs), "launch_raw")
