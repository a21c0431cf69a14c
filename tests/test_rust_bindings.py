"""The Rust FFI crate is reviewed-only source (no Rust toolchain where this is built), so it is checked
against what is built: the generated table is current, every function in it is exported by
librvllm_b200.so, and its parameter count equals the C header's and the ctypes table's."""
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CRATE = os.path.join(ROOT, "rvllm-b200-sys")


def rust_functions():
    text = open(os.path.join(CRATE, "src", "lib.rs")).read()
    out = {}
    for m in re.finditer(r"pub fn ([A-Za-z0-9_]+)\((.*?)\)( -> [^;]+)?;", text):
        args = [a for a in m.group(2).split(",") if a.strip()]
        out[m.group(1)] = len(args)
    return out


def test_generated_table_is_current():
    assert subprocess.call([sys.executable, os.path.join(CRATE, "gen_bindings.py"), "--check"]) == 0, \
        "rvllm-b200-sys/src/lib.rs is stale: run python rvllm-b200-sys/gen_bindings.py"


def test_every_rust_symbol_is_exported_with_the_same_arity():
    sys.path.insert(0, CRATE)
    import gen_bindings as g
    from rvllm_b200 import _lib, build
    build.build_library()
    L = _lib.lib()
    rust = rust_functions()
    assert len(rust) > 80
    header = {}
    for h in g.HEADERS:
        for name, _, params in g.parse_prototypes(open(os.path.join(ROOT, "include", h)).read()):
            header[name] = len(params)
    assert set(rust) == set(header)
    for name, n in rust.items():
        assert hasattr(L, name), name + " is not exported by librvllm_b200.so"
        assert n == header[name], name
        if name in _lib.SIGNATURES:                      # the ctypes table the GPU tests call through
            assert n == len(_lib.SIGNATURES[name][1]), name


def test_patches_name_real_reference_lines():
    """Each patch cites the file it changes; the hunks keep the reference's own identifiers."""
    for fn, needle in (("0001-cutlass-backend-load-for-sm100.diff", "CutlassBackend::Absent"),
                       ("0002-attention-backend-sm100-fa-sm89-so.diff", "use_fa2_ptx"),
                       ("0003-policy-for-sm100.diff", "VariantId(100)")):
        text = open(os.path.join(CRATE, "patches", fn)).read()
        assert needle in text and "--- a/v3/crates/" in text and "+++ b/v3/crates/" in text
