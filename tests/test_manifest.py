"""Artifact-catalogue rules, replaying the reference's own unit tests
(v3/crates/rvllm-kernels/src/manifest.rs:440-535 round trip and digest drift;
loader.rs:179-198 fail-closed loading) plus one case per validation rule of
manifest.rs:282-371.  CPU only: a PTX load must fail closed when no driver is present."""
import hashlib
import json
import os

import pytest


def write_bundle(tmp, entries=None, revision="a" * 40, arch="sm_90", mutate=None, extra_top=None):
    body = b"HELLO PTX"
    (tmp / "argmax.ptx").write_bytes(body)
    ent = {"argmax": {"path": "argmax.ptx", "sha256": hashlib.sha256(body).hexdigest(), "bytes": len(body),
                      "kind": "ptx", "abi": "cuda-ptx-v1"}} if entries is None else entries
    m = {"revision": revision, "arch": arch, "entries": ent}
    if extra_top:
        m.update(extra_top)
    if mutate:
        mutate(m)
    text = json.dumps(m).encode()
    (tmp / "manifest.json").write_bytes(text)
    return str(tmp / "manifest.json"), hashlib.sha256(text).hexdigest()


def load(path, digest, revision="a" * 40, arch="sm_90"):
    from rvllm_b200.manifest import VerifiedManifest
    return VerifiedManifest(path, digest, revision, arch)


def test_sha256_known_answers():
    from rvllm_b200.manifest import sha256_hex
    assert sha256_hex(b"") == "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"
    assert sha256_hex(b"abc") == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"
    blob = bytes(range(256)) * 1000 + b"x" * 55
    assert sha256_hex(blob) == hashlib.sha256(blob).hexdigest()


def test_roundtrip_verify(tmp_path):
    path, digest = write_bundle(tmp_path)
    vm = load(path, digest)
    assert vm.revision == "a" * 40 and vm.arch == "sm_90" and len(vm) == 1
    data, kind, abi = vm.artifact("argmax")
    assert data == b"HELLO PTX" and kind == "ptx" and abi == "cuda-ptx-v1"


def test_drift_rejected(tmp_path):
    from rvllm_b200 import RvllmError
    path, digest = write_bundle(tmp_path)
    (tmp_path / "argmax.ptx").write_bytes(b"HELLO PTY")
    with pytest.raises(RvllmError) as e:
        load(path, digest)
    assert "sha256" in str(e.value)


def test_trust_pins(tmp_path, monkeypatch):
    from rvllm_b200 import RvllmError
    from rvllm_b200.manifest import VerifiedManifest
    path, digest = write_bundle(tmp_path)
    for kw in (dict(digest="0" * 64), dict(revision="b" * 40), dict(arch="sm_100")):
        args = dict(digest=digest, revision="a" * 40, arch="sm_90")
        args.update(kw)
        with pytest.raises(RvllmError):
            load(path, args["digest"], args["revision"], args["arch"])
    for v in ("RVLLM_KERNEL_MANIFEST_SHA256", "RVLLM_RELEASE_REVISION", "RVLLM_KERNEL_ARCH"):
        monkeypatch.delenv(v, raising=False)
    with pytest.raises(RvllmError) as e:       # no pins anywhere: refuse
        VerifiedManifest(path)
    assert "pin" in str(e.value)
    monkeypatch.setenv("RVLLM_KERNEL_MANIFEST_SHA256", digest)
    monkeypatch.setenv("RVLLM_RELEASE_REVISION", "a" * 40)
    monkeypatch.setenv("RVLLM_KERNEL_ARCH", "sm_90")
    assert VerifiedManifest(path).arch == "sm_90"


BAD = [
    ("unknown top-level field", dict(extra_top={"note": "x"})),
    ("unknown entry field", dict(mutate=lambda m: m["entries"]["argmax"].update(extra=1))),
    ("missing entry field", dict(mutate=lambda m: m["entries"]["argmax"].pop("abi"))),
    ("bad revision", dict(revision="xyz1234")),
    ("short revision", dict(revision="abc12")),
    ("unsupported arch", dict(arch="sm_75")),
    ("bad name", dict(mutate=lambda m: m["entries"].update({"a/b": m["entries"].pop("argmax")}))),
    ("uppercase digest", dict(mutate=lambda m: m["entries"]["argmax"].update(sha256="A" * 64))),
    ("kind/abi mismatch", dict(mutate=lambda m: m["entries"]["argmax"].update(abi="rvllm-cuda-so-v1"))),
    ("kind/ext mismatch", dict(mutate=lambda m: m["entries"]["argmax"].update(kind="shared_object", abi="rvllm-cuda-so-v1"))),
    ("absolute path", dict(mutate=lambda m: m["entries"]["argmax"].update(path="/etc/argmax.ptx"))),
    ("escaping path", dict(mutate=lambda m: m["entries"]["argmax"].update(path="../argmax.ptx"))),
    ("wrong size", dict(mutate=lambda m: m["entries"]["argmax"].update(bytes=8))),
    ("zero size", dict(mutate=lambda m: m["entries"]["argmax"].update(bytes=0))),
    ("missing file", dict(mutate=lambda m: m["entries"]["argmax"].update(path="nope.ptx"))),
]


@pytest.mark.parametrize("why,kw", BAD, ids=[b[0] for b in BAD])
def test_rejected_manifests(tmp_path, why, kw):
    from rvllm_b200 import RvllmError
    rev, arch = kw.get("revision", "a" * 40), kw.get("arch", "sm_90")
    path, digest = write_bundle(tmp_path, **kw)
    with pytest.raises(RvllmError):
        load(path, digest, rev, arch)


def test_symlinked_directory_that_leaves_the_root_is_rejected(tmp_path):
    """manifest.rs:226-238 canonicalises the artifact path and requires it under the canonical root: a
    lexically clean `sub/x.ptx` whose `sub` is a symlink out of the bundle must not be read."""
    from rvllm_b200 import RvllmError
    outside = tmp_path / "outside"
    outside.mkdir()
    body = b"HELLO PTX"
    (outside / "x.ptx").write_bytes(body)
    root = tmp_path / "bundle"
    root.mkdir()
    (root / "sub").symlink_to(outside, target_is_directory=True)
    ent = {"x": {"path": "sub/x.ptx", "sha256": hashlib.sha256(body).hexdigest(), "bytes": len(body), "kind": "ptx",
                 "abi": "cuda-ptx-v1"}}
    path, digest = write_bundle(root, entries=ent)
    with pytest.raises(RvllmError) as e:
        load(path, digest)
    assert "escapes" in str(e.value)
    # the same layout with a real directory is fine, and so is a symlink that stays inside the root
    (root / "sub").unlink()
    (root / "sub").mkdir()
    (root / "sub" / "x.ptx").write_bytes(body)
    (root / "alias").symlink_to(root / "sub", target_is_directory=True)
    ent["y"] = dict(ent["x"], path="alias/x.ptx")
    path, digest = write_bundle(root, entries=ent)
    assert len(load(path, digest)) == 2


def test_empty_entries_and_total_size_limit(tmp_path):
    """manifest.rs:190-195 (1..=4096 artifacts) and :217-224 (sum of declared sizes <= 4 x 512 MiB)."""
    from rvllm_b200 import RvllmError
    path, digest = write_bundle(tmp_path, entries={})
    with pytest.raises(RvllmError) as e:
        load(path, digest)
    assert "count" in str(e.value)
    body = b"HELLO PTX"
    big = 512 * 1024 * 1024  # each declared size is legal on its own; five of them exceed the release limit
    ent = {"a%d" % i: {"path": "argmax.ptx", "sha256": hashlib.sha256(body).hexdigest(), "bytes": big, "kind": "ptx",
                       "abi": "cuda-ptx-v1"} for i in range(5)}
    path, digest = write_bundle(tmp_path, entries=ent)
    with pytest.raises(RvllmError) as e:
        load(path, digest)
    assert "total" in str(e.value) or "size" in str(e.value)


def test_duplicate_fields_and_trailing_data_rejected(tmp_path):
    from rvllm_b200 import RvllmError
    path, _ = write_bundle(tmp_path)
    good = open(path, "rb").read()
    for text in (good.replace(b'"arch"', b'"arch": "sm_90", "arch"', 1), good + b" {}", good[:-1]):
        (tmp_path / "manifest.json").write_bytes(text)
        with pytest.raises(RvllmError):
            load(path, hashlib.sha256(text).hexdigest())


def test_oversized_manifest_rejected(tmp_path):
    from rvllm_b200 import RvllmError
    path, _ = write_bundle(tmp_path)
    text = open(path, "rb").read() + b" " * (1024 * 1024)
    (tmp_path / "manifest.json").write_bytes(text)
    with pytest.raises(RvllmError):
        load(path, hashlib.sha256(text).hexdigest())


def test_missing_artifact_name_and_fail_closed_load(tmp_path):
    from rvllm_b200 import RvllmError
    path, digest = write_bundle(tmp_path)
    vm = load(path, digest)
    with pytest.raises(RvllmError) as e:
        vm.artifact("silu")
    assert "silu" in str(e.value)
    with pytest.raises(RvllmError):          # "HELLO PTX" is not PTX, and a host without a CUDA driver cannot load anything: either way an error
        vm.load_ptx("argmax")
    with pytest.raises(RvllmError):
        vm.dlopen("argmax")                  # a PTX artifact is not a shared object


def test_built_bundle_verifies_and_names_every_module():
    """The bundle the build step writes is accepted by the verifier under its own pins."""
    from rvllm_b200 import build
    from rvllm_b200.manifest import VerifiedManifest
    kdir = build.build_ptx()
    mpath = os.path.join(kdir, "manifest.json")
    digest = open(os.path.join(kdir, "manifest.sha256")).read().split()[0]
    vm = VerifiedManifest(mpath, digest, build.REVISION, "sm_100")
    assert vm.arch == "sm_100"
    for stem in build.PTX_MODULES:
        data, kind, abi = vm.artifact(stem)
        assert kind == "ptx" and abi == "cuda-ptx-v1" and b".target sm_100a" in data and b"\x00" not in data
    text = vm.artifact("fused_rmsnorm_fp8_quant")[0]
    for sym in (b"fused_rmsnorm_fp8_quant_kernel", b"fused_add_rmsnorm_fp8_quant_kernel", b"quantize_fp8_per_token_kernel"):
        assert b".entry " + sym in text
    lib_bytes, kind, abi = vm.artifact("libfa_sm89_kernels")
    assert kind == "shared_object" and abi == "rvllm-cuda-so-v2" and lib_bytes[:4] == b"\x7fELF"
    so = vm.dlopen("libfa_sm89_kernels")      # sealed in-memory copy of the verified bytes
    assert so.rvllm_fa_sm89_abi_version() == 2
