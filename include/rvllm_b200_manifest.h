/*
 * rvllm_b200 artifact catalogue — C restatement of the reference's kernel-manifest boundary:
 * KernelManifest::load_and_verify_trusted and KernelLoader::{load_ptx, so_artifact}
 * (v3/crates/rvllm-kernels/src/manifest.rs:157-371, loader.rs:51-114, module.rs:56-329) and the
 * generic launcher launch_raw (v3/crates/rvllm-fused/src/launch_raw.rs:17-161).
 *
 * Same schema and rules: {"revision", "arch", "entries": {name: {"path", "sha256", "bytes",
 * "kind", "abi"}}}; unknown or duplicate fields are rejected; manifest <= 1 MiB, artifacts
 * <= 512 MiB, <= 4096 entries; names and ABI ids from [A-Za-z0-9._-]; paths relative and inside
 * the manifest's directory; kind/extension/ABI must agree ("ptx" + ".ptx" + "cuda-ptx-v1",
 * "shared_object" + ".so" + "rvllm-cuda-so-v*"); every artifact's size and SHA-256 is
 * re-checked; the manifest's own digest, revision and arch must equal the caller's trust pins
 * (or the RVLLM_KERNEL_MANIFEST_SHA256 / RVLLM_RELEASE_REVISION / RVLLM_KERNEL_ARCH environment
 * variables when a pin is NULL).  A missing artifact, symbol or pin is a hard error: there is
 * no fallback path.
 *
 * All functions return 0 or a negative RVLLM_E_* code (rvllm_b200.h); rvllm_b200_last_error()
 * carries the reason.
 */
#ifndef RVLLM_B200_MANIFEST_H
#define RVLLM_B200_MANIFEST_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rvllm_manifest rvllm_manifest;   /* a verified manifest with its artifacts' bytes */
typedef struct rvllm_module rvllm_module;       /* a PTX module loaded into the current context */

/* lowercase hex SHA-256 of a buffer; out must hold 65 bytes */
int rvllm_sha256_hex(const void* data, size_t len, char* out);

int rvllm_manifest_load_and_verify(rvllm_manifest** out, const char* manifest_path, const char* trusted_sha256,
                                   const char* trusted_revision, const char* trusted_arch);
void rvllm_manifest_free(rvllm_manifest* m);
const char* rvllm_manifest_arch(const rvllm_manifest* m);
const char* rvllm_manifest_revision(const rvllm_manifest* m);
int rvllm_manifest_entry_count(const rvllm_manifest* m);
/* Verified bytes of an artifact (owned by the manifest object).  kind: 0 ptx, 1 shared_object. */
int rvllm_manifest_artifact(const rvllm_manifest* m, const char* name, const void** bytes, uint64_t* len,
                            int* kind, const char** abi);

/* cuModuleLoadData of a verified PTX artifact (text, NUL-terminated here; an interior NUL is an
 * error as in module.rs:280-289) into the current CUDA context. */
int rvllm_module_load_ptx(rvllm_module** out, const rvllm_manifest* m, const char* name);
void rvllm_module_unload(rvllm_module* mod);
int rvllm_module_get_function(rvllm_module* mod, const char* symbol, void** function_out);
/* cuLaunchKernel with the launch_raw checks: no zero or oversized dimension, <= 1024 threads,
 * dynamic shared memory above 48 KiB raised through the function attribute first. */
int rvllm_launch_raw(void* function, uint32_t grid_x, uint32_t grid_y, uint32_t grid_z, uint32_t block_x,
                     uint32_t block_y, uint32_t block_z, uint32_t dynamic_smem_bytes, void* stream, void** args);
/* dlopen of a verified shared-object artifact from a sealed in-memory copy
 * (v3/crates/rvllm-cutlass/src/lib_so.rs:39-126); returns the dl handle. */
int rvllm_manifest_dlopen(const rvllm_manifest* m, const char* name, void** handle_out);

#ifdef __cplusplus
}
#endif
#endif /* RVLLM_B200_MANIFEST_H */
