// Host-side helpers shared by the C-ABI translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

// Records a thread-local error message (printf-style) and returns `code`.
int rv_fail(int code, const char* fmt, ...);
// Checks the launch that was just enqueued; returns 0 or RVLLM_E_LAUNCH with the reason recorded.
int rv_launched(const char* what);
inline bool rv_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline uint32_t rv_umin(uint32_t a, uint32_t b) { return a < b ? a : b; }
inline uint32_t rv_umax(uint32_t a, uint32_t b) { return a > b ? a : b; }

// Whether launches carry the programmatic-stream-serialization attribute (on by default).
bool rv_pdl_enabled();
void rv_set_pdl(bool on);

// Launch with optional cluster dimensions and, when enabled, programmatic dependent launch.
template <typename... KArgs, typename... Args>
inline cudaError_t rv_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             dim3 cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x;
        attr[n].val.clusterDim.y = cluster.y;
        attr[n].val.clusterDim.z = cluster.z;
        n++;
    }
    if (rv_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
