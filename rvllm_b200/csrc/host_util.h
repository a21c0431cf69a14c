// Host-side helpers shared by the C-ABI translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

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

// "Done once" bookkeeping per device ordinal.  cudaFuncSetAttribute (and cudaGetSymbolAddress) apply to
// the device that is current, not to the process: a flag per kernel instantiation would leave the second
// GPU of a process at the 48 KiB default.  One instance per kernel instantiation; `first(dev)` is true
// exactly once per ordinal until `forget(dev)`, and the caller holds the lock while it does the set-up.
class RvDeviceOnce {
  public:
    static constexpr int MAX_DEVICES = 128;
    // Runs `setup()` (returning 0 on success) the first time device `dev` is seen; later calls return 0
    // without calling it.  A failed set-up is not remembered, so the next launch tries again.
    template <typename F> int run(int dev, F&& setup) {
        if (dev < 0 || dev >= MAX_DEVICES) return setup();  // out of the table: set up every time
        std::lock_guard<std::mutex> lock(mu_);
        const uint64_t bit = 1ull << (dev & 63);
        if (done_[dev >> 6] & bit) return 0;
        const int rc = setup();
        if (rc == 0) done_[dev >> 6] |= bit;
        return rc;
    }
    bool seen(int dev) {
        if (dev < 0 || dev >= MAX_DEVICES) return false;
        std::lock_guard<std::mutex> lock(mu_);
        return (done_[dev >> 6] >> (dev & 63)) & 1u;
    }

  private:
    std::mutex mu_;
    uint64_t done_[MAX_DEVICES / 64] = {0, 0};
};

// Ordinal of the current device, or -1.
inline int rv_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return dev;
}

// Raises a kernel's dynamic shared-memory limit on the current device, once per (instantiation, device).
template <typename K> inline int rv_allow_smem(RvDeviceOnce& once, K kernel, int bytes) {
    return once.run(rv_current_device(), [&]() -> int {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
            cudaGetLastError();
            return -1;
        }
        return 0;
    });
}
